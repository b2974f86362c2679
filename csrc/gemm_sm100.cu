// Persistent warp-specialised GEMM for sm_100a:  C[b] = alpha * A[b] x B[b]^T + beta * Cin[b].
//
//   TMA (128-byte swizzle) -> 4-stage shared-memory ring -> tcgen05.mma (128x256x16, fp32
//   accumulators in tensor memory, two accumulator buffers) -> tcgen05.ld epilogue that
//   overlaps the next tile's main loop.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2-5 = epilogue (one TMEM lane quarter each).
// Operands are 16-bit (bf16 or fp16).  Each may be K-major (row = M/N index, K contiguous)
// or MN-major (row = K index, M/N contiguous), so forward, data-gradient and weight-gradient
// products run without explicit transposes.  A batch dimension (same-shape matrices with a
// fixed stride) serves the batched Newton-Schulz of Muon.
// The epilogue computes alpha*acc + beta*Cin with Cin of the output type: residual adds,
// gradient accumulation and the Newton-Schulz polynomials are all fused here.
#include <cuda.h>
#include <string.h>

#include "tc.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_STAGE = BM * BK * 2, B_STAGE = BN * BK * 2;
constexpr int EPI_PITCH = 144;                       // bytes per staged row: 64 bf16 + 16 (bank spread)
constexpr int EPI_WARP_BYTES = 32 * EPI_PITCH;       // one 32x64 bf16 chunk per epilogue warp
constexpr int SMEM_BYTES = STAGES * (A_STAGE + B_STAGE) + 1024 /*align*/ + 256 /*barriers*/ + 4 * EPI_WARP_BYTES;
constexpr int GROUP_M = 8;

struct GemmParams {
    int M, N, K, batch;
    int a_mn, b_mn;            // operand majors
    int a_fmt, b_fmt;          // 0 fp16, 1 bf16
    int out_type;              // 0 fp16, 1 bf16, 2 fp32
    float alpha, beta;
    void* C;
    const void* Cin;           // may be null (beta ignored) or alias C
    long long ldc, c_batch_stride;
    long long ldcin, cin_batch_stride;
    int* status;
    int split_k;               // > 1: each tile's K range is cut into split_k parts, fp32 atomic accumulation
};

// Optional coupling of the GEMM to a collective over NVLink peer memory (tensor parallelism with
// sequence parallelism):
//   * all-gather side: the gathered operand sits in a local staging buffer that the peers fill
//     shard by shard; the TMA producer waits (bounded) for a shard's ready flag before it loads
//     the first tile that touches it, and visits its own shard first.  Shards are row ranges
//     of A (ag_dim 0) or K ranges of both operands (ag_dim 1, the weight-gradient product);
//   * reduce-scatter side: the epilogue stores each bf16 output tile into the slab that the
//     tile's owner rank keeps for this source rank (plain peer stores), then adds one arrival
//     per epilogue warp to the owner's counter; the owner's reduce kernel sums the slabs.
struct GemmComm {
    const int* ag_flags;
    int ag_epoch, ag_rows, ag_dim;
    int rot;                       // visiting order starts at this M tile (ag_dim 0 / rs) or k-block (ag_dim 1)
    void* rs_out[8];
    int* rs_cnt[8];
    int rs_rows;
    unsigned long long limit_ns;
};

__device__ __forceinline__ int ld_relaxed_sys_i32(const int* p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Bounded wait for flag >= epoch: relaxed polls with back-off, one acquire fence at the end, and a
// proxy fence so that the TMA (async proxy) reads what the peer's stores wrote.
__device__ __forceinline__ bool wait_shard(const int* flag, int epoch, unsigned long long limit_ns,
                                           volatile int* abort_flag) {
    if (ld_relaxed_sys_i32(flag) < epoch) {
        const uint64_t t0 = global_timer_ns();
        unsigned sleep_ns = 64;
        while (ld_relaxed_sys_i32(flag) < epoch) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > limit_ns) {
                *abort_flag = 1;
                return false;
            }
            __nanosleep(sleep_ns);
            if (sleep_ns < 1024) sleep_ns <<= 1;
        }
    }
    __threadfence_system();
    asm volatile("fence.proxy.async;" ::: "memory");
    return true;
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& b, int& tm, int& tn) {
    const int per_batch = tiles_m * tiles_n;
    b = tile / per_batch;
    int t = tile % per_batch;
    const int group = GROUP_M * tiles_n;
    const int g = t / group;
    const int first_m = g * GROUP_M;
    const int gm = min(GROUP_M, tiles_m - first_m);
    t -= g * group;
    tm = first_m + t % gm;
    tn = t / gm;
}

template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* dst, const OutT* cin, const uint32_t* acc, float alpha, float beta,
                                            int ncols);

template <>
__device__ __forceinline__ void store_row32<float>(float* dst, const float* cin, const uint32_t* acc, float alpha,
                                                   float beta, int ncols) {
    // ncols < 0 encodes "32 columns, 16-byte aligned": vector path
    if (ncols < 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float4 v;
            v.x = alpha * __uint_as_float(acc[4 * j]);
            v.y = alpha * __uint_as_float(acc[4 * j + 1]);
            v.z = alpha * __uint_as_float(acc[4 * j + 2]);
            v.w = alpha * __uint_as_float(acc[4 * j + 3]);
            if (cin) {
                const float4 c = *reinterpret_cast<const float4*>(cin + 4 * j);
                v.x += beta * c.x; v.y += beta * c.y; v.z += beta * c.z; v.w += beta * c.w;
            }
            *reinterpret_cast<float4*>(dst + 4 * j) = v;
        }
    } else {
        for (int j = 0; j < ncols; ++j) {
            float v = alpha * __uint_as_float(acc[j]);
            if (cin) v += beta * cin[j];
            dst[j] = v;
        }
    }
}

template <typename T>
__device__ __forceinline__ float h2f(T x);
template <> __device__ __forceinline__ float h2f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float h2f<__half>(__half x) { return __half2float(x); }
template <typename T>
__device__ __forceinline__ T f2h(float x);
template <> __device__ __forceinline__ __nv_bfloat16 f2h<__nv_bfloat16>(float x) { return __float2bfloat16(x); }
template <> __device__ __forceinline__ __half f2h<__half>(float x) { return __float2half(x); }

template <typename T>
__device__ __forceinline__ void store_row32_16(T* dst, const T* cin, const uint32_t* acc, float alpha, float beta,
                                               int ncols, bool vec_ok) {
    if (ncols == 32 && vec_ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = alpha * __uint_as_float(acc[8 * j + i]);
            if (cin) {
                const uint4 raw = *reinterpret_cast<const uint4*>(cin + 8 * j);
                const T* c = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += beta * h2f<T>(c[i]);
            }
            uint4 o;
            T* op = reinterpret_cast<T*>(&o);
#pragma unroll
            for (int i = 0; i < 8; ++i) op[i] = f2h<T>(v[i]);
            *reinterpret_cast<uint4*>(dst + 8 * j) = o;
        }
    } else {
        for (int j = 0; j < ncols; ++j) {
            float v = alpha * __uint_as_float(acc[j]);
            if (cin) v += beta * h2f<T>(cin[j]);
            dst[j] = f2h<T>(v);
        }
    }
}

template <bool COMM>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmParams p, const GemmComm cm) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE + B_STAGE));
    uint64_t* full = bars;                 // [STAGES]  TMA -> MMA
    uint64_t* empty = bars + STAGES;       // [STAGES]  MMA -> TMA
    uint64_t* acc_full = bars + 2 * STAGES;      // [2] MMA -> epilogue
    uint64_t* acc_empty = bars + 2 * STAGES + 2; // [2] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n * p.batch * p.split_k;   // work items (tile, k-part)
    const int kblocks_total = (p.K + BK - 1) / BK;
    const int kb_per = (kblocks_total + p.split_k - 1) / p.split_k;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(&acc_full[b], 1);
            tc::mbar_init(&acc_empty[b], 4);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, 512);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // every pipeline wait sits behind the producer's wait for a peer's shard when the kernel is coupled to an
    // all-gather: give them that wait's limit on top of their own
    const uint64_t wait_ns = (COMM && cm.ag_flags) ? cm.limit_ns + 2000000000ull : 2000000000ull;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tc::prefetch_tmap(&tmA);
            tc::prefetch_tmap(&tmB);
            int stage = 0;
            uint32_t phase = 0;
            int issued = 0;
            bool ok = true;
            unsigned ready_mask = 0;       // shards already seen ready
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int b, tm, tn;
                tile_coords(tile / p.split_k, tiles_m, tiles_n, b, tm, tn);
                if (COMM && cm.ag_dim == 0) {
                    tm += cm.rot;
                    if (tm >= tiles_m) tm -= tiles_m;
                    if (cm.ag_flags) {
                        const int s0 = (tm * BM) / cm.ag_rows, s1 = (min(tm * BM + BM, p.M) - 1) / cm.ag_rows;
                        for (int sh = s0; sh <= s1 && ok; ++sh) {
                            if (ready_mask >> sh & 1) continue;
                            if (!wait_shard(cm.ag_flags + sh, cm.ag_epoch, cm.limit_ns, abort_flag)) {
                                atomicMax(p.status, (int)KB_TIMEOUT_PEER);
                                ok = false;
                            }
                            ready_mask |= 1u << sh;
                        }
                        if (!ok) break;
                    }
                }
                const int kb0 = (tile % p.split_k) * kb_per, kb1 = min(kblocks_total, kb0 + kb_per);
                for (int kbi = kb0; kbi < kb1; ++kbi) {
                    int kb = kbi;
                    if (COMM && cm.ag_dim == 1) {
                        kb += cm.rot;
                        if (kb >= kblocks_total) kb -= kblocks_total;
                        const int sh = (kb * BK) / cm.ag_rows;
                        if (cm.ag_flags && !(ready_mask >> sh & 1)) {
                            if (!wait_shard(cm.ag_flags + sh, cm.ag_epoch, cm.limit_ns, abort_flag)) {
                                atomicMax(p.status, (int)KB_TIMEOUT_PEER);
                                ok = false;
                                break;
                            }
                            ready_mask |= 1u << sh;
                        }
                    }
                    if (!tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag, wait_ns)) {
                        atomicMax(p.status, (int)KB_TIMEOUT_TMA);
                        ok = false;
                        break;
                    }
                    tc::mbar_expect_tx(&full[stage], A_STAGE + B_STAGE);
                    uint8_t* a_dst = sA + stage * A_STAGE;
                    uint8_t* b_dst = sB + stage * B_STAGE;
                    if (p.a_mn) {
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c)
                            tc::tma_load_3d(a_dst + c * (64 * BK * 2), &tmA, &full[stage], tm * BM + c * 64, kb * BK, b);
                    } else {
                        tc::tma_load_3d(a_dst, &tmA, &full[stage], kb * BK, tm * BM, b);
                    }
                    if (p.b_mn) {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c)
                            tc::tma_load_3d(b_dst + c * (64 * BK * 2), &tmB, &full[stage], tn * BN + c * 64, kb * BK, b);
                    } else {
                        tc::tma_load_3d(b_dst, &tmB, &full[stage], kb * BK, tn * BN, b);
                    }
                    ++issued;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // let copies already in flight land before the block can exit
                const int inflight = issued < STAGES ? issued : STAGES;
                for (int i = 0; i < inflight; ++i) {
                    int s = stage - 1 - i;
                    uint32_t ph = phase;
                    if (s < 0) { s += STAGES; ph ^= 1; }
                    const uint64_t t0 = global_timer_ns();
                    while (!tc::mbar_try_wait(&full[s], ph) && global_timer_ns() - t0 < 2000000ull) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = tc::instr_desc_f16(BM, BN, p.a_fmt, p.b_fmt, p.a_mn, p.b_mn);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                const int buf = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!tc::mbar_wait(&acc_empty[buf], acc_phase ^ 1, abort_flag, wait_ns)) {
                    atomicMax(p.status, (int)KB_TIMEOUT_MMA);
                    ok = false;
                    break;
                }
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const int kb0 = (tile % p.split_k) * kb_per, kb1 = min(kblocks_total, kb0 + kb_per);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!tc::mbar_wait(&full[stage], phase, abort_flag, wait_ns)) {
                        atomicMax(p.status, (int)KB_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    tc::tc_fence_after();
                    const uint32_t a_addr = smem_u32(sA + stage * A_STAGE);
                    const uint32_t b_addr = smem_u32(sB + stage * B_STAGE);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = p.a_mn ? tc::smem_desc_sw128(a_addr + k * 2048, 64 * BK * 2, 1024)
                                                   : tc::smem_desc_sw128(a_addr + k * 32, 16, 1024);
                        const uint64_t bd = p.b_mn ? tc::smem_desc_sw128(b_addr + k * 2048, 64 * BK * 2, 1024)
                                                   : tc::smem_desc_sw128(b_addr + k * 32, 16, 1024);
                        tc::mma_f16(d_tmem, ad, bd, idesc, ((kb - kb0) | k) != 0);
                    }
                    tc::tc_commit(&empty[stage]);   // stage reusable once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc::tc_commit(&acc_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;   // TMEM lanes [32*quarter, 32*quarter+32)
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
            int b, tm, tn;
            tile_coords(tile / p.split_k, tiles_m, tiles_n, b, tm, tn);
            if (COMM && cm.ag_dim == 0) {
                tm += cm.rot;
                if (tm >= tiles_m) tm -= tiles_m;
            }
            const bool has_k = (tile % p.split_k) * kb_per < kblocks_total;
            const int buf = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            if (!tc::mbar_wait(&acc_full[buf], acc_phase, abort_flag, wait_ns)) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                ok = false;
                break;
            }
            tc::tc_fence_after();
            const int row = tm * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
            if (COMM && cm.rs_rows > 0) {
                // Reduce-scatter store.  Peer stores should be wide and contiguous (a 16-byte store
                // per lane to 32 different rows becomes 32 small NVLink writes), so each 32x64 chunk
                // is transposed through shared memory and leaves as 128-byte row segments.
                uint8_t* stg = smem + STAGES * (A_STAGE + B_STAGE) + 256 + (warp - 2) * EPI_WARP_BYTES;
                const int owner = (tm * BM) / cm.rs_rows;
                __nv_bfloat16* obase = reinterpret_cast<__nv_bfloat16*>(cm.rs_out[owner]) +
                                       (long long)(tm * BM + quarter * 32 - owner * cm.rs_rows) * p.ldc;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    uint32_t acc[64];
                    tc::tmem_ld32(taddr + c0, acc);
                    tc::tmem_ld32(taddr + c0 + 32, acc + 32);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint4 o;
                        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            op[i] = __floats2bfloat162_rn(p.alpha * __uint_as_float(acc[8 * j + 2 * i]),
                                                          p.alpha * __uint_as_float(acc[8 * j + 2 * i + 1]));
                        *reinterpret_cast<uint4*>(stg + lane * EPI_PITCH + j * 16) = o;
                    }
                    __syncwarp();
                    const int seg = lane & 7, col = tn * BN + c0 + seg * 8;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = i * 4 + (lane >> 3);
                        const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * EPI_PITCH + seg * 16);
                        if (tm * BM + quarter * 32 + rr < p.M && col < p.N)
                            *reinterpret_cast<uint4*>(obase + (long long)rr * p.ldc + col) = v;
                    }
                    __syncwarp();
                }
            } else
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t acc[32];
                tc::tmem_ld32(taddr + c0, acc);
                tc::tmem_ld_wait();
                const int col = tn * BN + c0;
                const int ncols = min(32, p.N - col);
                if (p.split_k > 1) {
                    const int row0 = tm * BM + quarter * 32;
                    if (has_k && row0 < p.M && ncols > 0) {
                        if (ncols == 32 && ((p.ldc | col) & 3) == 0) {
                            // A lane that adds its own row issues 32 scattered atomics per instruction.  The
                            // 32x32 chunk is transposed through shared memory instead, so one instruction adds
                            // four 128-byte row segments with 16-byte vector atomics.
                            float* stg = reinterpret_cast<float*>(smem + STAGES * (A_STAGE + B_STAGE) + 256 +
                                                                  (warp - 2) * EPI_WARP_BYTES);
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *reinterpret_cast<float4*>(stg + lane * (EPI_PITCH / 4) + 4 * j) =
                                    make_float4(p.alpha * __uint_as_float(acc[4 * j]), p.alpha * __uint_as_float(acc[4 * j + 1]),
                                                p.alpha * __uint_as_float(acc[4 * j + 2]), p.alpha * __uint_as_float(acc[4 * j + 3]));
                            __syncwarp();
                            float* dst0 = reinterpret_cast<float*>(p.C) + (long long)b * p.c_batch_stride +
                                          (long long)row0 * p.ldc + col + (lane & 7) * 4;
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int rr = i * 4 + (lane >> 3);
                                if (row0 + rr < p.M) {
                                    const float4 v = *reinterpret_cast<const float4*>(stg + rr * (EPI_PITCH / 4) + (lane & 7) * 4);
                                    atomicAdd(reinterpret_cast<float4*>(dst0 + (long long)rr * p.ldc), v);
                                }
                            }
                            __syncwarp();
                        } else if (row < p.M) {
                            float* dst = reinterpret_cast<float*>(p.C) + (long long)b * p.c_batch_stride +
                                         (long long)row * p.ldc + col;
                            for (int j = 0; j < ncols; ++j) atomicAdd(dst + j, p.alpha * __uint_as_float(acc[j]));
                        }
                    }
                } else if (row < p.M && ncols > 0) {
                    const long long off = (long long)b * p.c_batch_stride + (long long)row * p.ldc + col;
                    const long long offin = (long long)b * p.cin_batch_stride + (long long)row * p.ldcin + col;
                    if (p.out_type == 2) {
                        float* dst = reinterpret_cast<float*>(p.C) + off;
                        const float* cin = p.Cin ? reinterpret_cast<const float*>(p.Cin) + offin : nullptr;
                        const bool vec = ((p.ldc | p.ldcin | col) & 3) == 0 && ncols == 32;
                        store_row32<float>(dst, cin, acc, p.alpha, p.beta, vec ? -1 : ncols);
                    } else {
                        const bool vec = ((p.ldc | p.ldcin | col) & 7) == 0;
                        if (p.out_type == 1) {
                            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
                            const __nv_bfloat16* cin =
                                p.Cin ? reinterpret_cast<const __nv_bfloat16*>(p.Cin) + offin : nullptr;
                            store_row32_16<__nv_bfloat16>(dst, cin, acc, p.alpha, p.beta, ncols, vec);
                        } else {
                            __half* dst = reinterpret_cast<__half*>(p.C) + off;
                            const __half* cin = p.Cin ? reinterpret_cast<const __half*>(p.Cin) + offin : nullptr;
                            store_row32_16<__half>(dst, cin, acc, p.alpha, p.beta, ncols, vec);
                        }
                    }
                }
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
            if (COMM && cm.rs_rows > 0) {
                // this warp's part of the tile has been stored to the owner: publish one arrival
                __threadfence_system();
                __syncwarp();
                if (lane == 0) {
                    int* cnt = cm.rs_cnt[(tm * BM) / cm.rs_rows];
                    asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(cnt) : "memory");
                }
            }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, 512);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// 16-bit matrix [rows, cols] (cols contiguous, leading dimension ld elements) x batch.
int make_tmap(CUtensorMap* m, const void* base, int fmt, long long cols, long long rows, long long ld,
              long long batch, long long batch_stride, int box_cols, int box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return 100;
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch > 1 ? batch_stride : rows * ld) * 2};
    cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(m, fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                           const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 200 + (int)r;
}

static int launch_gemm(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, int batch,
                       long long lda, long long ldb, long long ldc, long long ldcin, long long a_bs, long long b_bs,
                       long long c_bs, long long cin_bs, int a_mn, int b_mn, int a_fmt, int b_fmt, int out_type,
                       float alpha, float beta, int* status, int max_ctas, int split_k, const GemmComm* cm,
                       cudaStream_t st) {
    if (split_k < 1) split_k = 1;
    if (split_k > 1 && out_type != 2) return 5;
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 5;
    if ((lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return 6;
    if (batch > 1 && ((a_bs & 7) || (b_bs & 7))) return 6;
    static bool attr_flags[64] = {};
    bool* attr_set_p = kb_device_flag(attr_flags);
    if (!attr_set_p) return 7;
    if (!*attr_set_p) {
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 SMEM_BYTES) != cudaSuccess)
            return 7;
        *attr_set_p = true;
    }
    CUtensorMap tmA, tmB;
    int r;
    if (a_mn) r = make_tmap(&tmA, A, a_fmt, M, K, lda, batch, a_bs, 64, BK);
    else r = make_tmap(&tmA, A, a_fmt, K, M, lda, batch, a_bs, BK, BM);
    if (r) return r;
    if (b_mn) r = make_tmap(&tmB, B, b_fmt, N, K, ldb, batch, b_bs, 64, BK);
    else r = make_tmap(&tmB, B, b_fmt, K, N, ldb, batch, b_bs, BK, BN);
    if (r) return r;
    GemmParams p;
    p.M = M; p.N = N; p.K = K; p.batch = batch;
    p.a_mn = a_mn; p.b_mn = b_mn; p.a_fmt = a_fmt; p.b_fmt = b_fmt; p.out_type = out_type;
    p.alpha = alpha; p.beta = beta; p.C = C; p.Cin = Cin;
    p.ldc = ldc; p.c_batch_stride = c_bs; p.ldcin = ldcin; p.cin_batch_stride = cin_bs;
    p.status = status;
    p.split_k = split_k;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * batch * split_k;
    const int grid = tiles < sms ? tiles : sms;
    if (cm) {
        gemm_tcgen05_kernel<true><<<grid, 192, SMEM_BYTES, st>>>(tmA, tmB, p, *cm);
    } else {
        GemmComm none;
        memset(&none, 0, sizeof(none));
        gemm_tcgen05_kernel<false><<<grid, 192, SMEM_BYTES, st>>>(tmA, tmB, p, none);
    }
    return kb_launch_status();
}

}  // namespace

// C[b][M,N] = alpha * op(A[b]) * op(B[b])^T + beta * Cin[b].
//   a_mn = 0: A is [M,K] (lda = row stride);  a_mn = 1: A is stored [K,M].
//   b_mn = 0: B is [N,K];                      b_mn = 1: B is stored [K,N].
//   fmt: 0 fp16, 1 bf16.  out_type: 0 fp16, 1 bf16, 2 fp32.  status: device int, set on a wait timeout.
// Requirements: 16-byte aligned bases, lda/ldb multiples of 8 elements.
KB_API int kb_gemm(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, int batch,
                   long long lda, long long ldb, long long ldc, long long ldcin, long long a_bs, long long b_bs,
                   long long c_bs, long long cin_bs, int a_mn, int b_mn, int a_fmt, int b_fmt, int out_type,
                   float alpha, float beta, int* status, int max_ctas, int split_k, cudaStream_t st) {
    return launch_gemm(A, B, C, Cin, M, N, K, batch, lda, ldb, ldc, ldcin, a_bs, b_bs, c_bs, cin_bs, a_mn, b_mn,
                       a_fmt, b_fmt, out_type, alpha, beta, status, max_ctas, split_k, nullptr, st);
}

// All-gather -> GEMM.  One operand is a local staging buffer filled shard by shard by the peers
// (kb_ag_push): `ag_dim` 0 = A's rows come in `world` shards of `ag_rows` rows, 1 = the K
// dimension of both operands does (A local and complete, B staged).  ag_flags[s] >= ag_epoch marks
// shard s as landed; `own` is this rank's shard, visited first.  bf16 in, bf16 out;
// C = alpha*A*B^T + beta*Cin with Cin (nullable) laid out like C.
KB_API int kb_gemm_ag(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, long long lda,
                      long long ldb, long long ldc, int a_mn, int b_mn, float alpha, float beta,
                      const int* ag_flags, int ag_epoch,
                      int ag_rows, int ag_dim, int own, double limit_s, int* status, cudaStream_t st) {
    if (!ag_flags || ag_rows <= 0 || own < 0 || own > 7) return 5;
    if (ag_dim == 0 ? (ag_rows % BM) != 0 : (ag_rows % BK) != 0) return 5;
    if ((ag_dim == 0 ? M : K) > 8 * (long long)ag_rows) return 5;
    GemmComm cm;
    memset(&cm, 0, sizeof(cm));
    cm.ag_flags = ag_flags; cm.ag_epoch = ag_epoch; cm.ag_rows = ag_rows; cm.ag_dim = ag_dim;
    cm.rot = own * (ag_rows / (ag_dim == 0 ? BM : BK));
    cm.limit_ns = (unsigned long long)(limit_s * 1e9);
    return launch_gemm(A, B, C, Cin, M, N, K, 1, lda, ldb, ldc, ldc, 0, 0, 0, 0, a_mn, b_mn, 1, 1, 1, alpha, beta,
                       status, 0, 1, &cm, st);
}

// GEMM -> reduce-scatter, producer half.  Rows [o*rs_rows, (o+1)*rs_rows) of the bf16 product
// belong to rank o: they are stored to rs_out[o] (that rank's slab for this source, row stride
// ldc) while the other tiles are still being computed, and every epilogue warp adds one arrival
// to rs_cnt[o] when its quarter tile is out.  kb_gemm_rs_arrivals gives the arrivals per owner;
// kb_rs_reduce is the consumer half.  Tiles for rank+1 are computed first, the own ones last.
KB_API int kb_gemm_rs(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                      long long ldc, int a_mn, int b_mn, float alpha, void* const* rs_out, int* const* rs_cnt,
                      int world, int rank, int rs_rows, int* status, cudaStream_t st) {
    if (world < 1 || world > 8 || rs_rows <= 0 || (rs_rows % BM) != 0 || M != world * rs_rows) return 5;
    if ((N & 7) || (ldc & 7)) return 6;
    GemmComm cm;
    memset(&cm, 0, sizeof(cm));
    for (int i = 0; i < world; ++i) {
        cm.rs_out[i] = rs_out[i];
        cm.rs_cnt[i] = rs_cnt[i];
    }
    cm.rs_rows = rs_rows;
    cm.rot = ((rank + 1) % world) * (rs_rows / BM);
    return launch_gemm(A, B, rs_out[rank], nullptr, M, N, K, 1, lda, ldb, ldc, 0, 0, 0, 0, 0, a_mn, b_mn, 1, 1, 1,
                       alpha, 0.f, status, 0, 1, &cm, st);
}
KB_API int kb_gemm_rs_arrivals(int N, int rs_rows) { return (rs_rows / BM) * ((N + BN - 1) / BN) * 4; }
