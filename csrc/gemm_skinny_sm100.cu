// Skinny GEMM for decode-size activations (M <= 128 rows): C = alpha * A x B^T + beta * Cin, bf16,
// both operands K-major.  Such a product is a weight stream: the N x K weight must cross HBM once,
// and an M x N output has far too few 128 x 256 tiles to put every SM on that stream.  The K range
// of each output tile is therefore split over the CTAs of a thread-block cluster (up to 8), and the
// partial sums meet in distributed shared memory instead of in global memory:
//
//   TMA (128-byte swizzle) -> shared-memory ring -> tcgen05.mma (128 x BN x 16) over this CTA's
//   K range -> the fp32 partial tile goes from tensor memory to this CTA's shared memory (the ring,
//   now idle) -> cluster barrier -> every CTA sums its share of the rows over all CTAs of the
//   cluster with `ld.shared::cluster`, applies alpha / beta * Cin and stores bf16 -> cluster barrier.
//
// One launch, no fp32 workspace, no atomics, no finishing kernel (the split-K path of the general
// kernel needs all three).  BN is 256 or 128 and the cluster size is chosen per shape so that
// tiles x cluster size comes close to the number of SMs.
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2-5 =
// tensor memory -> shared memory, then the cluster reduction.  All waits are bounded; a CTA whose
// wait ran out still takes part in both cluster barriers, so its peers are never left waiting.
#include <cuda.h>
#include <string.h>

#include "tc.cuh"

namespace {

constexpr int BM = 128, BK = 64;
// AM: rows of A that get a slot in the ring (64 when M <= 64, else 128).  The MMA always reads a
// 128-row operand tile; with AM = 64 its upper half is whatever follows the slot in shared memory,
// and the products of those rows land in accumulator rows that nobody reads.  A smaller A slot
// means more stages, i.e. more weight bytes in flight per SM, which is what bounds this kernel.
template <int BN, int AM> struct Cfg {
    static constexpr int A_STAGE = AM * BK * 2;
    static constexpr int B_STAGE = BN * BK * 2;
    static constexpr int STAGES = (200 * 1024) / (A_STAGE + B_STAGE);
    static constexpr int RING = STAGES * (A_STAGE + B_STAGE);
    static constexpr int PITCH = BN * 4 + 16;            // bytes per staged fp32 row (+16: conflict-free row-per-lane stores)
    static constexpr int SMEM = RING + BM * BK * 2 /* slack: the 128-row read of the last A slot */ + 1024 + 256;
    static_assert(AM * PITCH <= RING, "the partial tile is staged in the ring");
    static_assert(SMEM <= 227 * 1024, "shared memory");
};

struct SkinnyParams {
    int M, N, K;
    float alpha, beta;
    __nv_bfloat16* C;
    const __nv_bfloat16* Cin;      // may be null, may alias C
    long long ldc, ldcin;
    int* status;
    // all-reduce over tensor-parallel ranks fused into the epilogue (AR kernels only): every rank's summed
    // tile rows are pushed into slot [parity][rank] of every rank's receive buffer, the last CTA raises this
    // rank's flag on every peer, and every CTA then sums its rows over the ranks' slots (+ Cin) into C
    void* ar_recv[8];              // peer receive buffers: [2 parities][world][ar_slot_elems] bf16
    void* ar_flags[8];             // peer flag arrays: int [2 parities][8]
    int ar_world, ar_rank;
    long long ar_slot_elems;
    int* ar_epoch;                 // device-side call counter (graph replay needs no host update)
    unsigned* ar_counters;         // two zero-initialised counters: last-CTA elections
    unsigned long long ar_limit_ns;
    int b_const;                   // B is never written while this process launches kernels (a served weight): its first
                                   // ring-full of tiles may be fetched before the kernels ahead on the stream have finished
    int b_packed;                  // B is stored tile-major: [N / 128][K / 64][128 rows][64 columns], 16 KB contiguous per tile
    int a_rows;                    // rows of A that TMA fetches per K block (M rounded up to 8): the rest of the 128-row
                                   // operand tile is left as it is - its products land in rows that nobody reads
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mapa(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t cluster_addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(cluster_addr));
    return v;
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

__device__ __forceinline__ void st_release_sys_i32(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys_i32(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// bounded wait for flag >= epoch (false on timeout)
__device__ __forceinline__ bool wait_flag_sk(const int* flag, int epoch, unsigned long long limit_ns) {
    if (ld_acquire_sys_i32(flag) >= epoch) return true;
    const uint64_t t0 = global_timer_ns();
    unsigned sleep_ns = 64;
    while (ld_acquire_sys_i32(flag) < epoch) {
        if (global_timer_ns() - t0 > limit_ns) return false;
        __nanosleep(sleep_ns);
        if (sleep_ns < 1024) sleep_ns <<= 1;
    }
    return true;
}

template <int BN, int AM, bool AR>
__global__ void __launch_bounds__(192, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const SkinnyParams p) {
    using C_ = Cfg<BN, AM>;
    constexpr int STAGES = C_::STAGES, A_STAGE = C_::A_STAGE, B_STAGE = C_::B_STAGE, PITCH = C_::PITCH;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // B slots first, A slots behind them: the 128-row read of an A slot may run into the next slot or
    // into the slack after the last one, never outside the allocation
    uint8_t* sB = smem;
    uint8_t* sA = smem + STAGES * B_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C_::RING + BM * BK * 2);
    uint64_t* full = bars;                 // [STAGES] TMA -> MMA
    uint64_t* empty = bars + STAGES;       // [STAGES] MMA -> TMA
    uint64_t* acc_full = bars + 2 * STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = (int)cluster_nctarank(), r = (int)cluster_ctarank();
    const int tn = blockIdx.y;
    const int kblocks_total = (p.K + BK - 1) / BK;
    const int kb_per = (kblocks_total + S - 1) / S;
    const int kb0 = min(kblocks_total, r * kb_per), kb1 = min(kblocks_total, kb0 + kb_per);

    auto load_b = [&](int kb, int stage) {                       // announces the bytes of both operands
        tc::mbar_expect_tx(&full[stage], p.a_rows * BK * 2 + B_STAGE);
        if (p.b_packed) tma_load_4d(sB + stage * B_STAGE, &tmB, &full[stage], 0, 0, kb, tn * (BN / 128));
        else tc::tma_load_3d(sB + stage * B_STAGE, &tmB, &full[stage], kb * BK, tn * BN, 0);
    };
    auto load_a = [&](int kb, int stage) { tc::tma_load_3d(sA + stage * A_STAGE, &tmA, &full[stage], kb * BK, 0, 0); };
    auto load_stage = [&](int kb, int stage) {
        load_b(kb, stage);
        load_a(kb, stage);
    };
    const int first = min(STAGES, kb1 - kb0);                    // loads that need no free-slot wait
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        tc::mbar_init(acc_full, 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
        // the first ring-full of loads goes out before the block-wide barrier below (which waits for
        // the tensor-memory allocation): their latency overlaps the rest of the prologue
        tc::prefetch_tmap(&tmA);
        tc::prefetch_tmap(&tmB);
        // Launched as a dependent of the kernel before it, this CTA may be running while that kernel still
        // is: the weight tiles of the first ring-full (up to 200 KB per CTA, most of a 3B projection over
        // the grid) stream in meanwhile; the activations are fetched after the wait.
        if (p.b_const) {
            for (int i = 0; i < first; ++i) load_b(kb0 + i, i);
            kb_dep_wait();
            for (int i = 0; i < first; ++i) load_a(kb0 + i, i);
        } else {
            kb_dep_wait();
            for (int i = 0; i < first; ++i) load_stage(kb0 + i, i);
        }
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, BN);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    kb_dep_wait();                       // every thread: returns at once after thread 0's wait above
    kb_dep_trigger();
    const uint32_t tmem_base = *tmem_slot;
    bool have_partial = kb1 > kb0;

    if (warp == 0) {
        if (lane == 0) {
            int stage = first == STAGES ? 0 : first;
            uint32_t phase = first == STAGES ? 1 : 0;
            for (int kb = kb0 + first; kb < kb1; ++kb) {
                if (!tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
                    atomicMax(p.status, (int)KB_TIMEOUT_TMA);
                    break;
                }
                load_stage(kb, stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && have_partial) {
            const uint32_t idesc = tc::instr_desc_f16(BM, BN, 1, 1, 0, 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!tc::mbar_wait(&full[stage], phase, abort_flag)) {
                    atomicMax(p.status, (int)KB_TIMEOUT_MMA);
                    ok = false;
                    break;
                }
                tc::tc_fence_after();
                const uint32_t a_addr = smem_u32(sA + stage * A_STAGE), b_addr = smem_u32(sB + stage * B_STAGE);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    tc::mma_f16(tmem_base, tc::smem_desc_sw128(a_addr + k * 32, 16, 1024),
                                tc::smem_desc_sw128(b_addr + k * 32, 16, 1024), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                tc::tc_commit(&empty[stage]);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok) tc::tc_commit(acc_full);
        }
    } else {
        // ---- tensor memory -> this CTA's shared memory (rows below M only), fp32, padded rows
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        if (have_partial) {
            if (!tc::mbar_wait(acc_full, 0, abort_flag)) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                have_partial = false;
            }
        }
        tc::tc_fence_after();
        if (quarter * 32 < p.M) {                                    // warp-uniform
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t acc[32];
                if (have_partial) {
                    tc::tmem_ld32(taddr + c0, acc);
                    tc::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[j] = 0u;
                }
                if (row < p.M) {
                    float4* dst = reinterpret_cast<float4*>(smem + (size_t)row * PITCH + c0 * 4);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        dst[j] = make_float4(__uint_as_float(acc[4 * j]), __uint_as_float(acc[4 * j + 1]),
                                             __uint_as_float(acc[4 * j + 2]), __uint_as_float(acc[4 * j + 3]));
                }
            }
        }
        tc::tc_fence_before();
    }
    // every CTA's partial tile is in its shared memory
    __syncthreads();
    cluster_sync_all();
    // ---- reduction over the cluster: this CTA owns rows r, r + S, ...; a thread takes 8 columns of a row
    constexpr int V8 = BN / 8;                                   // threads per row
    constexpr int ROWS_PER_PASS = 128 / V8;                      // 4 (BN 256) or 8 (BN 128)
    const int t = threadIdx.x - 64;
    const int c8 = t % V8, sub = t / V8;
    const int col = tn * BN + c8 * 8;
    const uint32_t sbase = smem_u32(smem);
    auto cluster_sum8 = [&](int row, float* acc) {
        const uint32_t off = sbase + (uint32_t)row * PITCH + (uint32_t)c8 * 32;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int q = 0; q < S; ++q) {
            const uint32_t a = mapa(off, (uint32_t)q);
            const float4 v0 = ld_dsmem_f4(a), v1 = ld_dsmem_f4(a + 16);
            acc[0] += v0.x; acc[1] += v0.y; acc[2] += v0.z; acc[3] += v0.w;
            acc[4] += v1.x; acc[5] += v1.y; acc[6] += v1.z; acc[7] += v1.w;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= p.alpha;
    };
    const bool vec_ok = ((p.ldc | p.ldcin) & 7) == 0 && col + 8 <= p.N;
    if (!AR) {
        if (warp >= 2) {
            for (int i = sub;; i += ROWS_PER_PASS) {
                const int row = r + i * S;
                if (row >= p.M) break;
                if (col >= p.N) continue;
                float o[8];
                cluster_sum8(row, o);
                __nv_bfloat16* dst = p.C + (long long)row * p.ldc + col;
                const __nv_bfloat16* cin = p.Cin ? p.Cin + (long long)row * p.ldcin + col : nullptr;
                if (vec_ok) {
                    if (cin) {
                        float ci[8];
                        unpack8(ld8(cin), ci);
#pragma unroll
                        for (int j = 0; j < 8; ++j) o[j] += p.beta * ci[j];
                    }
                    st8(dst, pack8(o));
                } else {
                    const int ncols = min(8, p.N - col);
                    for (int j = 0; j < ncols; ++j)
                        dst[j] = __float2bfloat16(o[j] + (cin ? p.beta * __bfloat162float(cin[j]) : 0.f));
                }
            }
        }
    } else {
        // ---- fused all-reduce (N is a multiple of 8 and C / Cin are dense [M, N]: checked by the launcher)
        __shared__ int s_last, s_ok;
        const int epoch = *reinterpret_cast<volatile int*>(p.ar_epoch) + 1;
        const int par = epoch & 1;
        const int W = p.ar_world;
        const long long my_slot = ((long long)par * W + p.ar_rank) * p.ar_slot_elems;
        if (threadIdx.x == 0) s_ok = 1;
        if (warp >= 2) {
            for (int i = sub;; i += ROWS_PER_PASS) {
                const int row = r + i * S;
                if (row >= p.M) break;
                if (col >= p.N) continue;
                float o[8];
                cluster_sum8(row, o);
                const bf16x8 v = pack8(o);
                const long long at = my_slot + (long long)row * p.N + col;
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    if (q < W) st8(reinterpret_cast<__nv_bfloat16*>(p.ar_recv[q]) + at, v);
            }
        }
        // this rank's flag goes up on every peer once all of its CTAs have pushed
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned total = gridDim.x * gridDim.y;
            const unsigned prev = atomicAdd(p.ar_counters, 1u);
            s_last = prev == total - 1;
            if (s_last) *p.ar_counters = 0;
        }
        __syncthreads();
        if (s_last && threadIdx.x < W) {
            __threadfence_system();
            st_release_sys_i32(reinterpret_cast<int*>(p.ar_flags[threadIdx.x]) + par * 8 + p.ar_rank, epoch);
        }
        if (threadIdx.x < W) {
            if (!wait_flag_sk(reinterpret_cast<const int*>(p.ar_flags[p.ar_rank]) + par * 8 + threadIdx.x, epoch, p.ar_limit_ns)) {
                atomicMax(p.status, (int)KB_TIMEOUT_PEER);
                s_ok = 0;
            }
        }
        __syncthreads();
        if (warp >= 2 && s_ok) {
            const __nv_bfloat16* mine = reinterpret_cast<const __nv_bfloat16*>(p.ar_recv[p.ar_rank]) + (long long)par * W * p.ar_slot_elems;
            for (int i = sub;; i += ROWS_PER_PASS) {
                const int row = r + i * S;
                if (row >= p.M) break;
                if (col >= p.N) continue;
                const long long at = (long long)row * p.N + col;
                float acc[8];
                if (p.Cin) {
                    unpack8(ld8(p.Cin + at), acc);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] *= p.beta;
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                }
                for (int q = 0; q < W; ++q) {                      // rank order: bitwise identical on every rank
                    float tq[8];
                    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(mine + q * p.ar_slot_elems + at));
                    unpack8(*reinterpret_cast<const bf16x8*>(&raw), tq);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] += tq[j];
                }
                st8(p.C + at, pack8(acc));
            }
        }
        // the last CTA to get here advances the call counter
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned total = gridDim.x * gridDim.y;
            const unsigned prev = atomicAdd(p.ar_counters + 1, 1u);
            if (prev == total - 1) {
                p.ar_counters[1] = 0;
                *p.ar_epoch = epoch;
            }
        }
    }
    // nobody leaves while a peer may still read its shared memory
    cluster_sync_all();
    if (warp == 1) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, BN);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_sk() {
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
// bf16 matrix [rows, cols], cols contiguous, row stride ld elements
int make_tmap_sk(CUtensorMap* m, const void* base, long long cols, long long rows, long long ld, int box_cols, int box_rows) {
    EncodeTiledFn enc = get_encode_sk();
    if (!enc) return 100;
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, 1};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(rows * ld) * 2};
    cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 200 + (int)r;
}

// the tile-major copy of a weight: dims {64, 128, K / 64, N / 128}, a box takes whole 16 KB tiles
int make_tmap_packed(CUtensorMap* m, const void* base, long long n_tiles, long long k_tiles, int box_n_tiles) {
    EncodeTiledFn enc = get_encode_sk();
    if (!enc) return 100;
    cuuint64_t dims[4] = {64, 128, (cuuint64_t)k_tiles, (cuuint64_t)n_tiles};
    cuuint64_t strides[3] = {128, 16384, (cuuint64_t)k_tiles * 16384};
    cuuint32_t box[4] = {64, 128, 1, (cuuint32_t)box_n_tiles};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 200 + (int)r;
}

template <int BN, int AM, bool AR>
int launch_skinny(const CUtensorMap& tmA, const CUtensorMap& tmB, const SkinnyParams& p, int tiles, int S, cudaStream_t st) {
    static bool attr_flags[64] = {};
    bool* attr = kb_device_flag(attr_flags);
    if (!attr) return 7;
    if (!*attr) {
        if (cudaFuncSetAttribute(gemm_skinny_kernel<BN, AM, AR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<BN, AM>::SMEM) != cudaSuccess)
            return 7;
        *attr = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(S, tiles, 1);
    cfg.blockDim = dim3(192, 1, 1);
    cfg.dynamicSmemBytes = Cfg<BN, AM>::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = S;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (AR) {
        // every CTA waits for flags that go up only after all CTAs of every rank have pushed: the whole
        // grid must be resident at once
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, gemm_skinny_kernel<BN, AM, AR>, &cfg) != cudaSuccess || clusters < tiles) {
            cudaGetLastError();
            return KB_LAUNCH_FAILED;
        }
    }
    cfg.numAttrs = g_kb_dependent_launch ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<BN, AM, AR>, tmA, tmB, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return KB_LAUNCH_FAILED;
    }
    return 0;
}



struct ArArgs {
    void* const* recv;
    void* const* flags;
    int world, rank;
    long long slot_elems;
    int* epoch;
    unsigned* counters;
    double limit_s;
};

static int skinny_dispatch(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, long long lda,
                           long long ldb, long long ldc, long long ldcin, float alpha, float beta, int split, int bn,
                           int b_packed, int* status, const ArArgs* ar, cudaStream_t st) {
    if (M <= 0 || M > BM || N <= 0 || K <= 0) return 5;
    if ((lda & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return 6;
    if ((b_packed & 1) ? (K % BK) != 0 : (ldb & 7) != 0) return 6;
    if (bn != 0 && bn != 128 && bn != 256) return 5;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int kt = (K + BK - 1) / BK;
    int best_bn = 256, best_s = 1, best_ctas = 0;
    // Cluster sizes 1, 2, 3, 4 and 8 place well; 5 to 7 were measured to run in more than one wave
    // (3072 x 3072: 19.0 us with 6 CTAs per cluster against 11.0 us with 4).  Among the candidates the
    // one with the most CTAs wins, the narrower tile on a tie.
    for (int cand : {128, 256}) {
        if (bn && cand != bn) continue;
        const int tiles = (N + cand - 1) / cand;
        int s = split > 0 ? split : sms / tiles;
        if (s > 8) s = 8;
        if (s > kt / 2) s = kt / 2;
        if (s < 1) s = 1;
        if (split <= 0 && s > 4 && s < 8) s = 4;
        const int per = (kt + s - 1) / s;
        s = (kt + per - 1) / per;                         // no empty K parts
        if (split <= 0 && s > 4 && s < 8) s = 4;
        if (tiles * s > best_ctas) { best_ctas = tiles * s; best_bn = cand; best_s = s; }
    }
    const int tiles = (N + best_bn - 1) / best_bn;
    if (ar && tiles * best_s > sms) return KB_LAUNCH_FAILED;      // the fused all-reduce needs the whole grid resident
    CUtensorMap tmA, tmB;
    const int a_rows = ((M + 7) / 8) * 8;
    int r = make_tmap_sk(&tmA, A, K, M, lda, BK, a_rows);
    if (r) return r;
    if (b_packed & 1) r = make_tmap_packed(&tmB, B, (N + 127) / 128, K / BK, best_bn / 128);
    else r = make_tmap_sk(&tmB, B, K, N, ldb, BK, best_bn);
    if (r) return r;
    SkinnyParams p;
    memset(&p, 0, sizeof(p));
    p.M = M; p.N = N; p.K = K; p.alpha = alpha; p.beta = beta;
    p.C = (__nv_bfloat16*)C; p.Cin = (const __nv_bfloat16*)Cin; p.ldc = ldc; p.ldcin = ldcin; p.status = status;
    p.a_rows = a_rows;
    p.b_packed = b_packed & 1;
    p.b_const = (b_packed >> 1) & 1;
    if (ar) {
        for (int i = 0; i < 8; ++i) {
            p.ar_recv[i] = i < ar->world ? ar->recv[i] : nullptr;
            p.ar_flags[i] = i < ar->world ? ar->flags[i] : nullptr;
        }
        p.ar_world = ar->world; p.ar_rank = ar->rank; p.ar_slot_elems = ar->slot_elems;
        p.ar_epoch = ar->epoch; p.ar_counters = ar->counters;
        p.ar_limit_ns = (unsigned long long)(ar->limit_s * 1e9);
        if (M <= 64)
            return best_bn == 256 ? launch_skinny<256, 64, true>(tmA, tmB, p, tiles, best_s, st)
                                  : launch_skinny<128, 64, true>(tmA, tmB, p, tiles, best_s, st);
        return best_bn == 256 ? launch_skinny<256, 128, true>(tmA, tmB, p, tiles, best_s, st)
                              : launch_skinny<128, 128, true>(tmA, tmB, p, tiles, best_s, st);
    }
    if (M <= 64)
        return best_bn == 256 ? launch_skinny<256, 64, false>(tmA, tmB, p, tiles, best_s, st)
                              : launch_skinny<128, 64, false>(tmA, tmB, p, tiles, best_s, st);
    return best_bn == 256 ? launch_skinny<256, 128, false>(tmA, tmB, p, tiles, best_s, st)
                          : launch_skinny<128, 128, false>(tmA, tmB, p, tiles, best_s, st);
}

}  // namespace

// C[M,N] = alpha * A[M,K] x B[N,K]^T + beta * Cin, all bf16, K contiguous in A and B (lda/ldb in
// elements, multiples of 8; 16-byte aligned bases), M <= 128.  `split` <= 0: chosen here (BN and the
// cluster size that put the most CTAs on the weight stream); otherwise the cluster size to use (1..8).
// Returns 0, a refusal code, or KB_LAUNCH_FAILED when the runtime cannot place the cluster.
// `b_packed` bit 1: B is a constant of the process (a served weight), so a dependent launch may fetch its tiles
// before the kernels ahead of it have finished.
// `b_packed` bit 0: B points at the tile-major copy made by kb_pack_weight_tiles ([ceil(N/128)][K/64][128][64],
// K a multiple of 64); every TMA box is then whole contiguous 16 KB tiles instead of 128-byte pieces 2K
// bytes apart.  Measured on the 3B decode shapes this is worth 3 % (the kernel is bound by the ~70 GB/s
// one SM can take in and by its fixed ~6 us of launch, prologue and cluster reduction, not by DRAM
// locality), so the serving engine does not make the copies unless asked to.
KB_API int kb_gemm_skinny(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, long long lda,
                          long long ldb, long long ldc, long long ldcin, float alpha, float beta, int split, int bn,
                          int b_packed, int* status, cudaStream_t st) {
    return skinny_dispatch(A, B, C, Cin, M, N, K, lda, ldb, ldc, ldcin, alpha, beta, split, bn, b_packed, status, nullptr, st);
}

// Row-parallel projection of tensor-parallel decode in ONE launch: out = sum over ranks of (A_r x B_r^T) + residual.
// The product is the cluster split-K above; its epilogue pushes the summed tile rows into every rank's
// receive buffer (plain peer stores), raises this rank's epoch flag on every peer and sums all ranks' slots.
// Buffers, flags, the device-side call counter and the two election counters are those of
// kb_allreduce_push (same layout, same protocol), so both entry points can share them.  out and residual
// are dense [M, N] bf16, N a multiple of 8, M * N <= slot_elems.  KB_LAUNCH_FAILED: the grid cannot be fully
// resident (the caller then runs the product and the all-reduce as two launches).
KB_API int kb_gemm_skinny_allreduce(const void* A, const void* B, void* out, const void* residual, int M, int N, int K,
                                    long long lda, long long ldb, int b_packed, void* const* peer_recv,
                                    void* const* peer_flags, int world, int rank, long long slot_elems, int* epoch_ptr,
                                    unsigned* counters, double limit_s, int* status, cudaStream_t st) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world || (N & 7) || (slot_elems & 7) ||
        (long long)M * N > slot_elems || !epoch_ptr || !counters)
        return 5;
    for (int i = 0; i < world; ++i)
        if (!peer_recv[i] || !peer_flags[i] || ((uintptr_t)peer_recv[i] & 15)) return 6;
    if (((uintptr_t)out & 15) || ((uintptr_t)residual & 15)) return 6;
    ArArgs ar{peer_recv, peer_flags, world, rank, slot_elems, epoch_ptr, counters, limit_s};
    return skinny_dispatch(A, B, out, residual, M, N, K, lda, ldb, N, N, 1.0f, 1.0f, 0, 0, b_packed, status, &ar, st);
}

// Tile-major copy of a K-major bf16 weight for kb_gemm_skinny: dst[nt][kt][r][c] = w[nt * 128 + r][kt * 64 + c]
// (zero for rows past N).  One-off, at load time.
namespace {
__global__ void pack_weight_tiles_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, __nv_bfloat16* __restrict__ dst,
                                         int N, int k_tiles) {
    const int nt = blockIdx.y, kt = blockIdx.x;
    uint4* out = reinterpret_cast<uint4*>(dst + ((long long)nt * k_tiles + kt) * 8192);
    for (int i = threadIdx.x; i < 1024; i += blockDim.x) {            // 128 rows x 8 chunks of 8 elements
        const int r = i >> 3, c8 = i & 7;
        const int row = nt * 128 + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < N) v = *reinterpret_cast<const uint4*>(w + (long long)row * ldw + kt * 64 + c8 * 8);
        out[i] = v;
    }
}
}  // namespace
KB_API int kb_pack_weight_tiles(const void* w, long long ldw, void* dst, int N, int K, cudaStream_t st) {
    if (N <= 0 || K <= 0 || (K % BK) || (ldw & 7) || ((uintptr_t)w & 15) || ((uintptr_t)dst & 15)) return 5;
    dim3 grid(K / BK, (N + 127) / 128);
    pack_weight_tiles_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)w, ldw, (__nv_bfloat16*)dst, N, K / BK);
    return kb_launch_status();
}
