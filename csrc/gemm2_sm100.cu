// Two-CTA variant of the persistent tcgen05 GEMM: a cluster of two CTAs (one per SM of a pair)
// computes one 256x256 tile with `tcgen05.mma.cta_group::2` (instruction shape 256x256x16).
// Each CTA stages its own 128 rows of A and half (128 rows) of the B tile, so the shared-memory
// fill per SM drops from 48 KB to 32 KB per 64-deep K block, which is what limited the one-CTA
// kernel.  No load names another CTA as a destination: every CTA fetches its own operand slices;
// only barrier traffic crosses the pair (TMA completion bytes counted on the leader's barrier,
// commits from the leader to both CTAs, epilogue arrivals from the peer to the leader).
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocation (+ MMA issue in
// the leader CTA only), warps 2-5 = epilogue.  Same operand majors, batching and fused
// alpha*acc + beta*Cin epilogue as the one-CTA kernel.
#include <cuda.h>
#include <stdlib.h>

#include "tc.cuh"

namespace {

constexpr int BM = 128;            // rows per CTA (256 per pair)
constexpr int BNI = 256;           // columns per MMA instruction (128 rows of B staged per CTA)
constexpr int BNH = 128;
constexpr int BK = 64;
constexpr int A_STAGE = BM * BK * 2, B_SUB = BNH * BK * 2;
// NSUB = 1: 256x256 tile per pair, six stages, two accumulator buffers (epilogue overlaps the next
// tile).  NSUB = 2: 256x512 tile (two MMAs per K step that share A), four stages, one accumulator
// set filling all 512 TMEM columns: 25 % less operand traffic per FLOP - the operand feed from L2
// is what bounds the narrow tile - at the price of an epilogue that is not hidden.
template <int NSUB> struct Cfg {
    static constexpr int BN = BNI * NSUB;
    static constexpr int STAGES = NSUB == 1 ? 6 : 4;
    static constexpr int B_STAGE = B_SUB * NSUB;
    static constexpr int NBUF = NSUB == 1 ? 2 : 1;
    static constexpr int SMEM = STAGES * (A_STAGE + B_STAGE) + 1024 + 256 + 4 * 32 * 144;
};
constexpr int EPI_PITCH = 144;                      // staged row: 64 bf16 + 16 bytes (bank spread)
constexpr int EPI_WARP_BYTES = 32 * EPI_PITCH;
constexpr int GROUP_M = 8;

struct Gemm2Params {
    int M, N, K, batch;
    int a_mn, b_mn, a_fmt, b_fmt, out_type;
    float alpha, beta;
    void* C;
    const void* Cin;
    long long ldc, c_batch_stride, ldcin, cin_batch_stride;
    int* status;
    int sym_upper;             // square symmetric result: tiles strictly below the diagonal are skipped
    int group_m;               // raster: tiles are visited in column sweeps over groups of this many tile rows
    int epi_staged;            // 16-bit output without addend: transpose chunks through shared memory, store 128-byte row segments
    int epi_cin_staged;        // 16-bit output and addend, no symmetry/diagonal: coalesced addend reads and stores
    // all-gather coupling (see kb_gemm_ag in gemm_sm100.cu): the gathered operand sits in a local staging
    // buffer that peers fill shard by shard; producers wait (bounded) for a shard's flag before its first tile
    const int* ag_flags;       // null: none
    int ag_epoch, ag_rows, ag_dim, ag_rot;   // rows per shard; 0 = shards along M (A rows), 1 = along K; ag_rot: first k-block (ag_dim 1)
    unsigned long long ag_limit_ns;
    int m_rot;                 // tile rows are visited starting from this one (own shard first / next rank's rows first)
    // reduce-scatter coupling (see kb_gemm_rs in gemm_sm100.cu): rows [o*rs_rows, (o+1)*rs_rows) are stored to
    // rs_out[o] (row stride ldc) and every epilogue warp adds one arrival to rs_cnt[o] per tile
    void* rs_out[8];
    int* rs_cnt[8];
    int rs_rows;               // 0: none
    float diag_add;            // added to the diagonal of the result (after alpha/beta): folds the a*X term of Newton-Schulz into B
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x,
                                                 int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma2_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on a barrier (cluster address) once all MMAs issued so far by this thread are done.
__device__ __forceinline__ void commit2(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& b, int& tm, int& tn,
                                            int group_m = GROUP_M) {
    const int per_batch = tiles_m * tiles_n;
    b = tile / per_batch;
    int t = tile % per_batch;
    const int group = group_m * tiles_n;
    const int g = t / group;
    const int first_m = g * group_m;
    const int gm = min(group_m, tiles_m - first_m);
    t -= g * group;
    tm = first_m + t % gm;
    tn = t / gm;
}

// Symmetric results (square, 256 x 256 pair tiles): only the tiles on and above the diagonal exist as work
// items - T (T + 1) / 2 per batch entry, numbered row by row - so that every CTA pair gets the same number of
// them.  (Skipping the lower tiles of a full enumeration left the pairs with 12 to 19 tiles each and the
// symmetric product at 88 % of the full one's time for 54 % of its tiles.)
__device__ __forceinline__ void sym_tile_coords(int tile, int T, int& b, int& tm, int& tn) {
    const int U = T * (T + 1) / 2;
    b = tile / U;
    int u = tile - b * U;
    tm = 0;
    while (u >= T - tm) {
        u -= T - tm;
        ++tm;
    }
    tn = tm + u;
}
__device__ __forceinline__ void work_coords(int tile, int tiles_m, int tiles_n, bool sym, int group_m, int& b, int& tm, int& tn) {
    if (sym) sym_tile_coords(tile, tiles_m, b, tm, tn);
    else tile_coords(tile, tiles_m, tiles_n, b, tm, tn, group_m);
}

__device__ __forceinline__ bool wait_shard2(const int* flag, int epoch, unsigned long long limit_ns,
                                            volatile int* abort_flag) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v < epoch) {
        const uint64_t t0 = global_timer_ns();
        unsigned sleep_ns = 64;
        for (;;) {
            asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v >= epoch) break;
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

template <typename T>
__device__ __forceinline__ float h2f(T x);
template <> __device__ __forceinline__ float h2f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float h2f<__half>(__half x) { return __half2float(x); }
template <typename T>
__device__ __forceinline__ T f2h(float x);
template <> __device__ __forceinline__ __nv_bfloat16 f2h<__nv_bfloat16>(float x) { return __float2bfloat16(x); }
template <> __device__ __forceinline__ __half f2h<__half>(float x) { return __float2half(x); }

template <typename T>
__device__ __forceinline__ void store32_16(T* dst, const T* cin, const uint32_t* acc, float alpha, float beta,
                                           int ncols, bool vec_ok, T* mdst = nullptr, long long mld = 0) {
    // mdst (symmetric results): this lane's element (row, col + j) is also written to (col + j, row);
    // for a fixed j the 32 lanes of the warp then write 32 consecutive elements of one row.
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
            if (mdst) {
#pragma unroll
                for (int i = 0; i < 8; ++i) mdst[(long long)(8 * j + i) * mld] = op[i];
            }
        }
    } else {
        for (int j = 0; j < ncols; ++j) {
            float v = alpha * __uint_as_float(acc[j]);
            if (cin) v += beta * h2f<T>(cin[j]);
            dst[j] = f2h<T>(v);
            if (mdst) mdst[(long long)j * mld] = f2h<T>(v);
        }
    }
}

template <int NSUB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const Gemm2Params p) {
    constexpr int BN = Cfg<NSUB>::BN, STAGES = Cfg<NSUB>::STAGES, B_STAGE = Cfg<NSUB>::B_STAGE, NBUF = Cfg<NSUB>::NBUF;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE + B_STAGE));
    uint64_t* full = bars;                          // [STAGES] in the leader: both CTAs' TMA bytes
    uint64_t* empty = bars + STAGES;                // [STAGES] per CTA: leader's commit
    uint64_t* acc_full = bars + 2 * STAGES;         // [2] per CTA: leader's commit
    uint64_t* acc_empty = bars + 2 * STAGES + 2;    // [2] in the leader: 8 epilogue warps
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM), tiles_n = (p.N + BN - 1) / BN;
    // symmetric enumeration needs a square tile grid, i.e. the 256 x 256 tile (BN == 2 * BM)
    const bool sym_enum = p.sym_upper && NSUB == 1 && tiles_m == tiles_n;
    const int num_tiles = sym_enum ? tiles_m * (tiles_m + 1) / 2 * p.batch : tiles_m * tiles_n * p.batch;
    const int kblocks = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            tc::mbar_init(&acc_full[b], 1);
            tc::mbar_init(&acc_empty[b], 8);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc2(tmem_slot, 512);
        tmem_relinquish2();
    }
    tc::tc_fence_before();
    __syncthreads();
    cluster_sync();                                  // peer barriers are initialised before anyone signals them
    tc::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // every pipeline wait sits behind the producer's wait for a peer's shard when the kernel is coupled to an
    // all-gather: give them that wait's limit on top of their own
    const uint64_t wait_ns = p.ag_flags ? p.ag_limit_ns + 2000000000ull : 2000000000ull;

    if (warp == 0) {
        if (lane == 0) {
            tc::prefetch_tmap(&tmA);
            tc::prefetch_tmap(&tmB);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            unsigned ready_mask = 0;        // shards already seen ready
            for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
                int b, tm, tn;
                work_coords(tile, tiles_m, tiles_n, sym_enum, p.group_m, b, tm, tn);
                if (p.sym_upper && !sym_enum && tn * BN + BN <= tm * 2 * BM) continue;
                if (p.m_rot) {
                    tm += p.m_rot;
                    if (tm >= tiles_m) tm -= tiles_m;
                }
                if (p.ag_flags && p.ag_dim == 0) {
                    const int s0 = (tm * 2 * BM) / p.ag_rows, s1 = (min(tm * 2 * BM + 2 * BM, p.M) - 1) / p.ag_rows;
                    for (int sh = s0; sh <= s1 && ok; ++sh) {
                        if (ready_mask >> sh & 1) continue;
                        if (!wait_shard2(p.ag_flags + sh, p.ag_epoch, p.ag_limit_ns, abort_flag)) {
                            atomicMax(p.status, (int)KB_TIMEOUT_PEER);
                            ok = false;
                        }
                        ready_mask |= 1u << sh;
                    }
                    if (!ok) break;
                }
                const int m0 = tm * 2 * BM + (int)rank * BM, n0 = tn * BN + (int)rank * BNH;   // sub-tile j adds j * BNI
                for (int kbi = 0; kbi < kblocks; ++kbi) {
                    int kb = kbi;
                    if (p.ag_flags && p.ag_dim == 1) {
                        kb += p.ag_rot;
                        if (kb >= kblocks) kb -= kblocks;
                        const int sh = (kb * BK) / p.ag_rows;
                        if (!(ready_mask >> sh & 1)) {
                            if (!wait_shard2(p.ag_flags + sh, p.ag_epoch, p.ag_limit_ns, abort_flag)) {
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
                    const uint32_t full_leader = mapa(smem_u32(&full[stage]), 0);
                    if (leader) tc::mbar_expect_tx(&full[stage], 2 * (A_STAGE + B_STAGE));
                    uint8_t* a_dst = sA + stage * A_STAGE;
                    uint8_t* b_dst = sB + stage * B_STAGE;
                    if (p.a_mn) {
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c)
                            tma_load_3d_pair(a_dst + c * (64 * BK * 2), &tmA, full_leader, m0 + c * 64, kb * BK, b);
                    } else {
                        tma_load_3d_pair(a_dst, &tmA, full_leader, kb * BK, m0, b);
                    }
#pragma unroll
                    for (int j = 0; j < NSUB; ++j) {
                        if (p.b_mn) {
#pragma unroll
                            for (int c = 0; c < BNH / 64; ++c)
                                tma_load_3d_pair(b_dst + j * B_SUB + c * (64 * BK * 2), &tmB, full_leader,
                                                 n0 + j * BNI + c * 64, kb * BK, b);
                        } else {
                            tma_load_3d_pair(b_dst + j * B_SUB, &tmB, full_leader, kb * BK, n0 + j * BNI, b);
                        }
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            const uint32_t idesc = tc::instr_desc_f16(2 * BM, BNI, p.a_fmt, p.b_fmt, p.a_mn, p.b_mn);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
                if (p.sym_upper && !sym_enum) {
                    int b_, tm_, tn_;
                    tile_coords(tile, tiles_m, tiles_n, b_, tm_, tn_, p.group_m);
                    if (tn_ * BN + BN <= tm_ * 2 * BM) continue;
                }
                const int buf = it % NBUF;
                const uint32_t acc_phase = (it / NBUF) & 1;
                ++it;
                if (!tc::mbar_wait(&acc_empty[buf], acc_phase ^ 1, abort_flag, wait_ns)) {
                    atomicMax(p.status, (int)KB_TIMEOUT_MMA);
                    ok = false;
                    break;
                }
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;      // NBUF * BN = 512 columns in both shapes
                for (int kb = 0; kb < kblocks; ++kb) {
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
#pragma unroll
                        for (int j = 0; j < NSUB; ++j) {
                            const uint32_t bj = b_addr + j * B_SUB;
                            const uint64_t bd = p.b_mn ? tc::smem_desc_sw128(bj + k * 2048, 64 * BK * 2, 1024)
                                                       : tc::smem_desc_sw128(bj + k * 32, 16, 1024);
                            mma2_f16(d_tmem + j * BNI, ad, bd, idesc, (kb | k) != 0);
                        }
                    }
                    // the stage is reusable in both CTAs once these MMAs have read it
                    commit2(mapa(smem_u32(&empty[stage]), 0));
                    commit2(mapa(smem_u32(&empty[stage]), 1));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) {
                    commit2(mapa(smem_u32(&acc_full[buf]), 0));
                    commit2(mapa(smem_u32(&acc_full[buf]), 1));
                }
            }
        }
    } else {
        const int quarter = warp & 3;
        int it = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
            int b, tm, tn;
            work_coords(tile, tiles_m, tiles_n, sym_enum, p.group_m, b, tm, tn);
            if (p.sym_upper && !sym_enum && tn * BN + BN <= tm * 2 * BM) continue;
            if (p.m_rot) {
                tm += p.m_rot;
                if (tm >= tiles_m) tm -= tiles_m;
            }
            const int buf = it % NBUF;
            const uint32_t acc_phase = (it / NBUF) & 1;
            ++it;
            if (!tc::mbar_wait(&acc_full[buf], acc_phase, abort_flag, wait_ns)) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                ok = false;
                break;
            }
            tc::tc_fence_after();
            const int row = tm * 2 * BM + (int)rank * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
            const bool mirror = NSUB == 1 && p.sym_upper && tn > tm;     // 256 x 256 pair tiles: tn > tm is strictly above the diagonal
            if (p.epi_staged) {
                // no addend, 16-bit output: each 32x64 chunk goes through shared memory so that a warp
                // store covers four 128-byte row segments instead of 32 scattered 16-byte pieces
                uint8_t* stg = smem + STAGES * (A_STAGE + B_STAGE) + 256 + (warp - 2) * EPI_WARP_BYTES;
                const int row0 = tm * 2 * BM + (int)rank * BM + quarter * 32;
                uint16_t* obase = reinterpret_cast<uint16_t*>(p.C) + (long long)b * p.c_batch_stride + (long long)row0 * p.ldc;
                if (p.rs_rows > 0) {
                    // reduce-scatter: these 32 rows go to their owner's slab, as 128-byte row segments over NVLink
                    const int owner = row0 / p.rs_rows;
                    obase = reinterpret_cast<uint16_t*>(p.rs_out[owner]) + (long long)(row0 - owner * p.rs_rows) * p.ldc;
                }
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    uint32_t acc[64];
                    tc::tmem_ld32(taddr + c0, acc);
                    tc::tmem_ld32(taddr + c0 + 32, acc + 32);
                    tc::tmem_ld_wait();
                    if (mirror && row0 + lane < p.M) {
                        // symmetric result, tile above the diagonal: element (row, col) also goes to (col, row)
                        uint16_t* mb = reinterpret_cast<uint16_t*>(p.C) + (long long)b * p.c_batch_stride + row0 + lane;
#pragma unroll
                        for (int j = 0; j < 64; ++j) {
                            const int cc = tn * BN + c0 + j;
                            if (cc < p.N) {
                                const float v = p.alpha * __uint_as_float(acc[j]);
                                mb[(long long)cc * p.ldc] = p.out_type == 1 ? __bfloat16_as_ushort(__float2bfloat16(v))
                                                                            : __half_as_ushort(__float2half(v));
                            }
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint4 o;
                        if (p.out_type == 1) {
                            __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                op[i] = __floats2bfloat162_rn(p.alpha * __uint_as_float(acc[8 * j + 2 * i]),
                                                              p.alpha * __uint_as_float(acc[8 * j + 2 * i + 1]));
                        } else {
                            __half2* op = reinterpret_cast<__half2*>(&o);
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                op[i] = __floats2half2_rn(p.alpha * __uint_as_float(acc[8 * j + 2 * i]),
                                                          p.alpha * __uint_as_float(acc[8 * j + 2 * i + 1]));
                        }
                        *reinterpret_cast<uint4*>(stg + lane * EPI_PITCH + j * 16) = o;
                    }
                    __syncwarp();
                    const int seg = lane & 7, col = tn * BN + c0 + seg * 8;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = i * 4 + (lane >> 3);
                        const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * EPI_PITCH + seg * 16);
                        if (row0 + rr < p.M && col < p.N)
                            *reinterpret_cast<uint4*>(obase + (long long)rr * p.ldc + col) = v;
                    }
                    __syncwarp();
                }
            } else if (p.epi_cin_staged) {
                // 16-bit output with a 16-bit addend: each 32x32 fp32 chunk is transposed through shared
                // memory; a lane then owns four consecutive columns of one row, so addend reads and result
                // stores are 64-byte row segments (eight lanes per row) instead of one row per lane
                float* stg = reinterpret_cast<float*>(smem + STAGES * (A_STAGE + B_STAGE) + 256 + (warp - 2) * EPI_WARP_BYTES);
                const int row0 = tm * 2 * BM + (int)rank * BM + quarter * 32;
                const long long obase = (long long)b * p.c_batch_stride + (long long)row0 * p.ldc;
                const long long ibase = (long long)b * p.cin_batch_stride + (long long)row0 * p.ldcin;
                const uint16_t* cin16 = reinterpret_cast<const uint16_t*>(p.Cin);
                uint16_t* out16 = reinterpret_cast<uint16_t*>(p.C);
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t acc[32];
                    tc::tmem_ld32(taddr + c0, acc);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4*>(stg + lane * (EPI_PITCH / 4) + 4 * j) =
                            make_float4(p.alpha * __uint_as_float(acc[4 * j]), p.alpha * __uint_as_float(acc[4 * j + 1]),
                                        p.alpha * __uint_as_float(acc[4 * j + 2]), p.alpha * __uint_as_float(acc[4 * j + 3]));
                    __syncwarp();
                    const int col = tn * BN + c0 + (lane & 7) * 4;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = i * 4 + (lane >> 3);
                        if (row0 + rr < p.M && col < p.N) {
                            float4 v = *reinterpret_cast<const float4*>(stg + rr * (EPI_PITCH / 4) + (lane & 7) * 4);
                            const uint2 craw = *reinterpret_cast<const uint2*>(cin16 + ibase + (long long)rr * p.ldcin + col);
                            uint2 o;
                            if (p.out_type == 1) {
                                const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&craw);
                                const float2 c01 = __bfloat1622float2(c2[0]), c23 = __bfloat1622float2(c2[1]);
                                __nv_bfloat162 r0 = __floats2bfloat162_rn(v.x + p.beta * c01.x, v.y + p.beta * c01.y);
                                __nv_bfloat162 r1 = __floats2bfloat162_rn(v.z + p.beta * c23.x, v.w + p.beta * c23.y);
                                o.x = *reinterpret_cast<uint32_t*>(&r0);
                                o.y = *reinterpret_cast<uint32_t*>(&r1);
                            } else {
                                const __half2* c2 = reinterpret_cast<const __half2*>(&craw);
                                const float2 c01 = __half22float2(c2[0]), c23 = __half22float2(c2[1]);
                                __half2 r0 = __floats2half2_rn(v.x + p.beta * c01.x, v.y + p.beta * c01.y);
                                __half2 r1 = __floats2half2_rn(v.z + p.beta * c23.x, v.w + p.beta * c23.y);
                                o.x = *reinterpret_cast<uint32_t*>(&r0);
                                o.y = *reinterpret_cast<uint32_t*>(&r1);
                            }
                            *reinterpret_cast<uint2*>(out16 + obase + (long long)rr * p.ldc + col) = o;
                        }
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
                if (p.diag_add != 0.f && row >= col && row < col + 32) {
                    const float d = p.diag_add / p.alpha;      // the stores below scale by alpha
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col + j == row) acc[j] = __float_as_uint(__uint_as_float(acc[j]) + d);
                }
                if (row < p.M && ncols > 0) {
                    const long long off = (long long)b * p.c_batch_stride + (long long)row * p.ldc + col;
                    const long long offin = (long long)b * p.cin_batch_stride + (long long)row * p.ldcin + col;
                    if (p.out_type == 2) {
                        float* dst = reinterpret_cast<float*>(p.C) + off;
                        const float* cin = p.Cin ? reinterpret_cast<const float*>(p.Cin) + offin : nullptr;
                        for (int j = 0; j < ncols; ++j) {
                            float v = p.alpha * __uint_as_float(acc[j]);
                            if (cin) v += p.beta * cin[j];
                            dst[j] = v;
                        }
                    } else {
                        const bool vec = ((p.ldc | p.ldcin | col) & 7) == 0;
                        if (p.out_type == 1) {
                            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
                            const __nv_bfloat16* cin =
                                p.Cin ? reinterpret_cast<const __nv_bfloat16*>(p.Cin) + offin : nullptr;
                            store32_16<__nv_bfloat16>(dst, cin, acc, p.alpha, p.beta, ncols, vec,
                                                      mirror ? reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)b * p.c_batch_stride + (long long)col * p.ldc + row : nullptr,
                                                      p.ldc);
                        } else {
                            __half* dst = reinterpret_cast<__half*>(p.C) + off;
                            const __half* cin = p.Cin ? reinterpret_cast<const __half*>(p.Cin) + offin : nullptr;
                            store32_16<__half>(dst, cin, acc, p.alpha, p.beta, ncols, vec,
                                               mirror ? reinterpret_cast<__half*>(p.C) + (long long)b * p.c_batch_stride + (long long)col * p.ldc + row : nullptr,
                                               p.ldc);
                        }
                    }
                }
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa(smem_u32(&acc_empty[buf]), 0));
            if (p.rs_rows > 0) {
                // this warp's 32 rows of the tile are with their owner: publish one arrival
                __threadfence_system();
                __syncwarp();
                if (lane == 0) {
                    int* cnt = p.rs_cnt[(tm * 2 * BM + (int)rank * BM) / p.rs_rows];
                    asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(cnt) : "memory");
                }
            }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    cluster_sync();                                  // no remote arrival may target a CTA that has left
    if (warp == 1) {
        tc::tc_fence_after();
        tmem_dealloc2(tmem_base, 512);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode2() {
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

int make_tmap2(CUtensorMap* m, const void* base, int fmt, long long cols, long long rows, long long ld,
               long long batch, long long batch_stride, int box_cols, int box_rows) {
    EncodeTiledFn enc = get_encode2();
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

}  // namespace

struct AgArgs {
    const int* flags;
    int epoch, rows, dim, own;
    double limit_s;
};
struct RsArgs {
    void* const* out;
    int* const* cnt;
    int world, rank, rows;
};

// Wide (256 x 512) tiles for large non-symmetric products without addend whose tile count still fills the
// machine; KB_GEMM2_WIDE=0/1 forces the choice (tuning).  Measured over the 3B projection shapes: 0.94x of
// cuBLAS with wide tiles against 0.87x without (products with an addend keep the narrow tile: reading the
// addend in an epilogue that is not hidden behind the next tile cost more than the wide tile gains).
static bool choose_wide(int M, int N, int batch, bool sym_upper, bool addend, int sms) {
    static int wide_env = -2;
    if (wide_env == -2) {
        const char* w = getenv("KB_GEMM2_WIDE");
        wide_env = w ? atoi(w) : -1;
    }
    const long long m_tiles = (M + 2 * BM - 1) / (2 * BM);
    const long long wide_tiles = m_tiles * ((N + 2 * BNI - 1) / (2 * BNI)) * batch;
    bool wide = !sym_upper && !addend && N >= 2 * BNI && wide_tiles >= 2 * (sms / 2);
    if (wide_env >= 0) wide = wide && wide_env != 0;
    return wide;
}
// Reduce-scatter products keep the narrow tile unless KB_GEMM2_RS_WIDE=1: its two accumulator buffers hide the
// slow peer stores of one tile behind the math of the next.
static bool rs_wide() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("KB_GEMM2_RS_WIDE");
        v = e ? (atoi(e) != 0) : 0;
    }
    return v != 0;
}
static int device_sms() {
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

static int launch_gemm2(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, int batch,
                        long long lda, long long ldb, long long ldc, long long ldcin, long long a_bs, long long b_bs,
                        long long c_bs, long long cin_bs, int a_mn, int b_mn, int a_fmt, int b_fmt, int out_type,
                        float alpha, float beta, int* status, int max_ctas, int sym_upper, float diag_add,
                        const AgArgs* ag, const RsArgs* rs, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 5;
    if (sym_upper && M != N) return 5;
    if ((lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return 6;
    if (batch > 1 && ((a_bs & 7) || (b_bs & 7))) return 6;
    static bool attr_flags[64] = {};
    bool* attr_set_p = kb_device_flag(attr_flags);
    if (!attr_set_p) return 7;
    if (!*attr_set_p) {
        if (cudaFuncSetAttribute(gemm_tcgen05_2cta_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<1>::SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_tcgen05_2cta_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<2>::SMEM) != cudaSuccess)
            return 7;
        *attr_set_p = true;
    }
    CUtensorMap tmA, tmB;
    int r;
    if (a_mn) r = make_tmap2(&tmA, A, a_fmt, M, K, lda, batch, a_bs, 64, BK);
    else r = make_tmap2(&tmA, A, a_fmt, K, M, lda, batch, a_bs, BK, BM);
    if (r) return r;
    if (b_mn) r = make_tmap2(&tmB, B, b_fmt, N, K, ldb, batch, b_bs, 64, BK);
    else r = make_tmap2(&tmB, B, b_fmt, K, N, ldb, batch, b_bs, BK, BNH);
    if (r) return r;
    Gemm2Params p;
    p.M = M; p.N = N; p.K = K; p.batch = batch;
    p.a_mn = a_mn; p.b_mn = b_mn; p.a_fmt = a_fmt; p.b_fmt = b_fmt; p.out_type = out_type;
    p.alpha = alpha; p.beta = beta; p.C = C; p.Cin = Cin;
    p.ldc = ldc; p.c_batch_stride = c_bs; p.ldcin = ldcin; p.cin_batch_stride = cin_bs;
    p.status = status;
    p.sym_upper = sym_upper;
    p.diag_add = diag_add;
    p.ag_flags = nullptr;
    p.ag_epoch = p.ag_rows = p.ag_dim = p.ag_rot = 0;
    p.ag_limit_ns = 0;
    p.m_rot = 0;
    p.rs_rows = 0;
    for (int i = 0; i < 8; ++i) { p.rs_out[i] = nullptr; p.rs_cnt[i] = nullptr; }
    if (ag) {
        p.ag_flags = ag->flags; p.ag_epoch = ag->epoch; p.ag_rows = ag->rows; p.ag_dim = ag->dim;
        if (ag->dim == 0) p.m_rot = ag->own * (ag->rows / (2 * BM));
        else p.ag_rot = ag->own * (ag->rows / BK);
        p.ag_limit_ns = (unsigned long long)(ag->limit_s * 1e9);
    }
    if (rs) {
        for (int i = 0; i < rs->world; ++i) { p.rs_out[i] = rs->out[i]; p.rs_cnt[i] = rs->cnt[i]; }
        p.rs_rows = rs->rows;
        p.m_rot = ((rs->rank + 1) % rs->world) * (rs->rows / (2 * BM));
    }
    if (diag_add != 0.f && (alpha == 0.f || !Cin)) return 5;     // implemented on the addend epilogue only
    {
        static int group_m = 0, staged = -1;
        if (!group_m) {
            const char* g = getenv("KB_GEMM2_GROUP_M");
            group_m = g ? atoi(g) : GROUP_M;
            if (group_m < 1) group_m = GROUP_M;
            const char* e = getenv("KB_GEMM2_EPI_STAGED");
            staged = e ? atoi(e) : 1;
        }
        p.group_m = group_m;
        p.epi_staged = staged && !Cin && out_type != 2 && !(N & 7) && !(ldc & 7) && !(c_bs & 7);
        if (rs) p.epi_staged = 1;      // the reduce-scatter stores exist on this epilogue only (its conditions were checked by the caller)
        // off unless KB_GEMM2_CIN_STAGED=1: measured slower (1-GPU step 861 -> 904 ms) - an addend read costs a
        // memory round trip per chunk, which only the narrow tile's second accumulator buffer hides
        static int cin_staged = -1;
        if (cin_staged < 0) {
            const char* e = getenv("KB_GEMM2_CIN_STAGED");
            cin_staged = e ? atoi(e) : 0;
        }
        p.epi_cin_staged = cin_staged && staged && Cin && out_type != 2 && !sym_upper && diag_add == 0.f && !(N & 3) && !(ldc & 3) &&
                           !(ldcin & 3) && !(c_bs & 3) && !(cin_bs & 3) && !((uintptr_t)C & 7) && !((uintptr_t)Cin & 7);
    }
    int sms = device_sms();
    if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
    const long long m_tiles = (M + 2 * BM - 1) / (2 * BM);
    const long long wide_tiles = m_tiles * ((N + 2 * BNI - 1) / (2 * BNI)) * batch;
    const bool wide = choose_wide(M, N, batch, sym_upper != 0, Cin != nullptr, sms) && (!rs || rs_wide());
    const long long tiles = wide ? wide_tiles : m_tiles * ((N + BNI - 1) / BNI) * batch;
    int pairs = sms / 2;
    if (tiles < pairs) pairs = (int)tiles;
    if (wide) gemm_tcgen05_2cta_kernel<2><<<2 * pairs, 192, Cfg<2>::SMEM, st>>>(tmA, tmB, p);
    else gemm_tcgen05_2cta_kernel<1><<<2 * pairs, 192, Cfg<1>::SMEM, st>>>(tmA, tmB, p);
    return kb_launch_status();
}

// Same contract as kb_gemm (no split-K); launched as clusters of two CTAs.
KB_API int kb_gemm_2cta(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, int batch,
                        long long lda, long long ldb, long long ldc, long long ldcin, long long a_bs, long long b_bs,
                        long long c_bs, long long cin_bs, int a_mn, int b_mn, int a_fmt, int b_fmt, int out_type,
                        float alpha, float beta, int* status, int max_ctas, int sym_upper, float diag_add,
                        cudaStream_t st) {
    return launch_gemm2(A, B, C, Cin, M, N, K, batch, lda, ldb, ldc, ldcin, a_bs, b_bs, c_bs, cin_bs, a_mn, b_mn,
                        a_fmt, b_fmt, out_type, alpha, beta, status, max_ctas, sym_upper, diag_add, nullptr, nullptr, st);
}

// All-gather -> GEMM on the CTA-pair kernel; same contract as kb_gemm_ag (shards of `ag_rows` rows of A
// for ag_dim 0, of the contraction dimension for ag_dim 1; ag_flags[s] >= ag_epoch marks shard s as landed;
// the own shard is visited first).  ag_rows must be a multiple of the 256-row tile (ag_dim 0) or of 64.
KB_API int kb_gemm_2cta_ag(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K,
                           long long lda, long long ldb, long long ldc, int a_mn, int b_mn, float alpha, float beta,
                           const int* ag_flags, int ag_epoch, int ag_rows, int ag_dim, int own, double limit_s,
                           int* status, cudaStream_t st) {
    if (!ag_flags || ag_rows <= 0 || own < 0 || own > 7) return 5;
    if (ag_dim == 0 ? (ag_rows % (2 * BM)) != 0 : (ag_rows % BK) != 0) return 5;
    if ((ag_dim == 0 ? M : K) > 8 * (long long)ag_rows) return 5;
    if ((ag_dim == 0 ? M : K) % ag_rows || (long long)own * ag_rows >= (ag_dim == 0 ? M : K)) return 5;
    AgArgs ag{ag_flags, ag_epoch, ag_rows, ag_dim, own, limit_s};
    return launch_gemm2(A, B, C, Cin, M, N, K, 1, lda, ldb, ldc, ldc, 0, 0, 0, 0, a_mn, b_mn, 1, 1, 1, alpha, beta,
                        status, 0, 0, 0.f, &ag, nullptr, st);
}

// GEMM -> reduce-scatter (producer half) on the CTA-pair kernel; same contract as kb_gemm_rs, rs_rows a
// multiple of the 256-row tile.  kb_gemm_2cta_rs_arrivals gives the arrivals each owner's counter receives.
KB_API int kb_gemm_2cta_rs(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                           long long ldc, int a_mn, int b_mn, float alpha, void* const* rs_out, int* const* rs_cnt,
                           int world, int rank, int rs_rows, int* status, cudaStream_t st) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world || rs_rows <= 0 || (rs_rows % (2 * BM)) != 0 ||
        M != world * rs_rows)
        return 5;
    if ((N & 7) || (ldc & 7)) return 6;
    for (int i = 0; i < world; ++i)
        if (!rs_out[i] || !rs_cnt[i] || ((uintptr_t)rs_out[i] & 15)) return 6;
    RsArgs rs{rs_out, rs_cnt, world, rank, rs_rows};
    return launch_gemm2(A, B, rs_out[rank], nullptr, M, N, K, 1, lda, ldb, ldc, 0, 0, 0, 0, 0, a_mn, b_mn, 1, 1, 1,
                        alpha, 0.f, status, 0, 0, 0.f, nullptr, &rs, st);
}
KB_API int kb_gemm_2cta_rs_arrivals(int M, int N, int rs_rows) {
    const int bn = choose_wide(M, N, 1, false, false, device_sms()) && rs_wide() ? 2 * BNI : BNI;
    return (rs_rows / BM) * ((N + bn - 1) / bn) * 4;
}
