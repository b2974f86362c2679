// Block-scaled fp8 (e4m3) GEMM on the hardware block-scaled tensor-core path of sm_100a:
//   C = alpha * sum_kb (A_kb x B_kb^T) * sa[kb][m] * sb[kb][n / b_gran]  + beta * Cin
// with the same operands and scale arrays as kb_gemm_fp8 (1x128 activation scales, 128x128 weight
// blocks or per-row scales), under one extra contract: every scale is a power of two.  Then a
// scale is exactly an 8-bit exponent (UE8M0), `tcgen05.mma.kind::mxf8f6f4.block_scale` applies
// sa*sb inside the tensor core, and the whole K loop accumulates in one TMEM accumulator: no
// per-K-block promotion through registers, which is what bounds kb_gemm_fp8.
//
//   TMA (128-byte swizzle; a 128-byte row = one K block of 128 e4m3) -> 4-stage ring
//   scale warps: fp32 scales -> exponent bytes -> tensor memory (tcgen05.st), 4 slots ahead
//   MMA thread : four 128x224x32 block-scaled MMAs per K block, scale byte selected per MMA
//   epilogue   : 4 warps drain one of two accumulators while the other one is being filled
//
// Scale factors in tensor memory: the scale of operand row r for the four 32-wide K steps of a
// K block is one 32-bit word (one byte per step) at lane r % 32, column r / 32, and every 32-lane
// quarter holds the same copy; A takes 4 columns (128 rows), B takes 8 (up to 256 rows).  The tile
// is 128 x 224 so that two accumulators (columns [0,224) and [256,480)) leave 2 x 32 columns for
// four scale slots.  Rows of an operand past its end are zero-filled by TMA; their scale index is
// clamped so that the exponent byte stays a valid number.
// Two launch shapes of one kernel.  CTAS = 1: a CTA per 128 x 224 tile.  CTAS = 2: a cluster of two
// CTAs (an SM pair) per 256 x 224 tile with `cta_group::2` MMAs: each CTA stages its own 128 rows of
// A and 112 rows of B, which halves the operand bytes drawn from L2 per FLOP - the limit of the
// one-CTA shape, as of the bf16 kernels - and takes the shared-memory read rate per MMA below the
// tensor core's appetite.  Each CTA of a pair writes the A scales of its own rows and the B scales
// of all 224 columns into its own tensor memory; only barrier traffic crosses the pair.
// All waits are bounded (status word).
#include <cuda.h>
#include <string.h>

#include "tc.cuh"

namespace {

constexpr int BM = 128, BN = 224, BK = 128, NBUF = 2, SF_SLOTS = 4;
constexpr int A_STAGE = BM * BK;                         // bytes (1 byte per element)
constexpr int EPI_PITCH = 80;                            // staged row: 32 bf16 + 16 bytes (conflict-free 16-byte accesses)
constexpr int EPI_WARP_BYTES = 32 * EPI_PITCH;
constexpr int THREADS = 320;                             // TMA, MMA, 4 scale warps, 4 epilogue warps
template <int CTAS> struct Cfg {
    static constexpr int B_ROWS = BN / CTAS;             // rows of the B tile staged by one CTA
    static constexpr int B_STAGE = B_ROWS * BK;
    static constexpr int STAGES = CTAS == 1 ? 4 : 6;
    static constexpr int SMEM = STAGES * (A_STAGE + B_STAGE) + 1024 + 256 + 4 * EPI_WARP_BYTES;
};

struct MxParams {
    int M, N, K;
    const float* sa;     // [K/128][M]
    const float* sb;     // [K/128][sb_ld]
    int b_gran, sb_ld;
    int out_type;        // 1 bf16, 2 fp32
    float alpha, beta;
    void* C;
    const void* Cin;
    long long ldc;
    int* status;
};

#ifdef KB_MX_PROFILE
__device__ unsigned long long kb_mx_prof_buf[32];
#define MX_T0() const long long _t0 = clock64()
#define MX_ACC(var) var += clock64() - _t0
#else
#define MX_T0()
#define MX_ACC(var)
#endif

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
// Arrival without memory ordering: what it publishes went to tensor memory (tcgen05.st, waited for and
// fenced), not to memory.  A release here would first wait for the arriving thread's outstanding
// global loads - the scale prefetch - which was measured to stretch the scale warps' loop tenfold.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
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
__device__ __forceinline__ void commit2(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}
__device__ __forceinline__ void mma_mx2(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
__device__ __forceinline__ void mma_mx(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
// Block-scaled instruction descriptor: e4m3 x e4m3 (format 0), K-major operands, UE8M0 scales;
// `step` selects the scale byte (K step within the K block) of both operands.
__device__ __forceinline__ uint32_t instr_desc_mx(int m, int n, int step) {
    uint32_t d = 0;
    d |= (uint32_t)(step & 3) << 4;                 // B scale id
    d |= (uint32_t)((n >> 3) & 0x3F) << 17;
    d |= 1u << 23;                                  // scale format: E8M0
    d |= (uint32_t)((m >> 4) & 0x1F) << 24;
    d |= (uint32_t)(step & 3) << 29;                // A scale id
    return d;
}
// fp32 power of two -> its exponent byte in all four bytes of a word
__device__ __forceinline__ uint32_t e8m0x4(float s) { return ((__float_as_uint(s) >> 23) & 0xFFu) * 0x01010101u; }

__device__ __forceinline__ uint32_t sf_slot_col(int slot) { return (uint32_t)((slot >> 1) * 256 + BN + (slot & 1) * 16); }

// The kernel body for both launch shapes; `rank` is the CTA's rank in its pair (0 when CTAS == 1).
template <int CTAS>
__device__ __forceinline__ void gemm_mxfp8_body(const CUtensorMap& tmA, const CUtensorMap& tmB, const MxParams& p) {
    constexpr int STAGES = Cfg<CTAS>::STAGES, B_STAGE = Cfg<CTAS>::B_STAGE, B_ROWS = Cfg<CTAS>::B_ROWS;
    constexpr int TILE_M = BM * CTAS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE + B_STAGE));
    uint64_t* full = bars;                               // [STAGES]   TMA -> MMA        (leader's copy is used)
    uint64_t* empty = bars + STAGES;                     // [STAGES]   MMA -> TMA        (per CTA)
    uint64_t* sf_full = bars + 2 * STAGES;               // [SF_SLOTS] scale warps -> MMA (leader's)
    uint64_t* sf_empty = bars + 2 * STAGES + SF_SLOTS;   // [SF_SLOTS] MMA -> scale warps (per CTA)
    uint64_t* acc_full = bars + 2 * STAGES + 2 * SF_SLOTS;          // [NBUF] MMA -> epilogue (per CTA)
    uint64_t* acc_empty = bars + 2 * STAGES + 2 * SF_SLOTS + NBUF;  // [NBUF] epilogue -> MMA (leader's)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * SF_SLOTS + 2 * NBUF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint8_t* epi_stage = smem + STAGES * (A_STAGE + B_STAGE) + 256;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = CTAS == 2 ? cluster_ctarank() : 0;
    const bool leader = rank == 0;
    const int worker = CTAS == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int nworkers = CTAS == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int tiles_m = (p.M + TILE_M - 1) / TILE_M, tiles_n = (p.N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int kblocks = p.K / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < SF_SLOTS; ++s) {
            tc::mbar_init(&sf_full[s], 4 * CTAS);
            tc::mbar_init(&sf_empty[s], 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            tc::mbar_init(&acc_full[b], 1);
            tc::mbar_init(&acc_empty[b], 4 * CTAS);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    if (warp == 1) {
        if (CTAS == 2) {
            tmem_alloc2(tmem_slot, 512);
            tmem_relinquish2();
        } else {
            tc::tmem_alloc(tmem_slot, 512);
            tc::tmem_relinquish();
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync();                       // the peer's barriers exist before anyone signals them
    tc::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    constexpr int GROUP_M = CTAS == 2 ? 8 : 16;

    auto coords = [&](int tile, int& tm, int& tn) {
        const int group = GROUP_M * tiles_n;
        const int g = tile / group;
        const int first_m = g * GROUP_M;
        const int gm = min(GROUP_M, tiles_m - first_m);
        const int t = tile - g * group;
        tm = first_m + t % gm;
        tn = t / gm;
    };
    // arrive on a barrier of the leader CTA / signal "MMAs so far are done" to a barrier in every CTA of the pair
    auto arrive_leader = [&](uint64_t* bar) {
        if (CTAS == 2) mbar_arrive_cluster(mapa(smem_u32(bar), 0));
        else tc::mbar_arrive(bar);
    };
    auto commit_all = [&](uint64_t* bar) {
        if (CTAS == 2) {
            commit2(mapa(smem_u32(bar), 0));
            commit2(mapa(smem_u32(bar), 1));
        } else {
            tc::tc_commit(bar);
        }
    };

    if (warp == 0) {
        if (lane == 0) {
            tc::prefetch_tmap(&tmA);
            tc::prefetch_tmap(&tmB);
            int stage = 0, issued = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long w_empty = 0;
            for (int tile = worker; tile < num_tiles && ok; tile += nworkers) {
                int tm, tn;
                coords(tile, tm, tn);
                const int m0 = tm * TILE_M + (int)rank * BM, n0 = tn * BN + (int)rank * B_ROWS;
                for (int kb = 0; kb < kblocks; ++kb) {
                    MX_T0();
                    const bool got = tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag);
                    MX_ACC(w_empty);
                    if (!got) {
                        atomicMax(p.status, (int)KB_TIMEOUT_TMA);
                        ok = false;
                        break;
                    }
                    if (CTAS == 2) {
                        const uint32_t full_leader = mapa(smem_u32(&full[stage]), 0);
                        if (leader) tc::mbar_expect_tx(&full[stage], 2 * (A_STAGE + B_STAGE));
                        tma_load_3d_pair(sA + stage * A_STAGE, &tmA, full_leader, kb * BK, m0, 0);
                        tma_load_3d_pair(sB + stage * B_STAGE, &tmB, full_leader, kb * BK, n0, 0);
                    } else {
                        tc::mbar_expect_tx(&full[stage], A_STAGE + B_STAGE);
                        tc::tma_load_3d(sA + stage * A_STAGE, &tmA, &full[stage], kb * BK, m0, 0);
                        tc::tma_load_3d(sB + stage * B_STAGE, &tmB, &full[stage], kb * BK, n0, 0);
                    }
                    ++issued;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
#ifdef KB_MX_PROFILE
            if (blockIdx.x < 2) kb_mx_prof_buf[blockIdx.x * 16 + 0] = w_empty;
#endif
            if (!ok && CTAS == 1) {
                // give the copies still in flight a moment to land before the CTA leaves
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
        if (lane == 0 && leader) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t it = 0;                         // K blocks issued so far: selects the scale slot
            uint32_t tcount = 0;
            bool ok = true;
            long long w_full = 0, w_sf = 0, w_acc = 0;
#ifdef KB_MX_PROFILE
            const long long t_begin = clock64();
#endif
            for (int tile = worker; tile < num_tiles && ok; tile += nworkers, ++tcount) {
                const int buf = tcount % NBUF;
                const uint32_t acc_phase = (tcount / NBUF) & 1;
                {
                    MX_T0();
                    const bool got = tc::mbar_wait(&acc_empty[buf], acc_phase ^ 1, abort_flag);
                    MX_ACC(w_acc);
                    if (!got) {
                        atomicMax(p.status, (int)KB_TIMEOUT_MMA);
                        break;
                    }
                }
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 256;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int slot = it % SF_SLOTS;
                    const uint32_t sphase = (it / SF_SLOTS) & 1;
                    bool got;
                    {
                        MX_T0();
                        got = tc::mbar_wait(&full[stage], phase, abort_flag);
                        MX_ACC(w_full);
                    }
                    if (got) {
                        MX_T0();
                        got = tc::mbar_wait(&sf_full[slot], sphase, abort_flag);
                        MX_ACC(w_sf);
                    }
                    if (!got) {
                        atomicMax(p.status, (int)KB_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    tc::tc_fence_after();
                    const uint32_t a_addr = smem_u32(sA + stage * A_STAGE);
                    const uint32_t b_addr = smem_u32(sB + stage * B_STAGE);
                    const uint32_t sfa = tmem_base + sf_slot_col(slot), sfb = sfa + 4;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k) {
                        const uint64_t ad = tc::smem_desc_sw128(a_addr + k * 32, 16, 1024);
                        const uint64_t bd = tc::smem_desc_sw128(b_addr + k * 32, 16, 1024);
                        if (CTAS == 2) mma_mx2(d_tmem, ad, bd, instr_desc_mx(TILE_M, BN, k), sfa, sfb, (kb | k) != 0);
                        else mma_mx(d_tmem, ad, bd, instr_desc_mx(TILE_M, BN, k), sfa, sfb, (kb | k) != 0);
                    }
                    commit_all(&empty[stage]);
                    commit_all(&sf_empty[slot]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) commit_all(&acc_full[buf]);
            }
#ifdef KB_MX_PROFILE
            if (blockIdx.x < 2) {
                kb_mx_prof_buf[blockIdx.x * 16 + 1] = w_full;
                kb_mx_prof_buf[blockIdx.x * 16 + 2] = w_sf;
                kb_mx_prof_buf[blockIdx.x * 16 + 3] = w_acc;
                kb_mx_prof_buf[blockIdx.x * 16 + 4] = clock64() - t_begin;
            }
#endif
        }
    } else if (warp < 6) {
        // ---- scale warps: one per TMEM lane quarter, all four write the same words
        const int quarter = warp & 3;
        uint32_t it = 0;
        bool ok = true;
        long long w_sfe = 0, w_body = 0;
        for (int tile = worker; tile < num_tiles && ok; tile += nworkers) {
            int tm, tn;
            coords(tile, tm, tn);
            const float* pa[4];
            const float* pb[8];
#pragma unroll
            for (int c = 0; c < 4; ++c) pa[c] = p.sa + min(tm * TILE_M + (int)rank * BM + 32 * c + lane, p.M - 1);
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const int n = tn * BN + 32 * g;
                pb[g] = p.sb + (p.b_gran == 1 ? min(n + lane, p.N - 1) : min(n, p.N - 1) / p.b_gran);
            }
            // scales are fetched two K blocks ahead of the one being written
            float cur[12], nx1[12], nx2[12];
            auto fetch = [&](int kb, float* dst) {
                const int kc = min(kb, kblocks - 1);
#pragma unroll
                for (int c = 0; c < 4; ++c) dst[c] = __ldg(pa[c] + (long long)kc * p.M);
#pragma unroll
                for (int g = 0; g < 8; ++g) dst[4 + g] = __ldg(pb[g] + (long long)kc * p.sb_ld);
            };
            fetch(0, cur);
            fetch(1, nx1);
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                fetch(kb + 2, nx2);
                const int slot = it % SF_SLOTS;
                const uint32_t sphase = (it / SF_SLOTS) & 1;
                bool got;
                {
                    MX_T0();
                    got = tc::mbar_wait(&sf_empty[slot], sphase ^ 1, abort_flag);
                    MX_ACC(w_sfe);
                }
                if (!got) {
                    if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                    ok = false;
                    break;
                }
                MX_T0();
                tc::tc_fence_after();
                uint32_t words[16];
#pragma unroll
                for (int j = 0; j < 12; ++j) words[j] = e8m0x4(cur[j]);
#pragma unroll
                for (int j = 12; j < 16; ++j) words[j] = 0x7F7F7F7Fu;
                tc::tmem_st16(tmem_base + sf_slot_col(slot) + ((uint32_t)(quarter * 32) << 16), words);
                tc::tmem_st_wait();
                tc::tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster_relaxed(CTAS == 2 ? mapa(smem_u32(&sf_full[slot]), 0)
                                                                     : smem_u32(&sf_full[slot]));
#pragma unroll
                for (int j = 0; j < 12; ++j) { cur[j] = nx1[j]; nx1[j] = nx2[j]; }
                MX_ACC(w_body);
            }
        }
#ifdef KB_MX_PROFILE
        if (blockIdx.x < 2 && warp == 2 && lane == 0) {
            kb_mx_prof_buf[blockIdx.x * 16 + 5] = w_sfe;
            kb_mx_prof_buf[blockIdx.x * 16 + 6] = w_body;
        }
#endif
    } else {
        // ---- epilogue warps
        const int quarter = warp & 3;
        uint8_t* stg = epi_stage + (warp - 6) * EPI_WARP_BYTES;
        uint32_t tcount = 0;
        for (int tile = worker; tile < num_tiles; tile += nworkers, ++tcount) {
            int tm, tn;
            coords(tile, tm, tn);
            const int buf = tcount % NBUF;
            const uint32_t acc_phase = (tcount / NBUF) & 1;
            if (!tc::mbar_wait(&acc_full[buf], acc_phase, abort_flag)) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                break;
            }
            tc::tc_fence_after();
            const int row0 = tm * TILE_M + (int)rank * BM + quarter * 32;
            const int row = row0 + lane;
            const uint32_t taddr = tmem_base + buf * 256 + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t acc[32];
                tc::tmem_ld32(taddr + c0, acc);
                tc::tmem_ld_wait();
                const int col = tn * BN + c0;
                if (col >= p.N) continue;                       // warp-uniform
                const int ncols = min(32, p.N - col);
                if (p.out_type == 2) {
                    if (row < p.M) {
                        float* dst = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col;
                        const float* cin = p.Cin ? reinterpret_cast<const float*>(p.Cin) + (long long)row * p.ldc + col : nullptr;
                        for (int j = 0; j < ncols; ++j)
                            dst[j] = p.alpha * __uint_as_float(acc[j]) + (cin ? p.beta * cin[j] : 0.f);
                    }
                    continue;
                }
                __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col;
                const __nv_bfloat16* cin =
                    p.Cin ? reinterpret_cast<const __nv_bfloat16*>(p.Cin) + (long long)row * p.ldc + col : nullptr;
                const bool vec = ncols == 32 && ((p.ldc | col) & 7) == 0;
                if (!vec) {
                    if (row < p.M)
                        for (int j = 0; j < ncols; ++j)
                            crow[j] = __float2bfloat16(p.alpha * __uint_as_float(acc[j]) +
                                                       (cin ? p.beta * __bfloat162float(cin[j]) : 0.f));
                    continue;
                }
                // 32 x 32 chunk through shared memory: a lane packs its row, then the warp stores
                // 64-byte row segments (whole sectors) instead of 32 scattered 16-byte pieces
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = p.alpha * __uint_as_float(acc[8 * j + i]);
                    if (cin && row < p.M) {
                        float ci[8];
                        unpack8(ld8(cin + 8 * j), ci);
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] += p.beta * ci[i];
                    }
                    const bf16x8 o = pack8(v);
                    *reinterpret_cast<uint4*>(stg + lane * EPI_PITCH + j * 16) = *reinterpret_cast<const uint4*>(&o);
                }
                __syncwarp();
                const int seg = lane & 3;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = i * 8 + (lane >> 2);
                    const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * EPI_PITCH + seg * 16);
                    if (row0 + rr < p.M)
                        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)(row0 + rr) * p.ldc + col + seg * 8) = v;
                }
                __syncwarp();
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_leader(&acc_empty[buf]);
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync();                       // no remote arrival may target a CTA that has left
    if (warp == 1) {
        tc::tc_fence_after();
        if (CTAS == 2) tmem_dealloc2(tmem_base, 512);
        else tc::tmem_dealloc(tmem_base, 512);
    }
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const MxParams p) {
    gemm_mxfp8_body<1>(tmA, tmB, p);
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_mxfp8_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const MxParams p) {
    gemm_mxfp8_body<2>(tmA, tmB, p);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_mx() {
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
// 8-bit matrix [rows, cols], cols contiguous, row stride ld bytes.
int make_tmap8_mx(CUtensorMap* m, const void* base, long long cols, long long rows, long long ld, int box_cols,
                  int box_rows) {
    EncodeTiledFn enc = get_encode_mx();
    if (!enc) return 100;
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, 1};
    cuuint64_t strides[2] = {(cuuint64_t)ld, (cuuint64_t)(rows * ld)};
    cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 200 + (int)r;
}

}  // namespace

#ifdef KB_MX_PROFILE
// Wait-time counters (clock cycles) of CTA 0 and 1 of the last launch: [cta][0] producer on empty, [1] MMA on
// full, [2] MMA on scales, [3] MMA on accumulator, [4] MMA thread total, [5] scale warp on sf_empty, [6] its body.
KB_API int kb_mx_prof_read(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, kb_mx_prof_buf, sizeof(unsigned long long) * 32) == cudaSuccess ? 0 : 1;
}
#endif

// Same operands as kb_gemm_fp8; every entry of sa and sb must be a power of two (the quantisers'
// `pow2` mode).  K a multiple of 128; b_gran 128 or 1.  `pair`: 1 = SM-pair kernel (256 x 224 tiles),
// 0 = one CTA per 128 x 224 tile, -1 = the pair kernel when the product has at least one pair tile
// per SM pair.
KB_API int kb_gemm_mxfp8(const void* A, const void* B, const float* sa, const float* sb, void* C, const void* Cin,
                         int M, int N, int K, long long lda, long long ldb, long long ldc, int b_gran, int sb_ld,
                         int out_type, float alpha, float beta, int* status, int pair, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0 || (K % BK) != 0) return 5;
    if (b_gran != 1 && b_gran != 128) return 5;
    if (out_type != 1 && out_type != 2) return 5;
    if ((lda & 15) || (ldb & 15) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return 6;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles_n = (N + BN - 1) / BN;
    const int pair_tiles = ((M + 2 * BM - 1) / (2 * BM)) * tiles_n;
    const bool use_pair = pair == 1;
    static bool attr_flags[64] = {};
    bool* attr_set_p = kb_device_flag(attr_flags);
    if (!attr_set_p) return 7;
    if (!*attr_set_p) {
        if (cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<1>::SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_mxfp8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<2>::SMEM) != cudaSuccess)
            return 7;
        *attr_set_p = true;
    }
    CUtensorMap tmA, tmB;
    int r = make_tmap8_mx(&tmA, A, K, M, lda, BK, BM);
    if (r) return r;
    r = make_tmap8_mx(&tmB, B, K, N, ldb, BK, use_pair ? Cfg<2>::B_ROWS : Cfg<1>::B_ROWS);
    if (r) return r;
    MxParams p;
    memset(&p, 0, sizeof(p));
    p.M = M; p.N = N; p.K = K; p.sa = sa; p.sb = sb; p.b_gran = b_gran; p.sb_ld = sb_ld; p.out_type = out_type;
    p.alpha = alpha; p.beta = beta; p.C = C; p.Cin = Cin; p.ldc = ldc; p.status = status;
    if (use_pair) {
        const int pairs = pair_tiles < sms / 2 ? pair_tiles : sms / 2;
        gemm_mxfp8_pair_kernel<<<2 * pairs, THREADS, Cfg<2>::SMEM, st>>>(tmA, tmB, p);
    } else {
        const int tiles = ((M + BM - 1) / BM) * tiles_n;
        gemm_mxfp8_kernel<<<tiles < sms ? tiles : sms, THREADS, Cfg<1>::SMEM, st>>>(tmA, tmB, p);
    }
    return kb_launch_status();
}
