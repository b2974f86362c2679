// Causal GQA flash-attention backward for sm_100a (head_dim 64 or 128, bf16, fixed-length
// batches).  Three kernels, no atomics, deterministic:
//
//   attn_dprep   D[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]                       (one warp per row)
//   attn_dq      one CTA per (query tile i, head): for every key tile j <= i
//                  S = Q_i K_j^T, dP = dO_i V_j^T           tcgen05.mma, operands in shared memory
//                  dS = P o (dP - D) * scale, P = 2^(S*c - lse)   thread = query row, half the columns
//                  dQ_i += dS K_j                           dS read from tensor memory (packed bf16)
//   attn_dkdv    one CTA per (key tile j, key/value head): for every query head of the group and
//                every query tile i >= j, in the transposed frame (thread = key row)
//                  S^T = K_j Q_i^T, dP^T = V_j dO_i^T
//                  dV_j += P^T dO_i, dK_j += dS^T Q_i       both with A read from tensor memory
//                so dK/dV of a key/value head are summed over its query heads inside the CTA.
// The score tile is recomputed in both kernels (7 tile products per (i, j) instead of 5); in
// exchange dQ needs no fp32 atomics, no fp32 staging buffer and no conversion pass.
//
// Tensor memory (512 columns) per CTA:
//   attn_dq    S[0] | S[1] | dP | dQ        dS(j) overwrites the first 16 columns of each quarter of S[j&1]
//   attn_dkdv  S^T  | dP^T | dV | dK        P^T and dS^T overwrite their own score tiles the same way
// Each of the four compute warpgroups handles 32 of a tile's 128 columns and writes its packed
// result at the start of its own quarter, so no warpgroup overwrites scores another has not read yet.
// Every wait is bounded (status word on timeout).
#include "attn_common.cuh"

namespace {

using namespace attn;

constexpr int BWD_THREADS = 576;                   // 16 compute warps, MMA warp, TMA warp
constexpr int EMU = 1;                             // of every 4 pairs of exponentials, this many run on the FMA pipe

struct BwdParams {
    int B, T, H, KV;
    float scale, scale_log2;
    const float* lse;                              // [B, H, T] natural log
    float* dsum;                                   // [B, H, T] D = rowsum(dO o O)
    int q_col0, k_col0, v_col0, do_col0;           // first column of head 0 inside each operand's rows
    __nv_bfloat16 *dq, *dk, *dv;                   // token-major outputs
    long long dq_stride, dk_stride, dv_stride;     // elements between tokens
    int n_tiles;                                   // ceil(T / 128)
    int* status;
};

#define KB_FAIL(code)                                  \
    {                                                  \
        atomicMax(p.status, (int)(code));              \
        break;                                         \
    }

// ---------------------------------------------------------------------------------- D = rowsum(dO o O)
template <int HD>
__global__ void __launch_bounds__(256)
attn_dprep_kernel(const __nv_bfloat16* __restrict__ o, long long o_stride, const __nv_bfloat16* __restrict__ dout,
                  long long do_stride, int do_col0, float* __restrict__ dsum, int B, int T, int H) {
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= (long long)B * T * H) return;
    const int head = (int)(w % H);
    const long long row = w / H;
    const int b = (int)(row / T), t = (int)(row % T);
    constexpr int E = HD / 32;
    const __nv_bfloat16* po = o + row * o_stride + head * HD + lane * E;
    const __nv_bfloat16* pd = dout + row * do_stride + do_col0 + head * HD + lane * E;
    float acc = 0.f;
    if constexpr (E == 4) {
        const uint2 a = *reinterpret_cast<const uint2*>(po), d = *reinterpret_cast<const uint2*>(pd);
        const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
        const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
        const float2 d0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d.x));
        const float2 d1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d.y));
        acc = a0.x * d0.x + a0.y * d0.y + a1.x * d1.x + a1.y * d1.y;
    } else {
        const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(po));
        const float2 d0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pd));
        acc = a0.x * d0.x + a0.y * d0.y;
    }
    acc = warp_sum(acc);
    if (lane == 0) dsum[((long long)b * H + head) * T + t] = acc;
}

// 32 scores -> 16 pairs of probabilities 2^(s*c - lse2).  `nl` holds -lse2: per column (shared
// memory, PER_COLUMN) or one value for the row.
template <bool PER_COLUMN>
__device__ __forceinline__ void probs32(const float* s, float scale_log2, const float* nl_cols, float nl_row,
                                        float2* pv) {
    const float2 sc2 = make_float2(scale_log2, scale_log2);
#pragma unroll
    for (int c = 0; c < 32; c += 2) {
        const float2 nl = PER_COLUMN ? *reinterpret_cast<const float2*>(nl_cols + c) : make_float2(nl_row, nl_row);
        pv[c >> 1] = exp2_pair<EMU>(__ffma2_rn(make_float2(s[c], s[c + 1]), sc2, nl), c >> 1);
    }
}

// ---------------------------------------------------------------------------------- dQ
constexpr int DQ_KST = 3, DQ_VST = 2;

template <int HD>
constexpr int dq_smem_bytes() {
    return (2 + DQ_KST + DQ_VST) * Tile<HD>::BYTES + 1024 + 256;
}

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const BwdParams p) {
    constexpr int TB = Tile<HD>::BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sDO = smem + TB;
    uint8_t* sK = smem + 2 * TB;
    uint8_t* sV = sK + DQ_KST * TB;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + DQ_VST * TB);
    uint64_t* qdo_full = bars;
    uint64_t* k_full = bars + 1;                   // [DQ_KST]
    uint64_t* k_empty = k_full + DQ_KST;
    uint64_t* v_full = k_empty + DQ_KST;           // [DQ_VST]
    uint64_t* v_empty = v_full + DQ_VST;
    uint64_t* s_full = v_empty + DQ_VST;           // [2] one per score buffer
    uint64_t* dp_full = s_full + 2;
    uint64_t* ds_ready = dp_full + 1;
    uint64_t* dq_done = ds_ready + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int HB = p.H * p.B;
    const int qt = p.n_tiles - 1 - (int)(blockIdx.x / HB);        // heavy tiles first
    const int hb = blockIdx.x % HB;
    const int head = hb % p.H, b = hb / p.H;
    const int kvh = head / (p.H / p.KV);
    const int seq_row0 = b * p.T;
    const int n = qt + 1;

    if (threadIdx.x == 0) {
        tc::mbar_init(qdo_full, 1);
        for (int i = 0; i < DQ_KST; ++i) { tc::mbar_init(k_full + i, 1); tc::mbar_init(k_empty + i, 1); }
        for (int i = 0; i < DQ_VST; ++i) { tc::mbar_init(v_full + i, 1); tc::mbar_init(v_empty + i, 1); }
        tc::mbar_init(s_full + 0, 1);
        tc::mbar_init(s_full + 1, 1);
        tc::mbar_init(dp_full, 1);
        tc::mbar_init(ds_ready, 16);
        tc::mbar_init(dq_done, 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    if (warp == 16) {
        tc::tmem_alloc(tmem_slot, 512);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem0 = *tmem_slot;
    const uint32_t tm_dp = tmem0 + 256, tm_dq = tmem0 + 384;

    if (warp == 17) {
        // ------------------------------------------------------------ TMA
        if (lane == 0) {
            tc::prefetch_tmap(&tmQ);
            tc::prefetch_tmap(&tmK);
            tc::prefetch_tmap(&tmV);
            tc::prefetch_tmap(&tmDO);
            const int kx = p.k_col0 + kvh * HD, vx = p.v_col0 + kvh * HD;
            tc::mbar_expect_tx(qdo_full, 2 * TB);
            load_tile<HD>(sQ, &tmQ, qdo_full, p.q_col0 + head * HD, seq_row0 + qt * BT);
            load_tile<HD>(sDO, &tmDO, qdo_full, p.do_col0 + head * HD, seq_row0 + qt * BT);
            for (int j = 0; j < n; ++j) {
                const int ks = j % DQ_KST, vs = j % DQ_VST;
                if (!tc::mbar_wait(k_empty + ks, ((j / DQ_KST) & 1) ^ 1, abort_flag)) KB_FAIL(KB_TIMEOUT_TMA)
                tc::mbar_expect_tx(k_full + ks, TB);
                load_tile<HD>(sK + ks * TB, &tmK, k_full + ks, kx, seq_row0 + j * BT);
                if (!tc::mbar_wait(v_empty + vs, ((j / DQ_VST) & 1) ^ 1, abort_flag)) KB_FAIL(KB_TIMEOUT_TMA)
                tc::mbar_expect_tx(v_full + vs, TB);
                load_tile<HD>(sV + vs * TB, &tmV, v_full + vs, vx, seq_row0 + j * BT);
            }
        }
    } else if (warp == 16) {
        // ------------------------------------------------------------ MMA issue (one thread)
        if (lane == 0) {
            const uint32_t idesc_s = tc::instr_desc_f16(BT, BT, 1, 1, 0, 0);
            const uint32_t idesc_q = tc::instr_desc_f16(BT, HD, 1, 1, 0, 1);
            const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sDO), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
            do {
                if (!tc::mbar_wait(qdo_full, 0, abort_flag) || !tc::mbar_wait(k_full, 0, abort_flag)) KB_FAIL(KB_TIMEOUT_TMA)
                tc::tc_fence_after();
                mma_nt_tiles<HD>(tmem0, q_addr, k_addr, idesc_s);
                tc::tc_commit(s_full + 0);
                if (!tc::mbar_wait(v_full, 0, abort_flag)) KB_FAIL(KB_TIMEOUT_TMA)
                tc::tc_fence_after();
                mma_nt_tiles<HD>(tm_dp, do_addr, v_addr, idesc_s);
                tc::tc_commit(dp_full);
                tc::tc_commit(v_empty + 0);
                if (n > 1) {
                    if (!tc::mbar_wait(k_full + 1, 0, abort_flag)) KB_FAIL(KB_TIMEOUT_TMA)
                    tc::tc_fence_after();
                    mma_nt_tiles<HD>(tmem0 + 128, q_addr, k_addr + TB, idesc_s);
                    tc::tc_commit(s_full + 1);
                }
                bool ok = true;
                for (int j = 0; j < n; ++j) {
                    if (!tc::mbar_wait(ds_ready, j & 1, abort_flag)) { atomicMax(p.status, (int)KB_TIMEOUT_MMA); ok = false; break; }
                    tc::tc_fence_after();
                    if (j + 1 < n) {
                        const int vs = (j + 1) % DQ_VST;
                        if (!tc::mbar_wait(v_full + vs, ((j + 1) / DQ_VST) & 1, abort_flag)) { atomicMax(p.status, (int)KB_TIMEOUT_TMA); ok = false; break; }
                        tc::tc_fence_after();
                        mma_nt_tiles<HD>(tm_dp, do_addr, v_addr + vs * TB, idesc_s);
                        tc::tc_commit(dp_full);
                        tc::tc_commit(v_empty + vs);
                    }
                    const int ks = j % DQ_KST;
                    mma_ts_tile<HD, true>(tm_dq, tmem0 + (j & 1) * 128, k_addr + ks * TB, idesc_q, j != 0);
                    tc::tc_commit(k_empty + ks);
                    if (j + 2 < n) {
                        const int k2 = (j + 2) % DQ_KST;
                        if (!tc::mbar_wait(k_full + k2, ((j + 2) / DQ_KST) & 1, abort_flag)) { atomicMax(p.status, (int)KB_TIMEOUT_TMA); ok = false; break; }
                        tc::tc_fence_after();
                        mma_nt_tiles<HD>(tmem0 + (j & 1) * 128, q_addr, k_addr + k2 * TB, idesc_s);
                        tc::tc_commit(s_full + (j & 1));
                    }
                }
                if (ok) tc::tc_commit(dq_done);
            } while (false);
        }
    } else if (warp < 16) {
        // ------------------------------------------------------------ compute: thread = (query row, column quarter)
        const int qd = warp >> 2;
        const int r = (warp & 3) * 32 + lane;
        const uint32_t lane_base = ((uint32_t)((warp & 3) * 32) << 16);
        const int qrow = qt * BT + r;
        const bool valid = qrow < p.T;
        const long long sidx = ((long long)b * p.H + head) * p.T + qrow;
        const float nl = valid ? -p.lse[sidx] * LOG2E : -INFINITY;
        // dS leaves as truncated bf16: its rounding bias rides on the scale constants (pack_bf16_trunc)
        const float nds = valid ? -p.dsum[sidx] * p.scale * TRUNC_BIAS : 0.f;      // -D * scale
        const float2 scale2 = make_float2(p.scale * TRUNC_BIAS, p.scale * TRUNC_BIAS), nds2 = make_float2(nds, nds);
        bool ok = true;
        float2 pv[16];                                                // probabilities of the tile in flight
        // P(j) only needs the scores, so it is computed while the tensor pipe still works on dP(j)
        auto compute_p = [&](int j) -> bool {
            if (!tc::mbar_wait(s_full + (j & 1), (j >> 1) & 1, abort_flag)) return false;
            tc::tc_fence_after();
            float s[32];
            tc::tmem_ld32(tmem0 + (j & 1) * 128 + qd * 32 + lane_base, reinterpret_cast<uint32_t*>(s));
            tc::tmem_ld_wait();
            probs32<false>(s, p.scale_log2, nullptr, nl, pv);
            if (j == qt) {                                            // diagonal tile: keys after the query get 0
                const int cmax = r - qd * 32;
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    pv[c >> 1].x = c <= cmax ? pv[c >> 1].x : 0.f;
                    pv[c >> 1].y = c + 1 <= cmax ? pv[c >> 1].y : 0.f;
                }
            }
            return true;
        };
        ok = compute_p(0);
        if (!ok && lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
        for (int j = 0; j < n && ok; ++j) {
            if (!tc::mbar_wait(dp_full, j & 1, abort_flag)) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                ok = false;
                break;
            }
            tc::tc_fence_after();
            float dp[32];
            tc::tmem_ld32(tm_dp + qd * 32 + lane_base, reinterpret_cast<uint32_t*>(dp));
            tc::tmem_ld_wait();
            uint32_t pk[16];
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
                const float2 d = __fmul2_rn(pv[c >> 1], __ffma2_rn(make_float2(dp[c], dp[c + 1]), scale2, nds2));
                pk[c >> 1] = pack_bf16_trunc(d.x, d.y);
            }
            tc::tmem_st16(tmem0 + (j & 1) * 128 + qd * 32 + lane_base, pk);
            tc::tmem_st_wait();
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(ds_ready);
            if (j + 1 < n && !compute_p(j + 1)) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                ok = false;
            }
        }
        if (ok) {
            if (tc::mbar_wait(dq_done, 0, abort_flag)) {
                tc::tc_fence_after();
                constexpr int CW = HD / 4;                            // output columns per thread
                __nv_bfloat16* dst = p.dq + (size_t)(seq_row0 + qrow) * p.dq_stride + head * HD + qd * CW;
                uint32_t o[CW];
                if constexpr (CW == 32) tc::tmem_ld32(tm_dq + qd * CW + lane_base, o);
                else tc::tmem_ld16(tm_dq + qd * CW + lane_base, o);
                tc::tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < CW; i += 8) st8(dst + i, pack8(reinterpret_cast<const float*>(o + i)));
                }
            } else if (lane == 0) {
                atomicMax(p.status, (int)KB_TIMEOUT_EPI);
            }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 16) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem0, 512);
    }
}

// ---------------------------------------------------------------------------------- dK, dV
// The query and output-gradient tiles of consecutive pairs share one ring of RING slots, filled
// in the order Q(0), dO(0), Q(1), dO(1), ...: load number u goes to slot u % RING.  With five
// slots a tile is requested more than a pair ahead of its first use, which keeps the TMA latency
// off the per-pair critical path (a slot is held from the tile's first product to its last).
constexpr int RING = 5, STAT_RING = 2;

template <int HD>
constexpr int dkdv_smem_bytes() {
    return (2 + RING) * Tile<HD>::BYTES + STAT_RING * 2 * BT * 4 + 256;
}

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const BwdParams p) {
    constexpr int TB = Tile<HD>::BYTES;
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023) {                   // the swizzled tiles need 1024-byte aligned slots
        if (threadIdx.x == 0) atomicMax(p.status, (int)KB_BAD_ARG);
        return;
    }
    uint8_t* sK = smem;
    uint8_t* sV = smem + TB;
    uint8_t* sRing = smem + 2 * TB;                // [RING]
    float* sStat = reinterpret_cast<float*>(sRing + RING * TB);    // [STAT_RING][2][128]: -lse * log2(e), -D * scale
    uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + STAT_RING * 2 * BT);
    uint64_t* kv_full = bars;
    uint64_t* full = bars + 1;                     // [RING]
    uint64_t* empty = full + RING;                 // [RING]
    uint64_t* stat_full = empty + RING;            // [STAT_RING]
    uint64_t* stat_empty = stat_full + STAT_RING;
    uint64_t* s_full = stat_empty + STAT_RING;
    uint64_t* dp_full = s_full + 1;
    uint64_t* p_ready = dp_full + 1;
    uint64_t* ds_ready = p_ready + 1;
    uint64_t* acc_done = ds_ready + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int GB = p.KV * p.B;
    const int jt = (int)(blockIdx.x / GB);                        // key tile; early tiles have the most work
    const int gb = blockIdx.x % GB;
    const int g = gb % p.KV, b = gb / p.KV;
    const int G = p.H / p.KV;
    const int seq_row0 = b * p.T;
    const int nqi = p.n_tiles - jt;                               // query tiles at or after this key tile
    const int np = G * nqi;                                       // (head, query tile) pairs

    if (threadIdx.x == 0) {
        tc::mbar_init(kv_full, 1);
        for (int i = 0; i < RING; ++i) {
            tc::mbar_init(full + i, 1);
            tc::mbar_init(empty + i, 1);
        }
        for (int i = 0; i < STAT_RING; ++i) {
            tc::mbar_init(stat_full + i, 1);
            tc::mbar_init(stat_empty + i, 16);
        }
        tc::mbar_init(s_full, 1);
        tc::mbar_init(dp_full, 1);
        tc::mbar_init(p_ready, 16);
        tc::mbar_init(ds_ready, 16);
        tc::mbar_init(acc_done, 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    if (warp == 16) {
        tc::tmem_alloc(tmem_slot, 512);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem0 = *tmem_slot;
    const uint32_t tm_dp = tmem0 + 128, tm_dv = tmem0 + 256, tm_dk = tmem0 + 384;

    if (warp == 17) {
        // ------------------------------------------------------------ TMA (lane 0) + row statistics (all lanes)
        if (lane == 0) {
            tc::prefetch_tmap(&tmQ);
            tc::prefetch_tmap(&tmK);
            tc::prefetch_tmap(&tmV);
            tc::prefetch_tmap(&tmDO);
            tc::mbar_expect_tx(kv_full, 2 * TB);
            load_tile<HD>(sK, &tmK, kv_full, p.k_col0 + g * HD, seq_row0 + jt * BT);
            load_tile<HD>(sV, &tmV, kv_full, p.v_col0 + g * HD, seq_row0 + jt * BT);
        }
        for (int t = 0; t < np; ++t) {
            const int head = g * G + t / nqi, qt = jt + t % nqi;
            int ok = 1;
            if (lane == 0) {
#pragma unroll
                for (int w = 0; w < 2 && ok; ++w) {                   // w = 0: Q(t), w = 1: dO(t)
                    const int u = 2 * t + w, sl = u % RING;
                    if (!tc::mbar_wait(empty + sl, ((u / RING) & 1) ^ 1, abort_flag)) { ok = 0; break; }
                    tc::mbar_expect_tx(full + sl, TB);
                    load_tile<HD>(sRing + sl * TB, w ? &tmDO : &tmQ, full + sl,
                                  (w ? p.do_col0 : p.q_col0) + head * HD, seq_row0 + qt * BT);
                }
            }
            const int st = t % STAT_RING;
            if (ok && !tc::mbar_wait(stat_empty + st, ((t / STAT_RING) & 1) ^ 1, abort_flag)) ok = 0;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_TMA);
                break;
            }
            float* dst = sStat + st * 2 * BT;
            const long long base = ((long long)b * p.H + head) * p.T;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int c = lane + e * 32, qrow = qt * BT + c;
                const bool valid = qrow < p.T;
                // both tables carry the truncation bias of the packed operands they feed (pack_bf16_trunc)
                dst[c] = valid ? TRUNC_BIAS_LOG2 - p.lse[base + qrow] * LOG2E : -INFINITY;
                dst[BT + c] = valid ? -p.dsum[base + qrow] * p.scale * TRUNC_BIAS : 0.f;
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(stat_full + st);
        }
    } else if (warp == 16) {
        // ------------------------------------------------------------ MMA issue (one thread)
        if (lane == 0) {
            const uint32_t idesc_s = tc::instr_desc_f16(BT, BT, 1, 1, 0, 0);
            const uint32_t idesc_a = tc::instr_desc_f16(BT, HD, 1, 1, 0, 1);
            const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), ring = smem_u32(sRing);
            auto slot_addr = [&](int u) { return ring + (u % RING) * TB; };
            auto wait_full = [&](int u) { return tc::mbar_wait(full + u % RING, (u / RING) & 1, abort_flag); };
            do {
                if (!tc::mbar_wait(kv_full, 0, abort_flag) || !wait_full(0)) KB_FAIL(KB_TIMEOUT_TMA)
                tc::tc_fence_after();
                mma_nt_tiles<HD>(tmem0, k_addr, slot_addr(0), idesc_s);
                tc::tc_commit(s_full);
                if (!wait_full(1)) KB_FAIL(KB_TIMEOUT_TMA)
                tc::tc_fence_after();
                mma_nt_tiles<HD>(tm_dp, v_addr, slot_addr(1), idesc_s);
                tc::tc_commit(dp_full);
                bool ok = true;
                for (int t = 0; t < np; ++t) {
                    const int uq = 2 * t, ud = 2 * t + 1;
                    if (!tc::mbar_wait(p_ready, t & 1, abort_flag)) { atomicMax(p.status, (int)KB_TIMEOUT_MMA); ok = false; break; }
                    tc::tc_fence_after();
                    mma_ts_tile<HD, true>(tm_dv, tmem0, slot_addr(ud), idesc_a, t != 0);
                    tc::tc_commit(empty + ud % RING);
                    if (t + 1 < np) {
                        if (!wait_full(uq + 2)) { atomicMax(p.status, (int)KB_TIMEOUT_TMA); ok = false; break; }
                        tc::tc_fence_after();
                        mma_nt_tiles<HD>(tmem0, k_addr, slot_addr(uq + 2), idesc_s);
                        tc::tc_commit(s_full);
                    }
                    if (!tc::mbar_wait(ds_ready, t & 1, abort_flag)) { atomicMax(p.status, (int)KB_TIMEOUT_MMA); ok = false; break; }
                    tc::tc_fence_after();
                    mma_ts_tile<HD, true>(tm_dk, tm_dp, slot_addr(uq), idesc_a, t != 0);
                    tc::tc_commit(empty + uq % RING);
                    if (t + 1 < np) {
                        if (!wait_full(ud + 2)) { atomicMax(p.status, (int)KB_TIMEOUT_TMA); ok = false; break; }
                        tc::tc_fence_after();
                        mma_nt_tiles<HD>(tm_dp, v_addr, slot_addr(ud + 2), idesc_s);
                        tc::tc_commit(dp_full);
                    }
                }
                if (ok) tc::tc_commit(acc_done);
            } while (false);
        }
    } else if (warp < 16) {
        // ------------------------------------------------------------ compute: thread = (key row, column quarter)
        const int qd = warp >> 2;
        const int r = (warp & 3) * 32 + lane;
        const uint32_t lane_base = ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t tm_s = tmem0 + qd * 32 + lane_base, tm_d = tm_dp + qd * 32 + lane_base;
        const float2 scale2 = make_float2(p.scale * TRUNC_BIAS, p.scale * TRUNC_BIAS);
        bool ok = true;
        for (int t = 0; t < np; ++t) {
            const int st = t % STAT_RING;
            const bool diag = t % nqi == 0;
            const float* nl = sStat + st * 2 * BT + qd * 32;          // -lse * log2(e) of this quarter's query positions
            const float* nds = nl + BT;                               // -D * scale
            if (!tc::mbar_wait(stat_full + st, (t / STAT_RING) & 1, abort_flag) || !tc::mbar_wait(s_full, t & 1, abort_flag)) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                ok = false;
                break;
            }
            tc::tc_fence_after();
            uint32_t pk[16];
            {
                float s[32];
                float2 pv[16];
                tc::tmem_ld32(tm_s, reinterpret_cast<uint32_t*>(s));
                tc::tmem_ld_wait();
                probs32<true>(s, p.scale_log2, nl, 0.f, pv);
                if (diag) {                                           // keep query positions at or after this key row
                    const int cmin = r - qd * 32;
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        pv[c >> 1].x = c >= cmin ? pv[c >> 1].x : 0.f;
                        pv[c >> 1].y = c + 1 >= cmin ? pv[c >> 1].y : 0.f;
                    }
                }
#pragma unroll
                for (int c = 0; c < 16; ++c) pk[c] = pack_bf16_trunc(pv[c].x, pv[c].y);
            }
            tc::tmem_st16(tm_s, pk);
            tc::tmem_st_wait();
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(p_ready);
            if (!tc::mbar_wait(dp_full, t & 1, abort_flag)) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                ok = false;
                break;
            }
            tc::tc_fence_after();
            {
                float dp[32];
                tc::tmem_ld32(tm_d, reinterpret_cast<uint32_t*>(dp));
                tc::tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const float2 pv = make_float2(__uint_as_float(pk[c >> 1] << 16), __uint_as_float(pk[c >> 1] & 0xffff0000u));
                    const float2 d = __fmul2_rn(pv, __ffma2_rn(make_float2(dp[c], dp[c + 1]), scale2,
                                                               *reinterpret_cast<const float2*>(nds + c)));
                    pk[c >> 1] = pack_bf16_trunc(d.x, d.y);
                }
            }
            tc::tmem_st16(tm_d, pk);
            tc::tmem_st_wait();
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                tc::mbar_arrive(ds_ready);
                tc::mbar_arrive(stat_empty + st);
            }
        }
        if (ok) {
            if (tc::mbar_wait(acc_done, 0, abort_flag)) {
                tc::tc_fence_after();
                constexpr int CW = HD / 4;                            // output columns per thread
                const int krow = jt * BT + r;
                const bool valid = krow < p.T;
                __nv_bfloat16* dv = p.dv + (size_t)(seq_row0 + krow) * p.dv_stride + g * HD + qd * CW;
                __nv_bfloat16* dk = p.dk + (size_t)(seq_row0 + krow) * p.dk_stride + g * HD + qd * CW;
                uint32_t o[CW], o2[CW];
                if constexpr (CW == 32) {
                    tc::tmem_ld32(tm_dv + qd * CW + lane_base, o);
                    tc::tmem_ld32(tm_dk + qd * CW + lane_base, o2);
                } else {
                    tc::tmem_ld16(tm_dv + qd * CW + lane_base, o);
                    tc::tmem_ld16(tm_dk + qd * CW + lane_base, o2);
                }
                tc::tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < CW; i += 8) {
                        st8(dv + i, pack8(reinterpret_cast<const float*>(o + i)));
                        st8(dk + i, pack8(reinterpret_cast<const float*>(o2 + i)));
                    }
                }
            } else if (lane == 0) {
                atomicMax(p.status, (int)KB_TIMEOUT_EPI);
            }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 16) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem0, 512);
    }
}

template <typename K>
int ensure_smem(K kernel, int bytes, bool* done_for_device) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 7;
    if (!done_for_device[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return 7;
        done_for_device[dev] = true;
    }
    return 0;
}

template <int HD>
int launch_bwd(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmDO,
               const BwdParams& p, const void* o, long long o_stride, const void* dout, long long do_stride, int which,
               cudaStream_t st) {
    static bool attr_dq[64] = {}, attr_kv[64] = {};
    int r = ensure_smem(attn_dq_kernel<HD>, dq_smem_bytes<HD>(), attr_dq);
    if (r) return r;
    r = ensure_smem(attn_dkdv_kernel<HD>, dkdv_smem_bytes<HD>(), attr_kv);
    if (r) return r;
    const long long rows = (long long)p.B * p.T * p.H;
    attn_dprep_kernel<HD><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(
        (const __nv_bfloat16*)o, o_stride, (const __nv_bfloat16*)dout, do_stride, p.do_col0, p.dsum, p.B, p.T, p.H);
    if (cudaGetLastError() != cudaSuccess) return 8;
    if (which & 1) {
        attn_dkdv_kernel<HD><<<p.n_tiles * p.KV * p.B, BWD_THREADS, dkdv_smem_bytes<HD>(), st>>>(tmQ, tmK, tmV, tmDO, p);
        if (cudaGetLastError() != cudaSuccess) return 8;
    }
    if (which & 2) {
        attn_dq_kernel<HD><<<p.n_tiles * p.H * p.B, BWD_THREADS, dq_smem_bytes<HD>(), st>>>(tmQ, tmK, tmV, tmDO, p);
        if (cudaGetLastError() != cudaSuccess) return 8;
    }
    return 0;
}

}  // namespace

// Gradients of causal GQA attention.  q/k/v/dout: token-major matrices [B*T, *] whose rows hold the
// heads side by side (row strides in elements; *_col0 = column of head 0); o[B*T, H*hd] with
// `o_stride`; lse[B,H,T] from the forward; dsum[B,H,T] fp32 workspace.  dq/dk/dv point at head 0 of
// the first token of their destination (any token stride), so the results land directly inside
// fused gradient buffers.  `which`: bit 0 = dK and dV, bit 1 = dQ (3 = all).
KB_API int kb_flash_bwd(const void* q, long long q_stride, int q_cols, int q_col0, const void* k, long long k_stride,
                        int k_cols, int k_col0, const void* v, long long v_stride, int v_cols, int v_col0,
                        const void* o, long long o_stride, const void* dout, long long do_stride, int do_cols,
                        int do_col0, const float* lse, float* dsum, void* dq, long long dq_stride, void* dk,
                        long long dk_stride, void* dv, long long dv_stride, int B, int T, int H, int KV, int hd,
                        float scale, int which, int* status, cudaStream_t st) {
    if ((hd != 128 && hd != 64) || T < 1 || B < 1 || KV < 1 || H % KV != 0) return 5;
    if (!operand_ok(q, q_stride, q_col0) || !operand_ok(k, k_stride, k_col0) || !operand_ok(v, v_stride, v_col0) ||
        !operand_ok(dout, do_stride, do_col0))
        return 6;
    if (((uintptr_t)o & 7) || (o_stride & 3)) return 6;
    if (((uintptr_t)dq & 15) || ((uintptr_t)dk & 15) || ((uintptr_t)dv & 15) || (dq_stride & 7) || (dk_stride & 7) ||
        (dv_stride & 7))
        return 6;
    const long long rows = (long long)B * T;
    CUtensorMap tmQ, tmK, tmV, tmDO;
    int r = make_rows_tmap(&tmQ, q, rows, q_cols, q_stride);
    if (r) return r;
    r = make_rows_tmap(&tmK, k, rows, k_cols, k_stride);
    if (r) return r;
    r = make_rows_tmap(&tmV, v, rows, v_cols, v_stride);
    if (r) return r;
    r = make_rows_tmap(&tmDO, dout, rows, do_cols, do_stride);
    if (r) return r;
    BwdParams p;
    p.B = B; p.T = T; p.H = H; p.KV = KV;
    p.scale = scale;
    p.scale_log2 = scale * LOG2E;
    p.lse = lse;
    p.dsum = dsum;
    p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0; p.do_col0 = do_col0;
    p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
    p.dq_stride = dq_stride; p.dk_stride = dk_stride; p.dv_stride = dv_stride;
    p.n_tiles = (T + BT - 1) / BT;
    p.status = status;
    return hd == 128 ? launch_bwd<128>(tmQ, tmK, tmV, tmDO, p, o, o_stride, dout, do_stride, which, st)
                     : launch_bwd<64>(tmQ, tmK, tmV, tmDO, p, o, o_stride, dout, do_stride, which, st);
}
