// Causal GQA flash-attention forward for sm_100a (head_dim 64 or 128, bf16), fixed-length
// batches or packed variable-length sequences (cu_seqlens).
//
// One CTA owns one 128-row query tile of one head and walks its key/value tiles.  Ten warps: eight
// softmax warps (two threads per query row, 64 key columns each; the row maximum and sum cross
// between them through shared memory), one MMA-issuing warp, one TMA warp.  The score tile is
// double-buffered in tensor memory, so the scores of the next key tile are already there when the
// softmax of the current one ends: the softmax warps never wait for the tensor pipe, and the
// tensor pipe only has the P V product of a tile on the path between two softmax passes.
//
//   tensor pipe:   S(j+1) ........ PV(j) S(j+2) ........ PV(j+1) S(j+3)
//   softmax:       softmax(j) ......... softmax(j+1) ......... softmax(j+2)
//
//   S = Q K^T      tcgen05.mma with Q read from tensor memory (written there once per CTA) and K
//                  K-major in shared memory (TMA, 128-byte swizzle): half the shared-memory traffic
//                  of the all-shared form, which is what bounds a 128 x 128 tile
//   softmax        tcgen05.ld the row, online max / sum in base 2 with packed two-wide arithmetic,
//                  P written back over the score columns as packed bf16 (tcgen05.st); a share of
//                  the exponentials is evaluated on the FMA pipe so that the special-function unit
//                  is not the only source
//   O += P V       tcgen05.mma with A read from tensor memory and V as an MN-major shared operand
// The softmax can finish tile j+1 before the issuing thread has looked at tile j, so every
// barrier that hands a score buffer over exists once per buffer (a single barrier would be two
// phases ahead of its waiter).  K tiles move through a three-stage ring (a tile is requested two products ahead), V tiles
// through a two-stage ring.  The running maximum is refreshed lazily: O and the running sum are
// rescaled only when a row's maximum grows by more than 2^8.
// Every wait is bounded (status word on timeout).
#include "attn_common.cuh"

namespace {

using namespace attn;

#define KB_FAIL_FWD(code)                              \
    {                                                  \
        atomicMax(p.status, (int)(code));              \
        break;                                         \
    }

constexpr int KST = 4, VST = 2;                    // ring depths
constexpr float RESCALE_THRESHOLD = 8.0f;          // in log2 units
constexpr int EMU = 2;                             // of every 4 pairs of exponentials, this many run on the FMA pipe
constexpr int FWD_THREADS = 320;                   // 8 softmax warps, MMA warp, TMA warp

struct FlashParams {
    int B, T, H, KV;
    const int* cu_seqlens;                         // [B + 1] token offsets, or null: sequence b = rows [b*T, (b+1)*T)
    float scale_log2;                              // softmax scale * log2(e)
    __nv_bfloat16* out;                            // token-major, heads side by side
    long long out_stride;                          // elements between tokens of `out`
    float* lse;                                    // natural log; index head * lse_hs + (b * lse_bs | cu[b]) + t
    long long lse_hs, lse_bs;
    int q_col0, k_col0, v_col0;                    // first column of head 0 inside each operand's rows
    const __nv_bfloat16* q_ptr;                    // the query matrix itself (rows are read directly, once per CTA)
    long long q_stride, q_rows;
    int n_tiles;                                   // query tiles per sequence (grid decode)
    int* status;
};

#ifdef KB_ATTN_PROFILE
// Phase timing of CTA 0 (clock64 sums), for tuning builds only.
__device__ long long g_attn_dbg[16];
#define KB_TICK(i, t0)                                       \
    if (prof) {                                              \
        const long long t1_ = clock64();                     \
        dbg[i] += t1_ - t0;                                  \
        t0 = t1_;                                            \
    }
#else
#define KB_TICK(i, t0)
#endif

template <int HD>
constexpr int fwd_smem_bytes() {
    return (KST + VST) * Tile<HD>::BYTES + 1024 + 256 + 6 * BT * 4;
}

template <int HD>
__global__ void __launch_bounds__(FWD_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
    constexpr int TB = Tile<HD>::BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;
    uint8_t* sV = sK + KST * TB;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + VST * TB);
    uint64_t* q_ready = bars + 0;                  // the query tile sits in tensor memory
    uint64_t* k_full = bars + 1;                   // [KST]
    uint64_t* k_empty = k_full + KST;
    uint64_t* v_full = k_empty + KST;              // [VST]
    uint64_t* v_empty = v_full + VST;
    uint64_t* s_full = v_empty + VST;              // [2] one per score buffer
    uint64_t* p_ready = s_full + 2;                // [2] one per score buffer
    uint64_t* o_done = p_ready + 2;
    uint64_t* xch = o_done + 1;                    // the two halves of a row exchange their maximum / sum
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xch + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // row maxima [tile parity][half][row] and, at the end, row sums [4 + half][row] of the two threads
    // that share a query row
    float* row_buf = reinterpret_cast<float*>(smem + (KST + VST) * TB + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heavy tiles (late queries) first
    const int HB = p.H * p.B;
    const int qt = p.n_tiles - 1 - (int)(blockIdx.x / HB);
    const int hb = blockIdx.x % HB;
    const int head = hb % p.H, b = hb / p.H;
    const int kvh = head / (p.H / p.KV);
    int seq_row0, Tb;
    if (p.cu_seqlens) {
        seq_row0 = p.cu_seqlens[b];
        Tb = p.cu_seqlens[b + 1] - seq_row0;
    } else {
        seq_row0 = b * p.T;
        Tb = p.T;
    }
    // key tiles of this query tile; a tile that starts past the sequence end has none
    const int n = qt * BT < Tb ? qt + 1 : 0;

    if (threadIdx.x == 0) {
        tc::mbar_init(q_ready, 8);
        for (int i = 0; i < KST; ++i) { tc::mbar_init(k_full + i, 1); tc::mbar_init(k_empty + i, 1); }
        for (int i = 0; i < VST; ++i) { tc::mbar_init(v_full + i, 1); tc::mbar_init(v_empty + i, 1); }
        tc::mbar_init(s_full + 0, 1);
        tc::mbar_init(s_full + 1, 1);
        tc::mbar_init(p_ready + 0, 8);
        tc::mbar_init(p_ready + 1, 8);
        tc::mbar_init(o_done, 1);
        tc::mbar_init(xch, 8);
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    if (warp == 8) {
        tc::tmem_alloc(tmem_slot, 512);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    // score buffers at columns 0 and 128, output accumulator at 256, the query tile (packed bf16) at 384
    const uint32_t tmem0 = *tmem_slot;
    const uint32_t tmem_oacc = tmem0 + 256, tmem_q = tmem0 + 384;

    if (n == 0) {
        // nothing to do (sequence shorter than the grid was sized for)
    } else if (warp == 9) {
        // ------------------------------------------------------------ TMA
        if (lane == 0) {
            tc::prefetch_tmap(&tmK);
            tc::prefetch_tmap(&tmV);
            const int kx = p.k_col0 + kvh * HD, vx = p.v_col0 + kvh * HD;
            // order of need: K0 K1 V0 K2 V1 K3 V2 ...
            auto load_k = [&](int j) -> bool {
                const int ks = j % KST;
                if (!tc::mbar_wait(k_empty + ks, ((j / KST) & 1) ^ 1, abort_flag)) return false;
                tc::mbar_expect_tx(k_full + ks, TB);
                load_tile<HD>(sK + ks * TB, &tmK, k_full + ks, kx, seq_row0 + j * BT);
                return true;
            };
            bool ok = load_k(0) && (n < 2 || load_k(1));
            for (int j = 0; j < n && ok; ++j) {
                const int vs = j % VST;
                if (!tc::mbar_wait(v_empty + vs, ((j / VST) & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc::mbar_expect_tx(v_full + vs, TB);
                load_tile<HD>(sV + vs * TB, &tmV, v_full + vs, vx, seq_row0 + j * BT);
                if (j + 2 < n) ok = load_k(j + 2);
            }
            if (!ok) atomicMax(p.status, (int)KB_TIMEOUT_TMA);
        }
    } else if (warp == 8) {
        // ------------------------------------------------------------ MMA issue (one thread)
        if (lane == 0) {
            const uint32_t idesc_s = tc::instr_desc_f16(BT, BT, 1, 1, 0, 0);
            const uint32_t idesc_o = tc::instr_desc_f16(BT, HD, 1, 1, 0, 1);
            const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
            do {
                if (!tc::mbar_wait(q_ready, 0, abort_flag) || !tc::mbar_wait(k_full, 0, abort_flag)) KB_FAIL_FWD(KB_TIMEOUT_TMA)
                tc::tc_fence_after();
                mma_tn_tile<HD>(tmem0, tmem_q, k_addr, idesc_s);
                tc::tc_commit(s_full + 0);
                tc::tc_commit(k_empty + 0);
                if (n > 1) {
                    if (!tc::mbar_wait(k_full + 1, 0, abort_flag)) KB_FAIL_FWD(KB_TIMEOUT_TMA)
                    tc::tc_fence_after();
                    mma_tn_tile<HD>(tmem0 + 128, tmem_q, k_addr + TB, idesc_s);
                    tc::tc_commit(s_full + 1);
                    tc::tc_commit(k_empty + 1);
                }
                for (int j = 0; j < n; ++j) {
                    const int vs = j % VST;
                    if (!tc::mbar_wait(v_full + vs, (j / VST) & 1, abort_flag)) KB_FAIL_FWD(KB_TIMEOUT_TMA)
                    if (!tc::mbar_wait(p_ready + (j & 1), (j >> 1) & 1, abort_flag)) KB_FAIL_FWD(KB_TIMEOUT_MMA)
                    tc::tc_fence_after();
                    mma_ts_tile<HD, false>(tmem_oacc, tmem0 + (j & 1) * 128, v_addr + vs * TB, idesc_o, j != 0);
                    tc::tc_commit(o_done);
                    tc::tc_commit(v_empty + vs);
                    if (j + 2 < n) {
                        const int ks = (j + 2) % KST;
                        if (!tc::mbar_wait(k_full + ks, ((j + 2) / KST) & 1, abort_flag)) KB_FAIL_FWD(KB_TIMEOUT_TMA)
                        tc::tc_fence_after();
                        mma_tn_tile<HD>(tmem0 + (j & 1) * 128, tmem_q, k_addr + ks * TB, idesc_s);
                        tc::tc_commit(s_full + (j & 1));
                        tc::tc_commit(k_empty + ks);
                    }
                }
            } while (false);
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------ softmax: two threads per query row
        const int hf = warp >> 2;                                  // which 64 of the tile's 128 key columns
        const int r = (warp & 3) * 32 + lane;                      // row inside the tile
        const uint32_t lane_base = ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t tmem_o = tmem_oacc + lane_base;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        {
            // this thread's half of its query row goes to tensor memory as the A operand of every S = Q K^T
            constexpr int QW = HD / 2;                              // elements per thread
            const long long grow = (long long)seq_row0 + qt * BT + r;
            const __nv_bfloat16* src = p.q_ptr + grow * p.q_stride + p.q_col0 + head * HD + hf * QW;
            uint32_t qp[QW / 2];
#pragma unroll
            for (int i = 0; i < QW / 8; ++i) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (grow < p.q_rows) v = *reinterpret_cast<const uint4*>(src + i * 8);
                qp[4 * i] = v.x; qp[4 * i + 1] = v.y; qp[4 * i + 2] = v.z; qp[4 * i + 3] = v.w;
            }
            if constexpr (QW == 64) tc::tmem_st32(tmem_q + hf * 32 + lane_base, qp);
            else tc::tmem_st16(tmem_q + hf * 16 + lane_base, qp);
            tc::tmem_st_wait();
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(q_ready);
        }
#ifdef KB_ATTN_PROFILE
        const bool prof = blockIdx.x == 0 && threadIdx.x == 0;
        long long dbg[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long tk = clock64();
#endif
        for (int j = 0; j < n && ok; ++j) {
            const uint32_t tmem_s = tmem0 + (j & 1) * 128 + lane_base;
            KB_TICK(0, tk)                                              // loop overhead / arrive
            if (!tc::mbar_wait(s_full + (j & 1), (j >> 1) & 1, abort_flag)) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                ok = false;
                break;
            }
            tc::tc_fence_after();
            KB_TICK(1, tk)                                              // wait for the scores
            float s[64];
            tc::tmem_ld32(tmem_s + hf * 64, reinterpret_cast<uint32_t*>(s));
            tc::tmem_ld32(tmem_s + hf * 64 + 32, reinterpret_cast<uint32_t*>(s + 32));
            tc::tmem_ld_wait();
            KB_TICK(2, tk)                                              // tensor-memory load
            if (j == qt) {                                          // diagonal tile: causal mask
                const int cmax = r - hf * 64;
#pragma unroll
                for (int c = 0; c < 64; ++c) s[c] = c <= cmax ? s[c] : -INFINITY;
            }
            float mx8[8];                                           // eight chains: latency, not count, matters here
#pragma unroll
            for (int i = 0; i < 8; ++i) mx8[i] = fmaxf(s[2 * i], s[2 * i + 1]);
#pragma unroll
            for (int c = 16; c < 64; c += 16) {
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = fmax3(mx8[i], s[c + 2 * i], s[c + 2 * i + 1]);
            }
            float mx = fmax3(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]));
            // The row maximum spans both halves: exchange through shared memory.  The barrier also
            // orders "both halves have read their scores" before either writes P over them.
            row_buf[((j & 1) * 2 + hf) * BT + r] = mx;
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(xch);
            if (!tc::mbar_wait(xch, j & 1, abort_flag)) {           // bounded, like every other wait
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                ok = false;
                break;
            }
            mx = fmaxf(mx, row_buf[((j & 1) * 2 + (hf ^ 1)) * BT + r]) * p.scale_log2;
            const bool grow = mx > m_used + RESCALE_THRESHOLD;      // first tile: m_used = -inf -> true
            if (j == 0) {
                m_used = mx;
            } else if (__any_sync(0xffffffffu, grow)) {
                // O holds sums of p * v with p relative to m_used: move it to the new maximum.  Both
                // halves see the same maxima and take the same branch; each rescales half of O's columns.
                if (!tc::mbar_wait(o_done, (j - 1) & 1, abort_flag)) {
                    if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                    ok = false;
                    break;
                }
                tc::tc_fence_after();
                const float m_new = fmaxf(m_used, mx);
                const float f = exp2f(m_used - m_new);
#pragma unroll 1
                for (int c = 0; c < HD / 2; c += 32) {
                    uint32_t o[32];
                    tc::tmem_ld32(tmem_o + hf * (HD / 2) + c, o);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                    tc::tmem_st32(tmem_o + hf * (HD / 2) + c, o);
                }
                tc::tmem_st_wait();
                l *= f;
                m_used = m_new;
            }
            KB_TICK(3, tk)                                              // max, exchange and rescale check
            // P carries the truncation bias (see pack_bf16_trunc); so does the running sum, which the
            // epilogue divides out
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
            const float2 nm2 = make_float2(TRUNC_BIAS_LOG2 - m_used, TRUNC_BIAS_LOG2 - m_used);
            float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4) {                        // 32 scores -> 16 packed columns at a time
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const float2 x = __ffma2_rn(make_float2(s[q4 * 32 + c], s[q4 * 32 + c + 1]), sc2, nm2);
                    const float2 e = exp2_pair<EMU>(x, c >> 1);
                    sum2[(c >> 1) & 1] = __fadd2_rn(sum2[(c >> 1) & 1], e);
                    pk[c >> 1] = pack_bf16_trunc(e.x, e.y);
                }
                tc::tmem_st16(tmem_s + hf * 32 + q4 * 16, pk);
            }
            l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
            KB_TICK(4, tk)                                              // exponentials, packing, store issue
            tc::tmem_st_wait();
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(p_ready + (j & 1));
            KB_TICK(5, tk)                                              // store wait, fence, arrive
        }
#ifdef KB_ATTN_PROFILE
        if (prof) {
            for (int i = 0; i < 6; ++i) g_attn_dbg[i] = dbg[i];
            g_attn_dbg[6] = n;
        }
#endif
        // the row sum spans both halves too
        if (ok) {
            row_buf[(4 + hf) * BT + r] = l;
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(xch);
            if (tc::mbar_wait(xch, n & 1, abort_flag)) {
                l += row_buf[(4 + (hf ^ 1)) * BT + r];
            } else {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                ok = false;
            }
        }
        if (ok) {
            if (tc::mbar_wait(o_done, (n - 1) & 1, abort_flag)) {
                tc::tc_fence_after();
                const float inv = TRUNC_BIAS / l;
                // Rows past the end of the sequence (zero-filled by TMA, or the first rows of the next
                // sequence) are computed but never stored; for the valid rows the causal mask already
                // excludes every key at or beyond the end.
                const bool valid = qt * BT + r < Tb;
                __nv_bfloat16* dst = p.out + (size_t)(seq_row0 + qt * BT + r) * p.out_stride + head * HD + hf * (HD / 2);
#pragma unroll 1
                for (int c = 0; c < HD / 2; c += 32) {
                    uint32_t o[32];
                    tc::tmem_ld32(tmem_o + hf * (HD / 2) + c, o);
                    tc::tmem_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            float f8[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) f8[e] = __uint_as_float(o[i + e]) * inv;
                            st8(dst + c + i, pack8(f8));
                        }
                    }
                }
                if (valid && hf == 0) {
                    const long long base = p.cu_seqlens ? (long long)seq_row0 : (long long)b * p.lse_bs;
                    p.lse[(long long)head * p.lse_hs + base + qt * BT + r] = (m_used + log2f(l) - TRUNC_BIAS_LOG2) * LN2;
                }
            } else if (lane == 0) {
                atomicMax(p.status, (int)KB_TIMEOUT_EPI);
            }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem0, 512);
    }
}

// Per-device opt-in to the kernel's dynamic shared memory (an attribute of the function on one
// device: a second device in the same process needs its own call).
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
int launch_fwd(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const FlashParams& p,
               int max_T, cudaStream_t st) {
    static bool attr[64] = {};
    int r = ensure_smem(flash_fwd_kernel<HD>, fwd_smem_bytes<HD>(), attr);
    if (r) return r;
    const int grid = p.n_tiles * p.H * p.B;
    flash_fwd_kernel<HD><<<grid, FWD_THREADS, fwd_smem_bytes<HD>(), st>>>(tmQ, tmK, tmV, p);
    return cudaGetLastError() == cudaSuccess ? 0 : 8;
}

}  // namespace

#ifdef KB_ATTN_PROFILE
KB_API int kb_attn_dbg_read(long long* host16) {
    return cudaMemcpyFromSymbol(host16, g_attn_dbg, sizeof(long long) * 16) == cudaSuccess ? 0 : 1;
}
#endif

// q/k/v: token-major matrices [total tokens, *] whose rows hold the heads side by side (row strides
// in elements; *_col0 = column of head 0).  out: token-major with `out_stride` elements per token.
// Fixed-length batches: cu_seqlens null, B sequences of T tokens, lse[B, H, T].  Packed sequences:
// cu_seqlens[B + 1] (device), `total` tokens, max_T the longest sequence, lse[H, total].
KB_API int kb_flash_fwd(const void* q, long long q_stride, int q_cols, int q_col0, const void* k, long long k_stride,
                        int k_cols, int k_col0, const void* v, long long v_stride, int v_cols, int v_col0, void* out,
                        long long out_stride, float* lse, const int* cu_seqlens, long long total, int B, int max_T, int H,
                        int KV, int hd, float scale, int* status, cudaStream_t st) {
    if ((hd != 128 && hd != 64) || max_T < 1 || B < 1 || KV < 1 || H % KV != 0) return 5;
    if (!operand_ok(q, q_stride, q_col0) || !operand_ok(k, k_stride, k_col0) || !operand_ok(v, v_stride, v_col0)) return 6;
    if (((uintptr_t)out & 15) || (out_stride & 7)) return 6;
    const long long rows = cu_seqlens ? total : (long long)B * max_T;
    CUtensorMap tmQ, tmK, tmV;
    int r = make_rows_tmap(&tmQ, q, rows, q_cols, q_stride);
    if (r) return r;
    r = make_rows_tmap(&tmK, k, rows, k_cols, k_stride);
    if (r) return r;
    r = make_rows_tmap(&tmV, v, rows, v_cols, v_stride);
    if (r) return r;
    FlashParams p;
    p.B = B; p.T = max_T; p.H = H; p.KV = KV;
    p.cu_seqlens = cu_seqlens;
    p.scale_log2 = scale * LOG2E;
    p.out = (__nv_bfloat16*)out;
    p.out_stride = out_stride;
    p.lse = lse;
    p.lse_hs = cu_seqlens ? total : max_T;
    p.lse_bs = cu_seqlens ? 0 : (long long)H * max_T;
    p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
    p.q_ptr = (const __nv_bfloat16*)q;
    p.q_stride = q_stride;
    p.q_rows = rows;
    p.n_tiles = (max_T + BT - 1) / BT;
    p.status = status;
    return hd == 128 ? launch_fwd<128>(tmQ, tmK, tmV, p, max_T, st) : launch_fwd<64>(tmQ, tmK, tmV, p, max_T, st);
}
