// Memory-bound kernels of the training step (bf16 activations, fp32 statistics):
//   * AttnRes depth routing fused with the RMSNorm that follows it, forward and backward.
//     Sources are passed by pointer (no stacked buffer); the backward accumulates source
//     gradients in place and reduces the query / norm-weight gradients deterministically.
//   * per-head QK RMSNorm + rotate-half RoPE, forward and backward
//   * SwiGLU, cross-entropy + z-loss on a logits chunk, embedding gather / scatter-add
//   * fused AdamW, Muon momentum / apply, sum of squares, tiled transpose, column sums
// The routing math follows the reference's `_route_static` (src/model/llama.py:630-644) and
// its Triton backward (src/model/flash_attn_res/kernels/phase_1.py:204-249).
#include "common.cuh"

typedef __nv_bfloat16 bf16;

// Switch of the dependent launches (common.cuh: kb_launch_dep).  The serving engine turns it on around its
// decode steps, whose ~320 launches of a few microseconds each otherwise pay a launch gap apiece.
int g_kb_dependent_launch = 0;
KB_API int kb_set_dependent_launch(int on) {
    const int was = g_kb_dependent_launch;
    g_kb_dependent_launch = on ? 1 : 0;
    return was;
}

static inline int kb_num_sms() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// ============================================================================ routing
struct RouteSrcs {
    const bf16* p[16];
};
struct RouteDsts {
    bf16* p[16];
    unsigned acc_mask;  // bit s set: accumulate into p[s], else overwrite
};

template <int MAXS, int CPT>
__device__ __forceinline__ void route_load(const RouteSrcs& srcs, int S, size_t base, int nchunks,
                                           bf16x8 (&u)[MAXS][CPT]) {
#pragma unroll
    for (int s = 0; s < MAXS; ++s) {
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (s < S && c < nchunks) {
                u[s][k] = ld8(srcs.p[s] + base + (size_t)c * 8);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) u[s][k].v[i] = __floats2bfloat162_rn(0.f, 0.f);
            }
        }
    }
}

template <int MAXS, int CPT>
__global__ void __launch_bounds__(256)
route_norm_fwd_kernel(RouteSrcs srcs, int S, const bf16* __restrict__ q, const bf16* __restrict__ rn_w,
                      const bf16* __restrict__ n_w, bf16* __restrict__ xn, float* __restrict__ alpha_o,
                      float* __restrict__ r_o, float* __restrict__ logit_o, float* __restrict__ rstd_o, int N, int D,
                      float eps) {
    __shared__ float scratch[2 * MAXS * 32];
    const int nchunks = D >> 3;
    const float invD = 1.f / (float)D;
    for (int tok = blockIdx.x; tok < N; tok += gridDim.x) {
        bf16x8 u[MAXS][CPT];
        const size_t base = (size_t)tok * D;
        route_load<MAXS, CPT>(srcs, S, base, nchunks, u);
        float al[MAXS];
        if (q != nullptr) {
            float red[2 * MAXS];
#pragma unroll
            for (int i = 0; i < 2 * MAXS; ++i) red[i] = 0.f;
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const int c = threadIdx.x + k * blockDim.x;
                if (c < nchunks) {
                    float w[8], t[8];
                    unpack8(ld8(q + c * 8), w);
                    unpack8(ld8(rn_w + c * 8), t);
#pragma unroll
                    for (int i = 0; i < 8; ++i) w[i] *= t[i];
#pragma unroll
                    for (int s = 0; s < MAXS; ++s) {
                        if (s < S) {
                            unpack8(u[s][k], t);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                red[2 * s] += t[i] * w[i];
                                red[2 * s + 1] += t[i] * t[i];
                            }
                        }
                    }
                }
            }
            block_sum<2 * MAXS>(red, scratch);
            float mx = -INFINITY, rr[MAXS], lg[MAXS];
#pragma unroll
            for (int s = 0; s < MAXS; ++s) {
                rr[s] = rsqrtf(red[2 * s + 1] * invD + eps);
                lg[s] = red[2 * s] * rr[s];
                if (s < S) mx = fmaxf(mx, lg[s]);
            }
            float den = 0.f;
#pragma unroll
            for (int s = 0; s < MAXS; ++s) {
                al[s] = s < S ? __expf(lg[s] - mx) : 0.f;
                den += al[s];
            }
            const float inv = 1.f / den;
#pragma unroll
            for (int s = 0; s < MAXS; ++s) al[s] *= inv;
            if (threadIdx.x == 0) {
#pragma unroll
                for (int s = 0; s < MAXS; ++s) {
                    if (s < S) {
                        alpha_o[(size_t)tok * S + s] = al[s];
                        r_o[(size_t)tok * S + s] = rr[s];
                        logit_o[(size_t)tok * S + s] = lg[s];
                    }
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < MAXS; ++s) al[s] = s == 0 ? 1.f : 0.f;
        }
        float h[CPT][8];
        float hsq[1] = {0.f};
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
#pragma unroll
            for (int i = 0; i < 8; ++i) h[k][i] = 0.f;
#pragma unroll
            for (int s = 0; s < MAXS; ++s) {
                if (s < S) {
                    float t[8];
                    unpack8(u[s][k], t);
#pragma unroll
                    for (int i = 0; i < 8; ++i) h[k][i] += al[s] * t[i];
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) hsq[0] += h[k][i] * h[k][i];
        }
        block_sum<1>(hsq, scratch);
        const float rs = rsqrtf(hsq[0] * invD + eps);
        if (threadIdx.x == 0) rstd_o[tok] = rs;
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nchunks) {
                float w[8], o[8];
                unpack8(ld8(n_w + c * 8), w);
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = h[k][i] * rs * w[i];
                st8(xn + base + (size_t)c * 8, pack8(o));
            }
        }
    }
}

template <int MAXS, int CPT>
__global__ void __launch_bounds__(256)
route_norm_bwd_kernel(RouteSrcs srcs, RouteDsts dsts, int S, const bf16* __restrict__ dxn,
                      const bf16* __restrict__ q, const bf16* __restrict__ rn_w, const bf16* __restrict__ n_w,
                      const float* __restrict__ alpha_i, const float* __restrict__ r_i,
                      const float* __restrict__ logit_i, const float* __restrict__ rstd_i,
                      float* __restrict__ dw_part, float* __restrict__ dnw_part, int N, int D) {
    __shared__ float scratch[MAXS * 32];
    const int nchunks = D >> 3;
    const float invD = 1.f / (float)D;
    const bool routing = q != nullptr;
    float dw_acc[CPT][8], dnw_acc[CPT][8];
#pragma unroll
    for (int k = 0; k < CPT; ++k) {
#pragma unroll
        for (int i = 0; i < 8; ++i) dw_acc[k][i] = dnw_acc[k][i] = 0.f;
    }
    for (int tok = blockIdx.x; tok < N; tok += gridDim.x) {
        bf16x8 u[MAXS][CPT];
        const size_t base = (size_t)tok * D;
        route_load<MAXS, CPT>(srcs, S, base, nchunks, u);
        float al[MAXS], rr[MAXS], lg[MAXS];
#pragma unroll
        for (int s = 0; s < MAXS; ++s) {
            if (routing && s < S) {
                al[s] = alpha_i[(size_t)tok * S + s];
                rr[s] = r_i[(size_t)tok * S + s];
                lg[s] = logit_i[(size_t)tok * S + s];
            } else {
                al[s] = (!routing && s == 0) ? 1.f : 0.f;
                rr[s] = 0.f;
                lg[s] = 0.f;
            }
        }
        const float rs = rstd_i[tok];
        // RMSNorm backward: dh = rs * (gw - hn * mean(gw*hn)), hn = h*rs, gw = dxn*n_w
        float hn[CPT][8], dh[CPT][8];
        float c1[1] = {0.f};
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
#pragma unroll
            for (int i = 0; i < 8; ++i) hn[k][i] = 0.f;
#pragma unroll
            for (int s = 0; s < MAXS; ++s) {
                if (s < S) {
                    float t[8];
                    unpack8(u[s][k], t);
#pragma unroll
                    for (int i = 0; i < 8; ++i) hn[k][i] += al[s] * t[i];
                }
            }
            float g[8], w[8];
            if (c < nchunks) {
                unpack8(ld8(dxn + base + (size_t)c * 8), g);
                unpack8(ld8(n_w + c * 8), w);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) g[i] = w[i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                hn[k][i] *= rs;
                dnw_acc[k][i] += g[i] * hn[k][i];
                dh[k][i] = g[i] * w[i];
                c1[0] += dh[k][i] * hn[k][i];
            }
        }
        block_sum<1>(c1, scratch);
        const float m = c1[0] * invD;
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
#pragma unroll
            for (int i = 0; i < 8; ++i) dh[k][i] = rs * (dh[k][i] - hn[k][i] * m);
        }
        float dl[MAXS];
        if (routing) {
            float a[MAXS];
#pragma unroll
            for (int s = 0; s < MAXS; ++s) {
                a[s] = 0.f;
                if (s < S) {
#pragma unroll
                    for (int k = 0; k < CPT; ++k) {
                        float t[8];
                        unpack8(u[s][k], t);
#pragma unroll
                        for (int i = 0; i < 8; ++i) a[s] += dh[k][i] * t[i];
                    }
                }
            }
            block_sum<MAXS>(a, scratch);
            float abar = 0.f;
#pragma unroll
            for (int s = 0; s < MAXS; ++s) abar += al[s] * a[s];
#pragma unroll
            for (int s = 0; s < MAXS; ++s) dl[s] = al[s] * (a[s] - abar);
        } else {
#pragma unroll
            for (int s = 0; s < MAXS; ++s) dl[s] = 0.f;
        }
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c >= nchunks) continue;
            float w[8];
            if (routing) {
                float t[8];
                unpack8(ld8(q + c * 8), w);
                unpack8(ld8(rn_w + c * 8), t);
#pragma unroll
                for (int i = 0; i < 8; ++i) w[i] *= t[i];
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) w[i] = 0.f;
            }
#pragma unroll
            for (int s = 0; s < MAXS; ++s) {
                if (s < S) {
                    float t[8], du[8];
                    unpack8(u[s][k], t);
                    const float c_w = dl[s] * rr[s];
                    const float c_u = dl[s] * lg[s] * rr[s] * rr[s] * invD;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        du[i] = al[s] * dh[k][i] + c_w * w[i] - c_u * t[i];
                        dw_acc[k][i] += c_w * t[i];
                    }
                    bf16* dst = dsts.p[s] + base + (size_t)c * 8;
                    if (dsts.acc_mask >> s & 1u) {
                        float o[8];
                        unpack8(ld8(dst), o);
#pragma unroll
                        for (int i = 0; i < 8; ++i) du[i] += o[i];
                    }
                    st8(dst, pack8(du));
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < CPT; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < nchunks) {
            float* a = dnw_part + (size_t)blockIdx.x * D + (size_t)c * 8;
            float* b = dw_part + (size_t)blockIdx.x * D + (size_t)c * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                a[i] = dnw_acc[k][i];
                if (routing) b[i] = dw_acc[k][i];
            }
        }
    }
}

static inline void route_cfg(int D, int& cpt, int& threads) {
    const int nchunks = D / 8;
    cpt = (nchunks + 255) / 256;
    threads = ((nchunks + cpt - 1) / cpt + 31) / 32 * 32;
}

#define ROUTE_DISPATCH_CPT(MAXS_, CALL)                          \
    switch (cpt) {                                               \
        case 1: { constexpr int MAXS = MAXS_, CPT = 1; CALL; break; } \
        case 2: { constexpr int MAXS = MAXS_, CPT = 2; CALL; break; } \
        case 3: { constexpr int MAXS = MAXS_, CPT = 3; CALL; break; } \
        case 4: { constexpr int MAXS = MAXS_, CPT = 4; CALL; break; } \
        default: return 5;                                       \
    }
#define ROUTE_DISPATCH(CALL)                                     \
    if (S <= 1) { ROUTE_DISPATCH_CPT(1, CALL) }                  \
    else if (S <= 2) { ROUTE_DISPATCH_CPT(2, CALL) }             \
    else if (S <= 4) { ROUTE_DISPATCH_CPT(4, CALL) }             \
    else if (S <= 8) { ROUTE_DISPATCH_CPT(8, CALL) }             \
    else if (S <= 12) { ROUTE_DISPATCH_CPT(12, CALL) }           \
    else { ROUTE_DISPATCH_CPT(16, CALL) }

// Grid size used by the routing backward; the caller sizes the partial buffers with it.
KB_API int kb_route_bwd_grid(int N) {
    const int g = kb_num_sms() * 4;
    return N < g ? N : g;
}

KB_API int kb_route_norm_fwd(const void* const* srcs, int S, const void* q, const void* rn_w, const void* n_w,
                             void* xn, float* alpha, float* r, float* logit, float* rstd, int N, int D, float eps,
                             cudaStream_t st) {
    if (S < 1 || S > 16 || D % 8 != 0 || D > 8192) return 5;
    RouteSrcs rs;
    for (int s = 0; s < 16; ++s) rs.p[s] = s < S ? (const bf16*)srcs[s] : nullptr;
    int cpt, threads;
    route_cfg(D, cpt, threads);
    const int grid = N < kb_num_sms() * 8 ? N : kb_num_sms() * 8;
    ROUTE_DISPATCH((route_norm_fwd_kernel<MAXS, CPT><<<grid, threads, 0, st>>>(
        rs, S, (const bf16*)q, (const bf16*)rn_w, (const bf16*)n_w, (bf16*)xn, alpha, r, logit, rstd, N, D, eps)))
    return kb_launch_status();
}

KB_API int kb_route_norm_bwd(const void* const* srcs, void* const* dsts, unsigned acc_mask, int S, const void* dxn,
                             const void* q, const void* rn_w, const void* n_w, const float* alpha, const float* r,
                             const float* logit, const float* rstd, float* dw_part, float* dnw_part, int N, int D,
                             cudaStream_t st) {
    if (S < 1 || S > 16 || D % 8 != 0 || D > 8192) return 5;
    RouteSrcs rs;
    RouteDsts ds;
    for (int s = 0; s < 16; ++s) {
        rs.p[s] = s < S ? (const bf16*)srcs[s] : nullptr;
        ds.p[s] = s < S ? (bf16*)dsts[s] : nullptr;
    }
    ds.acc_mask = acc_mask;
    int cpt, threads;
    route_cfg(D, cpt, threads);
    const int grid = kb_route_bwd_grid(N);
    ROUTE_DISPATCH((route_norm_bwd_kernel<MAXS, CPT><<<grid, threads, 0, st>>>(
        rs, ds, S, (const bf16*)dxn, (const bf16*)q, (const bf16*)rn_w, (const bf16*)n_w, alpha, r, logit, rstd,
        dw_part, dnw_part, N, D)))
    return kb_launch_status();
}

// out[c] = sum_r part[r, c] ; block (128, 8): 8 row groups reduced through shared memory.
__global__ void colsum_kernel(const float* __restrict__ part, float* __restrict__ out, int R, int C) {
    __shared__ float sm[8][128];
    const int c = blockIdx.x * 128 + threadIdx.x;
    float acc = 0.f;
    if (c < C)
        for (int r = threadIdx.y; r < R; r += 8) acc += part[(size_t)r * C + c];
    sm[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float t = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) t += sm[j][threadIdx.x];
        out[c] = t;
    }
}
KB_API int kb_colsum(const float* part, float* out, int R, int C, cudaStream_t st) {
    colsum_kernel<<<(C + 127) / 128, dim3(128, 8), 0, st>>>(part, out, R, C);
    return kb_launch_status();
}

// ============================================================================ QK-norm + RoPE
// One warp per token.  A head is covered by HD/16 lanes (lane `sub` owns elements [8*sub, 8*sub+8) of
// each half, one 16-byte access per half), so a warp takes 32/(HD/16) heads per pass; the token's
// cos/sin row and the norm weights stay in registers across all heads of the token.
// APPEND (serving): the rotated keys and the untouched values of token n also go to slot[n] of the paged cache
// ([pages][nkv][16][HD]; slot = page * 16 + offset, negative = skip, at or past num_slots = skipped and recorded
// as KB_BAD_INDEX) - the value heads are walked as nkv more heads that are only copied.
template <int HD, bool NORM, bool APPEND>
__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ qw, const bf16* __restrict__ kw,
                       const float* __restrict__ cosT, const float* __restrict__ sinT, bf16* __restrict__ out,
                       float* __restrict__ rstd_o, int N, int T, int nq, int nkv, int pos_offset, float eps,
                       const int* __restrict__ positions, bf16* __restrict__ k_pages, bf16* __restrict__ v_pages,
                       const long long* __restrict__ slot, long long num_slots, int* __restrict__ status) {
    constexpr int LPH = HD / 16, HPW = 32 / LPH;
    kb_dep_trigger();
    kb_dep_wait();
    const int nh = nq + nkv;
    const int nwalk = APPEND ? nh + nkv : nh;            // heads this kernel walks
    const int lane = threadIdx.x & 31, sub = lane % LPH, hsel = lane / LPH, e0 = sub * 8;
    const int in_stride = (nq + 2 * nkv) * HD, out_stride = nh * HD;
    float wq1[8], wq2[8], wk1[8], wk2[8];
    if (NORM) {
        unpack8(ld8(qw + e0), wq1);
        unpack8(ld8(qw + HD / 2 + e0), wq2);
        unpack8(ld8(kw + e0), wk1);
        unpack8(ld8(kw + HD / 2 + e0), wk2);
    }
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    // few tokens (decode): a warp takes one pass of HPW heads of one token instead of the whole token
    const int ngroups = (nwalk + HPW - 1) / HPW;
    const int gsplit = N >= nwarps ? 1 : ngroups;
    for (long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); item < (long long)N * gsplit;
         item += nwarps) {
        const long long tok = item / gsplit;
        const int h_lo = gsplit == 1 ? 0 : (int)(item % gsplit) * HPW, h_hi = gsplit == 1 ? nwalk : min(nwalk, h_lo + HPW);
        const int pos = positions ? positions[tok] : (int)(tok % T) + pos_offset;
        long long cslot = -1;
        if (APPEND) {
            cslot = slot[tok];
            if (cslot >= num_slots) {
                if (lane == 0 && h_lo == 0 && status) atomicMax(status, (int)KB_BAD_INDEX);
                cslot = -1;
            }
        }
        float c[8], sn[8];
        *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cosT + (size_t)pos * HD + e0);
        *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cosT + (size_t)pos * HD + e0 + 4);
        *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sinT + (size_t)pos * HD + e0);
        *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sinT + (size_t)pos * HD + e0 + 4);
        const bf16* src = qkv + (size_t)tok * in_stride;
        bf16* dst = out + (size_t)tok * out_stride;
#pragma unroll 2
        for (int h0 = h_lo; h0 < h_hi; h0 += HPW) {
            const int head = h0 + hsel;
            const bool isv = APPEND && head >= nh && head < nwalk;       // a value head: copied to its page only
            const bool ok = head < nh;
            const bool isq = head < nq;
            float x1[8], x2[8];
            if (ok || isv) {
                unpack8(ld8(src + head * HD + e0), x1);
                unpack8(ld8(src + head * HD + HD / 2 + e0), x2);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) x1[i] = x2[i] = 0.f;
            }
            if (NORM) {
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) ss += x1[i] * x1[i] + x2[i] * x2[i];
#pragma unroll
                for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                const float rs = rsqrtf(ss / HD + eps);
                if (ok && sub == 0) rstd_o[tok * nh + head] = rs;
                if (!isv) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        x1[i] *= rs * (isq ? wq1[i] : wk1[i]);
                        x2[i] *= rs * (isq ? wq2[i] : wk2[i]);
                    }
                }
            } else if (ok && sub == 0) {
                rstd_o[tok * nh + head] = 1.f;
            }
            float o1[8], o2[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                o1[i] = x1[i] * c[i] - x2[i] * sn[i];
                o2[i] = x2[i] * c[i] + x1[i] * sn[i];
            }
            if (ok) {
                st8(dst + head * HD + e0, pack8(o1));
                st8(dst + head * HD + HD / 2 + e0, pack8(o2));
            }
            if (APPEND && cslot >= 0 && (isv || (ok && !isq))) {
                const int kvh = isv ? head - nh : head - nq;
                const size_t at = (((size_t)(cslot / 16) * nkv + kvh) * 16 + (size_t)(cslot % 16)) * HD + e0;
                bf16* page = isv ? v_pages : k_pages;
                st8(page + at, pack8(isv ? x1 : o1));
                st8(page + at + HD / 2, pack8(isv ? x2 : o2));
            }
        }
    }
}

// Backward; per-warp weight-gradient partials go to dw_part[warp_global][2][HD] (q then k).
template <int HD, bool NORM>
__global__ void __launch_bounds__(256, 2)
qknorm_rope_bwd_kernel(const bf16* __restrict__ dqk, const bf16* __restrict__ qkv, const bf16* __restrict__ qw,
                       const bf16* __restrict__ kw, const float* __restrict__ cosT, const float* __restrict__ sinT,
                       const float* __restrict__ rstd_i, bf16* __restrict__ dqkv, float* __restrict__ dw_part, int N,
                       int T, int nq, int nkv, int pos_offset) {
    constexpr int LPH = HD / 16, HPW = 32 / LPH;
    const int nh = nq + nkv;
    const int lane = threadIdx.x & 31, sub = lane % LPH, hsel = lane / LPH, e0 = sub * 8;
    const int full_stride = (nq + 2 * nkv) * HD, qk_stride = nh * HD;
    float wq1[8], wq2[8], wk1[8], wk2[8];
    float aq1[8], aq2[8], ak1[8], ak2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) aq1[i] = aq2[i] = ak1[i] = ak2[i] = 0.f;
    if (NORM) {
        unpack8(ld8(qw + e0), wq1);
        unpack8(ld8(qw + HD / 2 + e0), wq2);
        unpack8(ld8(kw + e0), wk1);
        unpack8(ld8(kw + HD / 2 + e0), wk2);
    }
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long tok = wid; tok < N; tok += nwarps) {
        const int pos = (int)(tok % T) + pos_offset;
        float c[8], sn[8];
        *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cosT + (size_t)pos * HD + e0);
        *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cosT + (size_t)pos * HD + e0 + 4);
        *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sinT + (size_t)pos * HD + e0);
        *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sinT + (size_t)pos * HD + e0 + 4);
        const bf16* gsrc = dqk + (size_t)tok * qk_stride;
        const bf16* xsrc = qkv + (size_t)tok * full_stride;
        bf16* dst = dqkv + (size_t)tok * full_stride;
#pragma unroll 2
        for (int h0 = 0; h0 < nh; h0 += HPW) {
            const int head = h0 + hsel;
            const bool ok = head < nh;
            const bool isq = head < nq;
            float d1[8], d2[8];
            {
                float g1[8], g2[8];
                if (ok) {
                    unpack8(ld8(gsrc + head * HD + e0), g1);
                    unpack8(ld8(gsrc + head * HD + HD / 2 + e0), g2);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) g1[i] = g2[i] = 0.f;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    d1[i] = g1[i] * c[i] + g2[i] * sn[i];
                    d2[i] = g2[i] * c[i] - g1[i] * sn[i];
                }
            }
            if (NORM) {
                float xh1[8], xh2[8];
                float rs = 0.f;
                if (ok) {
                    unpack8(ld8(xsrc + head * HD + e0), xh1);
                    unpack8(ld8(xsrc + head * HD + HD / 2 + e0), xh2);
                    rs = rstd_i[tok * nh + head];
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) xh1[i] = xh2[i] = 0.f;
                }
                const float fq = isq ? 1.f : 0.f, fk = 1.f - fq;       // rows past the last head carry zeros
                float m = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    xh1[i] *= rs;
                    xh2[i] *= rs;
                    const float t1 = d1[i] * xh1[i], t2 = d2[i] * xh2[i];
                    aq1[i] += fq * t1; aq2[i] += fq * t2;
                    ak1[i] += fk * t1; ak2[i] += fk * t2;
                    d1[i] *= isq ? wq1[i] : wk1[i];
                    d2[i] *= isq ? wq2[i] : wk2[i];
                    m += d1[i] * xh1[i] + d2[i] * xh2[i];
                }
#pragma unroll
                for (int o = LPH / 2; o > 0; o >>= 1) m += __shfl_xor_sync(0xffffffffu, m, o);
                m *= 1.f / HD;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    d1[i] = rs * (d1[i] - xh1[i] * m);
                    d2[i] = rs * (d2[i] - xh2[i] * m);
                }
            }
            if (ok) {
                st8(dst + head * HD + e0, pack8(d1));
                st8(dst + head * HD + HD / 2 + e0, pack8(d2));
            }
        }
    }
    if (NORM) {
        // sum the head slots of the warp, then the lanes of slot 0 write this warp's partial row
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int o = LPH; o < 32; o <<= 1) {
                aq1[i] += __shfl_xor_sync(0xffffffffu, aq1[i], o);
                aq2[i] += __shfl_xor_sync(0xffffffffu, aq2[i], o);
                ak1[i] += __shfl_xor_sync(0xffffffffu, ak1[i], o);
                ak2[i] += __shfl_xor_sync(0xffffffffu, ak2[i], o);
            }
        }
        if (hsel == 0) {
            float* p = dw_part + (size_t)wid * 2 * HD;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                p[e0 + i] = aq1[i];
                p[HD / 2 + e0 + i] = aq2[i];
                p[HD + e0 + i] = ak1[i];
                p[HD + HD / 2 + e0 + i] = ak2[i];
            }
        }
    }
}

KB_API int kb_qknorm_grid_warps() { return kb_num_sms() * 8 * 8; }

// `k_pages` non-null: also append to the paged cache (see the kernel); `slot`, `num_slots`, `status` as kb_kv_append.
static int qknorm_rope_fwd_launch(const void* qkv, const void* qw, const void* kw, const float* cosT, const float* sinT,
                                  void* out, float* rstd, int N, int T, int nq, int nkv, int hd, int pos_offset,
                                  float eps, const int* positions, void* k_pages, void* v_pages, const long long* slot,
                                  long long num_slots, int* status, cudaStream_t st) {
    const bool append = k_pages != nullptr;
    if (append && (!v_pages || !slot)) return 5;
    const int nwalk = nq + nkv + (append ? nkv : 0);
    long long blocks = ((long long)N * ((nwalk + 3) / 4) + 7) / 8;       // at most one warp per (token, head group)
    if (blocks > kb_num_sms() * 8) blocks = kb_num_sms() * 8;
    if (blocks < 1) blocks = 1;
    const bool norm = qw != nullptr;
#define QK_FWD(E, NORM, APP) kb_launch_dep(qknorm_rope_fwd_kernel<E, NORM, APP>, dim3((unsigned)blocks), dim3(256), 0, st, \
        (const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, cosT, sinT, (bf16*)out, rstd, N, T, nq, nkv, pos_offset, eps, \
        positions, (bf16*)k_pages, (bf16*)v_pages, slot, num_slots, status)
    if (hd == 128) {
        if (append) return norm ? QK_FWD(128, true, true) : QK_FWD(128, false, true);
        return norm ? QK_FWD(128, true, false) : QK_FWD(128, false, false);
    }
    if (hd == 64) {
        if (append) return norm ? QK_FWD(64, true, true) : QK_FWD(64, false, true);
        return norm ? QK_FWD(64, true, false) : QK_FWD(64, false, false);
    }
    return 5;
}
KB_API int kb_qknorm_rope_fwd(const void* qkv, const void* qw, const void* kw, const float* cosT, const float* sinT,
                              void* out, float* rstd, int N, int T, int nq, int nkv, int hd, int pos_offset,
                              float eps, const int* positions, cudaStream_t st) {
    return qknorm_rope_fwd_launch(qkv, qw, kw, cosT, sinT, out, rstd, N, T, nq, nkv, hd, pos_offset, eps, positions,
                                  nullptr, nullptr, nullptr, 0, nullptr, st);
}
// QK-norm + RoPE and the cache append of the new tokens in one launch (serving).
KB_API int kb_qknorm_rope_append(const void* qkv, const void* qw, const void* kw, const float* cosT, const float* sinT,
                                 void* out, float* rstd, int N, int T, int nq, int nkv, int hd, int pos_offset,
                                 float eps, const int* positions, void* k_pages, void* v_pages, const long long* slot,
                                 long long num_slots, int* status, cudaStream_t st) {
    if (!k_pages) return 5;
    return qknorm_rope_fwd_launch(qkv, qw, kw, cosT, sinT, out, rstd, N, T, nq, nkv, hd, pos_offset, eps, positions,
                                  k_pages, v_pages, slot, num_slots, status, st);
}

KB_API int kb_qknorm_rope_bwd(const void* dqk, const void* qkv, const void* qw, const void* kw, const float* cosT,
                              const float* sinT, const float* rstd, void* dqkv, float* dw_part, int N, int T, int nq,
                              int nkv, int hd, int pos_offset, cudaStream_t st) {
    const int blocks = kb_num_sms() * 8;  // 8 warps each -> kb_qknorm_grid_warps() partial rows
    const bool norm = qw != nullptr;
#define QK_BWD(E, NORM) qknorm_rope_bwd_kernel<E, NORM><<<blocks, 256, 0, st>>>( \
        (const bf16*)dqk, (const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, cosT, sinT, rstd, (bf16*)dqkv, dw_part, \
        N, T, nq, nkv, pos_offset)
    if (hd == 128) { if (norm) QK_BWD(128, true); else QK_BWD(128, false); }
    else if (hd == 64) { if (norm) QK_BWD(64, true); else QK_BWD(64, false); }
    else return 5;
    return kb_launch_status();
}

// ============================================================================ SwiGLU
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ act, long long N, int F) {
    kb_dep_trigger();
    kb_dep_wait();
    const int fc = F >> 3;
    const long long total = N * fc;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / fc;
        const int c = (int)(i % fc);
        float g[8], u[8], o[8];
        unpack8(ld8(gu + row * 2 * F + (size_t)c * 8), g);
        unpack8(ld8(gu + row * 2 * F + F + (size_t)c * 8), u);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
        st8(act + row * F + (size_t)c * 8, pack8(o));
    }
}
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ gu, const bf16* __restrict__ dact,
                                  bf16* __restrict__ dgu, long long N, int F) {
    const int fc = F >> 3;
    const long long total = N * fc;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / fc;
        const int c = (int)(i % fc);
        float g[8], u[8], d[8], dg[8], du[8];
        unpack8(ld8(gu + row * 2 * F + (size_t)c * 8), g);
        unpack8(ld8(gu + row * 2 * F + F + (size_t)c * 8), u);
        unpack8(ld8(dact + row * F + (size_t)c * 8), d);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float sg = 1.f / (1.f + __expf(-g[j]));
            dg[j] = d[j] * u[j] * sg * (1.f + g[j] * (1.f - sg));
            du[j] = d[j] * g[j] * sg;
        }
        st8(dgu + row * 2 * F + (size_t)c * 8, pack8(dg));
        st8(dgu + row * 2 * F + F + (size_t)c * 8, pack8(du));
    }
}
static inline int ew_grid(long long work, int threads) {
    long long b = (work + threads - 1) / threads;
    const long long cap = (long long)kb_num_sms() * 16;
    return (int)(b < cap ? (b < 1 ? 1 : b) : cap);
}
KB_API int kb_swiglu_fwd(const void* gu, void* act, long long N, int F, cudaStream_t st) {
    if (F % 8) return 5;
    return kb_launch_dep(swiglu_fwd_kernel, dim3(ew_grid(N * (F / 8), 256)), dim3(256), 0, st, (const bf16*)gu, (bf16*)act, N, F);
}
KB_API int kb_swiglu_bwd(const void* gu, const void* dact, void* dgu, long long N, int F, cudaStream_t st) {
    if (F % 8) return 5;
    swiglu_bwd_kernel<<<ew_grid(N * (F / 8), 256), 256, 0, st>>>((const bf16*)gu, (const bf16*)dact, (bf16*)dgu, N, F);
    return kb_launch_status();
}

// ============================================================================ CE + z-loss
// One block per row of a bf16 logits chunk; the chunk is overwritten with the gradient of
// scale * (ce + z_w * lse^2) / n_valid.  Per-row ce and lse^2 go to row_ce / row_z (0 for
// ignored rows).  inv_count points to 1/n_valid on the device.
__global__ void __launch_bounds__(512)
ce_zloss_kernel(bf16* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ row_ce,
                float* __restrict__ row_z, const float* __restrict__ inv_count, float z_w, float scale, int V,
                int write_grad, int* __restrict__ status) {
    __shared__ float scratch[2 * 32];
    const int row = blockIdx.x;
    bf16* lg = logits + (size_t)row * V;
    long long y = labels[row];
    if (y >= V) {
        // a label outside the vocabulary: recorded, and the row is treated as ignored (negative labels are the ignore index)
        if (threadIdx.x == 0 && status) atomicMax(status, (int)KB_BAD_INDEX);
        y = -1;
    }
    const int nchunks = V >> 3;
    float mx = -INFINITY, se = 0.f;
    for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
        float t[8];
        unpack8(ld8(lg + (size_t)c * 8), t);
        float lm = t[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) lm = fmaxf(lm, t[i]);
        if (lm > mx) { se *= __expf(mx - lm); mx = lm; }
#pragma unroll
        for (int i = 0; i < 8; ++i) se += __expf(t[i] - mx);
    }
    // combine (mx, se) across the block
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, mx, o), os = __shfl_xor_sync(0xffffffffu, se, o);
        const float nm = fmaxf(mx, om);
        se = (mx == -INFINITY ? 0.f : se * __expf(mx - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
        mx = nm;
    }
    if (lane == 0) { scratch[warp] = mx; scratch[32 + warp] = se; }
    __syncthreads();
    mx = lane < nwarp ? scratch[lane] : -INFINITY;
    se = lane < nwarp ? scratch[32 + lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, mx, o), os = __shfl_xor_sync(0xffffffffu, se, o);
        const float nm = fmaxf(mx, om);
        se = (mx == -INFINITY ? 0.f : se * __expf(mx - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
        mx = nm;
    }
    const float lse = mx + logf(se);
    const bool valid = y >= 0;
    if (threadIdx.x == 0) {
        const float ty = valid ? __bfloat162float(lg[y]) : 0.f;
        row_ce[row] = valid ? lse - ty : 0.f;
        row_z[row] = valid ? lse * lse : 0.f;
    }
    if (!write_grad) return;
    __syncthreads();  // the target logit was read above before anyone overwrites it
    const float k = valid ? scale * inv_count[0] : 0.f;
    const float pf = k * (1.f + 2.f * z_w * lse);
    for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
        float t[8];
        unpack8(ld8(lg + (size_t)c * 8), t);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float g = pf * __expf(t[i] - lse);
            if ((long long)c * 8 + i == y) g -= k;
            t[i] = g;
        }
        st8(lg + (size_t)c * 8, pack8(t));
    }
}
KB_API int kb_ce_zloss(void* logits, const long long* labels, float* row_ce, float* row_z, const float* inv_count,
                       float z_w, float scale, int rows, int V, int write_grad, int* status, cudaStream_t st) {
    if (V % 8) return 5;
    ce_zloss_kernel<<<rows, 512, 0, st>>>((bf16*)logits, labels, row_ce, row_z, inv_count, z_w, scale, V, write_grad,
                                          status);
    return kb_launch_status();
}

// ============================================================================ embedding
// Token ids come from data: an id outside [0, V) is recorded in the status word (KB_BAD_INDEX) and
// its row is written as zeros (forward) or skipped (backward) instead of being dereferenced.
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ w,
                                     bf16* __restrict__ out, int N, int D, int V, int* __restrict__ status) {
    const int dc = D >> 3;
    const long long total = (long long)N * dc;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / dc;
        const int c = (int)(i % dc);
        const long long id = ids[row];
        if (id < 0 || id >= V) {
            if (c == 0 && status) atomicMax(status, (int)KB_BAD_INDEX);
            *reinterpret_cast<uint4*>(out + row * D + (size_t)c * 8) = make_uint4(0, 0, 0, 0);
            continue;
        }
        st8(out + row * D + (size_t)c * 8, ld8(w + id * D + (size_t)c * 8));
    }
}
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ dout,
                                     bf16* __restrict__ dw, int N, int D, int V, int* __restrict__ status) {
    const int dc = D >> 1;
    const long long total = (long long)N * dc;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / dc;
        const int c = (int)(i % dc);
        const long long id = ids[row];
        if (id < 0 || id >= V) {
            if (c == 0 && status) atomicMax(status, (int)KB_BAD_INDEX);
            continue;
        }
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(dout + row * D + (size_t)c * 2);
        atomicAdd(reinterpret_cast<__nv_bfloat162*>(dw + id * D + (size_t)c * 2), v);
    }
}
KB_API int kb_embedding_fwd(const long long* ids, const void* w, void* out, int N, int D, int V, int* status,
                            cudaStream_t st) {
    if (D % 8 || V < 1) return 5;
    embedding_fwd_kernel<<<ew_grid((long long)N * (D / 8), 256), 256, 0, st>>>(ids, (const bf16*)w, (bf16*)out, N, D, V,
                                                                              status);
    return kb_launch_status();
}
KB_API int kb_embedding_bwd(const long long* ids, const void* dout, void* dw, int N, int D, int V, int* status,
                            cudaStream_t st) {
    if (D % 2 || V < 1) return 5;
    embedding_bwd_kernel<<<ew_grid((long long)N * (D / 2), 256), 256, 0, st>>>(ids, (const bf16*)dout, (bf16*)dw, N, D, V,
                                                                              status);
    return kb_launch_status();
}

// ============================================================================ reductions
// Deterministic two-stage sum of squares: partial[gridDim] then a single block.
template <typename T>
__device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<bf16>(bf16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }

template <typename T>
__global__ void sumsq_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ partial) {
    __shared__ float scratch[32];
    float acc[1] = {0.f};
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = to_f<T>(x[i]);
        acc[0] += v * v;
    }
    block_sum<1>(acc, scratch);
    if (threadIdx.x == 0) partial[blockIdx.x] = acc[0];
}
__global__ void sum_final_kernel(const float* __restrict__ partial, int n, float* __restrict__ out, int accumulate) {
    __shared__ float scratch[32];
    float acc[1] = {0.f};
    for (int i = threadIdx.x; i < n; i += blockDim.x) acc[0] += partial[i];
    block_sum<1>(acc, scratch);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + acc[0] : acc[0];
}
// dtype: 0 bf16, 1 fp16, 2 fp32.  `partial` needs 1024 floats.
KB_API int kb_sumsq(const void* x, long long n, int dtype, float* partial, float* out, int accumulate,
                    cudaStream_t st) {
    const int grid = 1024;
    if (dtype == 0) sumsq_partial_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)x, n, partial);
    else if (dtype == 1) sumsq_partial_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, n, partial);
    else sumsq_partial_kernel<float><<<grid, 256, 0, st>>>((const float*)x, n, partial);
    sum_final_kernel<<<1, 256, 0, st>>>(partial, grid, out, accumulate);
    return kb_launch_status();
}
KB_API int kb_sum_f32(const float* x, int n, float* out, cudaStream_t st) {
    sum_final_kernel<<<1, 256, 0, st>>>(x, n, out, 0);
    return kb_launch_status();
}

// ============================================================================ optimizers
// AdamW on a flat bf16 parameter range with fp32 moments; gscale is a device scalar (clip coefficient).
__global__ void adamw_kernel(bf16* __restrict__ p, const bf16* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, long long n, const float* __restrict__ gscale, float lr, float b1,
                             float b2, float eps, float wd, float bc1, float bc2_sqrt) {
    const float gs = gscale ? gscale[0] : 1.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float gi = __bfloat162float(g[i]) * gs;
        const float mi = b1 * m[i] + (1.f - b1) * gi;
        const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
        m[i] = mi;
        v[i] = vi;
        float pi = __bfloat162float(p[i]) * (1.f - lr * wd);
        pi -= (lr / bc1) * mi / (sqrtf(vi) / bc2_sqrt + eps);
        p[i] = __float2bfloat16(pi);
    }
}
KB_API int kb_adamw(void* p, const void* g, float* m, float* v, long long n, const float* gscale, float lr, float b1,
                    float b2, float eps, float wd, int step, cudaStream_t st) {
    const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
    adamw_kernel<<<ew_grid(n, 256), 256, 0, st>>>((bf16*)p, (const bf16*)g, m, v, n, gscale, lr, b1, b2, eps, wd, bc1,
                                                 sqrtf(bc2));
    return kb_launch_status();
}

// Muon momentum: buf = mom*buf + g*gs (bf16), x = (nesterov ? mom*buf + g*gs : buf) as fp16,
// plus per-block partial sums of x^2 into partial[gridDim] (grid fixed at 1024).
__global__ void muon_momentum_kernel(const bf16* __restrict__ g, bf16* __restrict__ buf, __half* __restrict__ x,
                                     long long n, const float* __restrict__ gscale, float mom, int nesterov,
                                     float* __restrict__ partial) {
    __shared__ float scratch[32];
    const float gs = gscale ? gscale[0] : 1.f;
    float acc[1] = {0.f};
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float gi = __bfloat162float(__float2bfloat16(__bfloat162float(g[i]) * gs));
        const float b = __bfloat162float(__float2bfloat16(mom * __bfloat162float(buf[i]) + gi));
        buf[i] = __float2bfloat16(b);
        const float u = nesterov ? __bfloat162float(__float2bfloat16(mom * b + gi)) : b;
        const __half h = __float2half(u);
        x[i] = h;
        const float hf = __half2float(h);
        acc[0] += hf * hf;
    }
    block_sum<1>(acc, scratch);
    if (threadIdx.x == 0) partial[blockIdx.x] = acc[0];
}
KB_API int kb_muon_momentum(const void* g, void* buf, void* x, long long n, const float* gscale, float mom,
                            int nesterov, float* partial, float* sumsq_out, cudaStream_t st) {
    muon_momentum_kernel<<<1024, 256, 0, st>>>((const bf16*)g, (bf16*)buf, (__half*)x, n, gscale, mom, nesterov, partial);
    sum_final_kernel<<<1, 256, 0, st>>>(partial, 1024, sumsq_out, 0);
    return kb_launch_status();
}

// x *= 1/(sqrt(sumsq)+1e-7)   (fp16, in place)
__global__ void ns_normalize_kernel(__half* __restrict__ x, long long n, const float* __restrict__ sumsq) {
    const float inv = 1.f / (sqrtf(sumsq[0]) + 1e-7f);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = __float2half(__half2float(x[i]) * inv);
}
KB_API int kb_ns_normalize(void* x, long long n, const float* sumsq, cudaStream_t st) {
    ns_normalize_kernel<<<ew_grid(n, 256), 256, 0, st>>>((__half*)x, n, sumsq);
    return kb_launch_status();
}

// p = p*(1-lr*wd) - lr*scale*orth   (p bf16 [R,C]; orth fp16 [R,C] or [C,R] when transposed)
__global__ void muon_apply_kernel(bf16* __restrict__ p, const __half* __restrict__ o, int R, int C, float decay,
                                  float alpha, int transposed) {
    __shared__ float tile[32][33];
    const int bx = blockIdx.x * 32, by = blockIdx.y * 32;
    if (transposed) {
        // o is [C,R]: read tile rows along C
        for (int j = threadIdx.y; j < 32; j += blockDim.y) {
            const int oc = bx + j, orow = by + threadIdx.x;  // o[oc][orow]
            tile[j][threadIdx.x] = (oc < C && orow < R) ? __half2float(o[(size_t)oc * R + orow]) : 0.f;
        }
        __syncthreads();
        for (int j = threadIdx.y; j < 32; j += blockDim.y) {
            const int r = by + j, c = bx + threadIdx.x;
            if (r < R && c < C) {
                const size_t idx = (size_t)r * C + c;
                p[idx] = __float2bfloat16(__bfloat162float(p[idx]) * decay - alpha * tile[threadIdx.x][j]);
            }
        }
    } else {
        for (int j = threadIdx.y; j < 32; j += blockDim.y) {
            const int r = by + j, c = bx + threadIdx.x;
            if (r < R && c < C) {
                const size_t idx = (size_t)r * C + c;
                p[idx] = __float2bfloat16(__bfloat162float(p[idx]) * decay - alpha * __half2float(o[idx]));
            }
        }
    }
}
KB_API int kb_muon_apply(void* p, const void* orth, int R, int C, float lr, float wd, float scale, int transposed,
                         cudaStream_t st) {
    dim3 grid((C + 31) / 32, (R + 31) / 32), block(32, 8);
    muon_apply_kernel<<<grid, block, 0, st>>>((bf16*)p, (const __half*)orth, R, C, wd > 0 ? 1.f - lr * wd : 1.f,
                                              lr * scale, transposed);
    return kb_launch_status();
}

// out[C,R] = in[R,C]^T for 16-bit elements.
__global__ void transpose16_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int R, int C) {
    __shared__ uint16_t tile[64][66];
    const int bx = blockIdx.x * 64, by = blockIdx.y * 64;
    for (int j = threadIdx.y; j < 64; j += blockDim.y) {
        const int r = by + j;
        for (int i = threadIdx.x; i < 64; i += blockDim.x) {
            const int c = bx + i;
            tile[j][i] = (r < R && c < C) ? in[(size_t)r * C + c] : (uint16_t)0;
        }
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 64; j += blockDim.y) {
        const int c = bx + j;
        for (int i = threadIdx.x; i < 64; i += blockDim.x) {
            const int r = by + i;
            if (r < R && c < C) out[(size_t)c * R + r] = tile[i][j];
        }
    }
}
KB_API int kb_transpose16(const void* in, void* out, int R, int C, cudaStream_t st) {
    dim3 grid((C + 63) / 64, (R + 63) / 64), block(32, 8);
    transpose16_kernel<<<grid, block, 0, st>>>((const uint16_t*)in, (uint16_t*)out, R, C);
    return kb_launch_status();
}

// y = a*x + y_scale*y style helpers for Newton-Schulz epilogues done outside the GEMM (fp16).
__global__ void axpby_half_kernel(__half* __restrict__ y, const __half* __restrict__ x, long long n, float a, float b) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        y[i] = __float2half(a * __half2float(x[i]) + b * __half2float(y[i]));
}
KB_API int kb_axpby_half(void* y, const void* x, long long n, float a, float b, cudaStream_t st) {
    axpby_half_kernel<<<ew_grid(n, 256), 256, 0, st>>>((__half*)y, (const __half*)x, n, a, b);
    return kb_launch_status();
}

// Mirror the upper triangle of square 16-bit matrices into the lower one: A[i][j] = A[j][i], i > j.
// 64x64 tiles; only tiles on or below the diagonal do work.  Batched with a fixed stride.
__global__ void mirror_upper16_kernel(uint16_t* __restrict__ a, int R, long long ld, long long batch_stride) {
    __shared__ uint16_t tile[64][66];
    const int ti = blockIdx.y, tj = blockIdx.x;      // destination tile (rows ti, cols tj), tj <= ti
    if (tj > ti) return;
    uint16_t* base = a + (long long)blockIdx.z * batch_stride;
    // source tile is (tj, ti): rows tj*64.., cols ti*64..
    for (int j = threadIdx.y; j < 64; j += blockDim.y) {
        const int r = tj * 64 + j;
        for (int i = threadIdx.x; i < 64; i += blockDim.x) {
            const int c = ti * 64 + i;
            tile[j][i] = (r < R && c < R) ? base[(long long)r * ld + c] : (uint16_t)0;
        }
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 64; j += blockDim.y) {
        const int r = ti * 64 + j;
        for (int i = threadIdx.x; i < 64; i += blockDim.x) {
            const int c = tj * 64 + i;
            if (r < R && c < R && r > c) base[(long long)r * ld + c] = tile[i][j];
        }
    }
}
KB_API int kb_mirror_upper16(void* a, int R, long long ld, int batch, long long batch_stride, cudaStream_t st) {
    dim3 grid((R + 63) / 64, (R + 63) / 64, batch), block(32, 8);
    mirror_upper16_kernel<<<grid, block, 0, st>>>((uint16_t*)a, R, ld, batch_stride);
    return kb_launch_status();
}

// dst = bf16(src + beta * addend)  (addend optional): finishes a split-K GEMM.  With `rezero` the
// fp32 workspace is cleared on the way out, so the next split-K product that accumulates into it
// needs no separate fill.
__global__ void f32_to_bf16_add_kernel(float* __restrict__ src, const bf16* __restrict__ addend, float beta,
                                       bf16* __restrict__ dst, long long n, int rezero) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = src[i];
        if (rezero) src[i] = 0.f;
        if (addend) v += beta * __bfloat162float(addend[i]);
        dst[i] = __float2bfloat16(v);
    }
}
KB_API int kb_f32_to_bf16_add(float* src, const void* addend, float beta, void* dst, long long n, int rezero,
                              cudaStream_t st) {
    f32_to_bf16_add_kernel<<<ew_grid(n, 256), 256, 0, st>>>(src, (const bf16*)addend, beta, (bf16*)dst, n, rezero);
    return kb_launch_status();
}

KB_API int kb_last_error() { return (int)cudaGetLastError(); }
