// AttnRes depth routing fused with the following RMSNorm, forward and backward, as a
// bulk-copy pipeline: one thread of a persistent CTA streams each token's source rows
// (and, for the backward, the incoming gradient row) into a multi-stage shared-memory ring
// with cp.async.bulk + mbarrier transaction counts, while all threads compute on the
// previous token.  Bytes in flight are set by the ring, not by registers, which is what
// lets a 6-way-warp CTA keep HBM busy.
//
// Math (per token, sources u_1..u_S, w = query * key_norm_weight):
//   r_s = rsqrt(mean(u_s^2)+eps), l_s = (u_s.w) r_s, a = softmax(l), h = sum a_s u_s,
//   out = h * rsqrt(mean(h^2)+eps) * norm_weight            (reference: src/model/llama.py:630-644)
// Backward as in src/model/flash_attn_res/kernels/phase_1.py:204-249 plus the RMSNorm
// backward; source gradients are accumulated in place, weight gradients leave as per-CTA
// partial rows that a column-sum kernel reduces deterministically.
#include <stdlib.h>

#include "tc.cuh"

typedef __nv_bfloat16 bf16;

namespace {

struct RouteSrcs {
    const bf16* p[16];
};
struct RouteDsts {
    bf16* p[16];
    unsigned acc_mask;
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

constexpr int MAX_STAGES = 4;

// Shared-memory layout: [stages][rows][D] bf16, then barriers.
template <int MAXS, int CPT, bool BWD>
__global__ void __launch_bounds__(BWD ? 384 : 256)
route_pipe_kernel(RouteSrcs srcs, RouteDsts dsts, int S, const bf16* __restrict__ dxn, const bf16* __restrict__ q,
                  const bf16* __restrict__ rn_w, const bf16* __restrict__ n_w, bf16* __restrict__ xn,
                  float* __restrict__ alpha_g, float* __restrict__ r_g, float* __restrict__ logit_g,
                  float* __restrict__ rstd_g, float* __restrict__ dw_part, float* __restrict__ dnw_part, int N, int D,
                  float eps, int stages, int* status) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float scratch[2 * MAXS * 32];
    __shared__ uint64_t full[MAX_STAGES];
    __shared__ int abort_flag;
    const int rows = S + (BWD ? 1 : 0);
    const uint32_t row_bytes = (uint32_t)D * 2;
    const int nchunks = D >> 3;
    const float invD = 1.f / (float)D;
    const bool routing = q != nullptr;
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) tc::mbar_init(&full[s], 1);
        abort_flag = 0;
        tc::fence_barrier_init();
    }
    __syncthreads();
    kb_dep_trigger();
    kb_dep_wait();                      // the sources are what the kernels before this one wrote
    const int my_tokens = blockIdx.x < N ? (N - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    auto issue = [&](int it) {
        const int st = it % stages;
        const size_t tok = (size_t)blockIdx.x + (size_t)it * gridDim.x;
        uint8_t* base = smem + (size_t)st * rows * row_bytes;
        tc::mbar_expect_tx(&full[st], rows * row_bytes);
        for (int s = 0; s < S; ++s) bulk_g2s(base + (size_t)s * row_bytes, srcs.p[s] + tok * D, row_bytes, &full[st]);
        if (BWD) bulk_g2s(base + (size_t)S * row_bytes, dxn + tok * D, row_bytes, &full[st]);
    };
    if (threadIdx.x == 0) {
        for (int it = 0; it < stages && it < my_tokens; ++it) issue(it);
    }
    float dw_acc[CPT][8], dnw_acc[CPT][8];
    if (BWD) {
#pragma unroll
        for (int k = 0; k < CPT; ++k)
#pragma unroll
            for (int i = 0; i < 8; ++i) dw_acc[k][i] = dnw_acc[k][i] = 0.f;
    }

    for (int it = 0; it < my_tokens; ++it) {
        const int st = it % stages;
        const uint32_t parity = (it / stages) & 1;
        const size_t tok = (size_t)blockIdx.x + (size_t)it * gridDim.x;
        if (!tc::mbar_wait(&full[st], parity, &abort_flag)) {
            if (threadIdx.x == 0) atomicMax(status, (int)KB_TIMEOUT_TMA);
            break;
        }
        const bf16* u = reinterpret_cast<const bf16*>(smem + (size_t)st * rows * row_bytes);
        float al[MAXS], rr[MAXS], lg[MAXS];
        if (!BWD) {
            if (routing) {
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
                                unpack8(ld8(u + (size_t)s * D + c * 8), t);
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
                float mx = -INFINITY;
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
                if (threadIdx.x < S) {
                    // each of the first S threads stores the statistics of one source
#pragma unroll
                    for (int s = 0; s < MAXS; ++s) {
                        if (s == (int)threadIdx.x) {
                            alpha_g[tok * S + s] = al[s];
                            r_g[tok * S + s] = rr[s];
                            logit_g[tok * S + s] = lg[s];
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
                const int c = threadIdx.x + k * blockDim.x;
#pragma unroll
                for (int i = 0; i < 8; ++i) h[k][i] = 0.f;
                if (c < nchunks) {
#pragma unroll
                    for (int s = 0; s < MAXS; ++s) {
                        if (s < S) {
                            float t[8];
                            unpack8(ld8(u + (size_t)s * D + c * 8), t);
#pragma unroll
                            for (int i = 0; i < 8; ++i) h[k][i] += al[s] * t[i];
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) hsq[0] += h[k][i] * h[k][i];
            }
            block_sum<1>(hsq, scratch);     // also: every thread is done reading this stage
            if (threadIdx.x == 0 && it + stages < my_tokens) issue(it + stages);
            const float rs = rsqrtf(hsq[0] * invD + eps);
            if (threadIdx.x == 0) rstd_g[tok] = rs;
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const int c = threadIdx.x + k * blockDim.x;
                if (c < nchunks) {
                    float w[8], o[8];
                    unpack8(ld8(n_w + c * 8), w);
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = h[k][i] * rs * w[i];
                    st8(xn + tok * D + (size_t)c * 8, pack8(o));
                }
            }
        } else {
            // ------------------------------------------------------------ backward
#pragma unroll
            for (int s = 0; s < MAXS; ++s) {
                if (routing && s < S) {
                    al[s] = alpha_g[tok * S + s];
                    rr[s] = r_g[tok * S + s];
                    lg[s] = logit_g[tok * S + s];
                } else {
                    al[s] = (!routing && s == 0) ? 1.f : 0.f;
                    rr[s] = 0.f;
                    lg[s] = 0.f;
                }
            }
            const float rs = rstd_g[tok];
            const bf16* gx = u + (size_t)S * D;
            float hn[CPT][8], dh[CPT][8];
            float c1[1] = {0.f};
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const int c = threadIdx.x + k * blockDim.x;
#pragma unroll
                for (int i = 0; i < 8; ++i) { hn[k][i] = 0.f; dh[k][i] = 0.f; }
                if (c < nchunks) {
#pragma unroll
                    for (int s = 0; s < MAXS; ++s) {
                        if (s < S) {
                            float t[8];
                            unpack8(ld8(u + (size_t)s * D + c * 8), t);
#pragma unroll
                            for (int i = 0; i < 8; ++i) hn[k][i] += al[s] * t[i];
                        }
                    }
                    float g[8], w[8];
                    unpack8(ld8(gx + c * 8), g);
                    unpack8(ld8(n_w + c * 8), w);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        hn[k][i] *= rs;
                        dnw_acc[k][i] += g[i] * hn[k][i];
                        dh[k][i] = g[i] * w[i];
                        c1[0] += dh[k][i] * hn[k][i];
                    }
                }
            }
            block_sum<1>(c1, scratch);
            const float m = c1[0] * invD;
#pragma unroll
            for (int k = 0; k < CPT; ++k)
#pragma unroll
                for (int i = 0; i < 8; ++i) dh[k][i] = rs * (dh[k][i] - hn[k][i] * m);
            // accumulate-targets of the first chunk are fetched now, so that the loads fly during
            // the reduction below
            bf16x8 old0[MAXS];
            {
                const int c = threadIdx.x;
                if (c < nchunks) {
#pragma unroll
                    for (int s = 0; s < MAXS; ++s)
                        if (s < S && (dsts.acc_mask >> s & 1u)) old0[s] = ld8(dsts.p[s] + tok * D + (size_t)c * 8);
                }
            }
            float dl[MAXS];
            if (routing) {
                float a[MAXS];
#pragma unroll
                for (int s = 0; s < MAXS; ++s) a[s] = 0.f;
#pragma unroll
                for (int k = 0; k < CPT; ++k) {
                    const int c = threadIdx.x + k * blockDim.x;
                    if (c < nchunks) {
#pragma unroll
                        for (int s = 0; s < MAXS; ++s) {
                            if (s < S) {
                                float t[8];
                                unpack8(ld8(u + (size_t)s * D + c * 8), t);
#pragma unroll
                                for (int i = 0; i < 8; ++i) a[s] += dh[k][i] * t[i];
                            }
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
                // read every accumulate-target first so the loads overlap
                bf16x8 old[MAXS];
#pragma unroll
                for (int s = 0; s < MAXS; ++s) {
                    if (s < S && (dsts.acc_mask >> s & 1u))
                        old[s] = k == 0 ? old0[s] : ld8(dsts.p[s] + tok * D + (size_t)c * 8);
                }
#pragma unroll
                for (int s = 0; s < MAXS; ++s) {
                    if (s < S) {
                        float t[8], du[8];
                        unpack8(ld8(u + (size_t)s * D + c * 8), t);
                        const float c_w = dl[s] * rr[s];
                        const float c_u = dl[s] * lg[s] * rr[s] * rr[s] * invD;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            du[i] = al[s] * dh[k][i] + c_w * w[i] - c_u * t[i];
                            dw_acc[k][i] += c_w * t[i];
                        }
                        if (dsts.acc_mask >> s & 1u) {
                            float o[8];
                            unpack8(old[s], o);
#pragma unroll
                            for (int i = 0; i < 8; ++i) du[i] += o[i];
                        }
                        st8(dsts.p[s] + tok * D + (size_t)c * 8, pack8(du));
                    }
                }
            }
            __syncthreads();                 // every thread is done reading this stage
            if (threadIdx.x == 0 && it + stages < my_tokens) issue(it + stages);
        }
    }
    if (BWD) {
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
    // copies still in flight must land before the CTA's shared memory is released
    if (threadIdx.x == 0 && abort_flag) {
        for (int s = 0; s < stages; ++s) {
            const uint64_t t0 = global_timer_ns();
            while (!tc::mbar_try_wait(&full[s], 0) && !tc::mbar_try_wait(&full[s], 1) &&
                   global_timer_ns() - t0 < 2000000ull) {}
        }
    }
}

int num_sms() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

struct PipeCfg {
    int cpt, threads, stages, ctas_per_sm;
    size_t smem;
    bool ok;
};

PipeCfg pipe_cfg(int S, int D, bool bwd) {
    PipeCfg c{};
    const int nchunks = D / 8;
    const int max_threads = bwd ? 384 : 256;      // 384 x 8 elements = D 3072 in one pass; leaves 170 registers per thread
    c.cpt = (nchunks + max_threads - 1) / max_threads;
    c.threads = ((nchunks + c.cpt - 1) / c.cpt + 31) / 32 * 32;
    const size_t stage = (size_t)(S + (bwd ? 1 : 0)) * D * 2;
    const size_t budget = 200 * 1024;
    c.ok = stage <= budget;
    if (!c.ok) return c;
    // The kernels are bound by instruction issue at low occupancy, so resident warps count for
    // more than ring depth: as many CTAs per SM as shared memory allows (up to 4 forward, where
    // registers permit), each with whatever stages are left.  KB_ROUTE_CTAS overrides (tuning).
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("KB_ROUTE_CTAS");
        forced = e ? atoi(e) : 0;
    }
    int want = bwd ? 1 : 4;
    if (forced > 0) want = forced;
    int fit = (int)(budget / stage);
    c.ctas_per_sm = want < fit ? want : fit;
    if (c.ctas_per_sm < 1) c.ctas_per_sm = 1;
    c.stages = (int)((budget / c.ctas_per_sm) / stage);
    if (c.stages < 1) c.stages = 1;
    if (c.stages > MAX_STAGES) c.stages = MAX_STAGES;
    c.smem = stage * c.stages;
    return c;
}

}  // namespace

#define PIPE_CASE(MAXS_, CPT_)                                                                              \
    {                                                                                                       \
        auto kern = route_pipe_kernel<MAXS_, CPT_, BWD>;                                                    \
        static bool attr_flags[64] = {}; /* per instantiation and device */                                \
        bool* attr = kb_device_flag(attr_flags);                                                            \
        if (!attr) return 7;                                                                                \
        if (!*attr) {                                                                                       \
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=      \
                cudaSuccess)                                                                                \
                return 7;                                                                                   \
            *attr = true;                                                                                   \
        }                                                                                                   \
        if (!BWD) /* the forward also runs in decode steps, where launch gaps matter */                     \
            return kb_launch_dep(kern, dim3(grid), dim3(cfg.threads), cfg.smem, st, rs, ds, S,              \
                                 (const bf16*)dxn, (const bf16*)q, (const bf16*)rn_w, (const bf16*)n_w,     \
                                 (bf16*)xn, alpha, r, logit, rstd, dw_part, dnw_part, N, D, eps,            \
                                 cfg.stages, status);                                                       \
        kern<<<grid, cfg.threads, cfg.smem, st>>>(rs, ds, S, (const bf16*)dxn, (const bf16*)q,              \
                                                   (const bf16*)rn_w, (const bf16*)n_w, (bf16*)xn, alpha, r, \
                                                   logit, rstd, dw_part, dnw_part, N, D, eps, cfg.stages,  \
                                                   status);                                                 \
        return kb_launch_status();                                                                          \
    }
#define PIPE_CPT(MAXS_)                   \
    switch (cfg.cpt) {                    \
        case 1: PIPE_CASE(MAXS_, 1)       \
        case 2: PIPE_CASE(MAXS_, 2)       \
        case 3: PIPE_CASE(MAXS_, 3)       \
        case 4: PIPE_CASE(MAXS_, 4)       \
        default: return 5;                \
    }

template <bool BWD>
static int launch_pipe(const void* const* srcs, void* const* dsts, unsigned acc_mask, int S, const void* dxn,
                       const void* q, const void* rn_w, const void* n_w, void* xn, float* alpha, float* r,
                       float* logit, float* rstd, float* dw_part, float* dnw_part, int N, int D, float eps, int grid,
                       int* status, cudaStream_t st) {
    if (S < 1 || S > 16 || D % 8 != 0 || D > 8192) return 5;
    const PipeCfg cfg = pipe_cfg(S, D, BWD);
    if (!cfg.ok) return 8;
    RouteSrcs rs;
    RouteDsts ds;
    for (int s = 0; s < 16; ++s) {
        rs.p[s] = s < S ? (const bf16*)srcs[s] : nullptr;
        ds.p[s] = (BWD && s < S) ? (bf16*)dsts[s] : nullptr;
    }
    ds.acc_mask = acc_mask;
    if (S <= 1) PIPE_CPT(1)
    else if (S <= 2) PIPE_CPT(2)
    else if (S <= 4) PIPE_CPT(4)
    else if (S <= 8) PIPE_CPT(8)
    else if (S <= 12) PIPE_CPT(12)
    else PIPE_CPT(16)
}

// Number of CTAs the pipelined backward uses for N tokens (rows of the partial buffers).
KB_API int kb_route_pipe_grid(int N, int S, int D, int bwd) {
    const PipeCfg cfg = pipe_cfg(S, D, bwd != 0);
    if (!cfg.ok) return 0;
    const int g = num_sms() * cfg.ctas_per_sm;
    return N < g ? N : g;
}

KB_API int kb_route_pipe_fwd(const void* const* srcs, int S, const void* q, const void* rn_w, const void* n_w,
                             void* xn, float* alpha, float* r, float* logit, float* rstd, int N, int D, float eps,
                             int* status, cudaStream_t st) {
    const int grid = kb_route_pipe_grid(N, S, D, 0);
    if (grid <= 0) return 8;
    return launch_pipe<false>(srcs, nullptr, 0, S, nullptr, q, rn_w, n_w, xn, alpha, r, logit, rstd, nullptr, nullptr,
                              N, D, eps, grid, status, st);
}

KB_API int kb_route_pipe_bwd(const void* const* srcs, void* const* dsts, unsigned acc_mask, int S, const void* dxn,
                             const void* q, const void* rn_w, const void* n_w, float* alpha, float* r, float* logit,
                             float* rstd, float* dw_part, float* dnw_part, int N, int D, int* status,
                             cudaStream_t st) {
    const int grid = kb_route_pipe_grid(N, S, D, 1);
    if (grid <= 0) return 8;
    return launch_pipe<true>(srcs, dsts, acc_mask, S, dxn, q, rn_w, n_w, nullptr, alpha, r, logit, rstd, dw_part,
                             dnw_part, N, D, 0.f, grid, status, st);
}
