// AttnRes depth routing in blocked form (reference: serve.py:113-164 and the Triton kernels
// src/model/flash_attn_res/kernels/phase_1.py, phase_2.py): the committed sources of a block do
// not change inside the block, so one phase-1 pass serves every sub-layer query of the block and
// each sub-layer only merges its own partial sum (phase 2), fused with the RMSNorm that follows.
//
//   phase 1 (Q queries, S committed sources u_s, w_q = query_q * key_norm_weight_q):
//     r_s = rsqrt(mean(u_s^2) + eps), l_qs = (u_s . w_q) r_s, lse_q = log sum_s e^{l_qs},
//     o_q = sum_s softmax(l_q)_s u_s
//   phase 2 (one query, partial p):
//     l_p = (p . w) r_p, pi = sigmoid(l_p - lse), h = o + pi (p - o), xn = h rstd(h) norm_weight
//
// Phase 1 streams each token's S source rows (and, backward, the Q incoming gradient rows) into a
// shared-memory ring with cp.async.bulk; the S x Q dot products of a token run on the tensor
// cores (mma.sync m16n8k16: the rows of the ring are both operands, each warp contracts its own
// 256-column slice), everything per element stays on 8-column chunks owned by one thread.
// Phase 2 forward is one warp per token with direct loads; phase 2 backward streams rows through
// a ring like phase 1 because its weight-gradient accumulators pin columns to threads.
// All statistics are fp32, activations and gradients bf16.  Every wait is bounded.
#include <stdlib.h>

#include "tc.cuh"

typedef __nv_bfloat16 bf16;

namespace {

constexpr int MAXQ = 8;          // queries per phase-1 launch
constexpr int MAXS = 8;          // committed sources per phase-1 launch
constexpr int KSW = 16;          // 16-column contraction steps per warp (warp slice = 256 columns)
constexpr int RB_STAGES = 4;
constexpr int RB_DYN_SMEM = 200 * 1024;   // dynamic shared memory of the ring kernels (their static tables take another 23 KB)

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

int rb_num_sms() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// ------------------------------------------------------------------------------------------------
// phase 2 forward: one warp per token
// ------------------------------------------------------------------------------------------------
template <int NCH>   // 16-byte chunks per lane: NCH * 256 >= D
__global__ void __launch_bounds__(256, NCH <= 16 ? 2 : 1)
route_p2_fwd_kernel(const bf16* __restrict__ o, const float* __restrict__ lse, const bf16* __restrict__ part,
                    const float* __restrict__ w, const bf16* __restrict__ n_w, bf16* __restrict__ xn,
                    float* __restrict__ stats2, int N, int D, float eps) {
    const int lane = threadIdx.x & 31;
    const int wpc = blockDim.x >> 5;
    const int nchunks = D >> 3;
    const float invD = 1.f / (float)D;
    for (long long tok = (long long)blockIdx.x * wpc + (threadIdx.x >> 5); tok < N; tok += (long long)gridDim.x * wpc) {
        bf16x8 vo[NCH], vp[NCH];
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const int c = lane + 32 * k;
            if (c < nchunks) {
                vo[k] = ld8(o + tok * D + (size_t)c * 8);
                if (part) vp[k] = ld8(part + tok * D + (size_t)c * 8);
            }
        }
        float pi = 0.f, lp = 0.f, rp = 0.f;
        if (part) {
            float ss = 0.f, dot = 0.f;
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const int c = lane + 32 * k;
                if (c < nchunks) {
                    float pf[8];
                    unpack8(vp[k], pf);
                    const float4 w0 = *reinterpret_cast<const float4*>(w + c * 8);
                    const float4 w1 = *reinterpret_cast<const float4*>(w + c * 8 + 4);
                    const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        ss += pf[i] * pf[i];
                        dot += pf[i] * wf[i];
                    }
                }
            }
            ss = warp_sum(ss);
            dot = warp_sum(dot);
            rp = rsqrtf(ss * invD + eps);
            lp = dot * rp;
            pi = 1.f / (1.f + __expf(lse[tok] - lp));
        }
        float hs = 0.f;
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const int c = lane + 32 * k;
            if (c < nchunks) {
                float of[8], pf[8];
                unpack8(vo[k], of);
                if (part) {
                    unpack8(vp[k], pf);
#pragma unroll
                    for (int i = 0; i < 8; ++i) of[i] += pi * (pf[i] - of[i]);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) hs += of[i] * of[i];
            }
        }
        hs = warp_sum(hs);
        const float rstd = rsqrtf(hs * invD + eps);
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const int c = lane + 32 * k;
            if (c < nchunks) {
                float of[8], pf[8], nw[8];
                unpack8(vo[k], of);
                if (part) {
                    unpack8(vp[k], pf);
#pragma unroll
                    for (int i = 0; i < 8; ++i) of[i] += pi * (pf[i] - of[i]);
                }
                unpack8(ld8(n_w + c * 8), nw);
#pragma unroll
                for (int i = 0; i < 8; ++i) of[i] *= rstd * nw[i];
                st8(xn + tok * D + (size_t)c * 8, pack8(of));
            }
        }
        if (lane == 0) *reinterpret_cast<float4*>(stats2 + tok * 4) = make_float4(pi, lp, rp, rstd);
    }
}

// ------------------------------------------------------------------------------------------------
// phase 2 backward: persistent CTAs, thread = 8-column chunk(s), rows through a bulk-copy ring
// ------------------------------------------------------------------------------------------------
// stage rows: [dxn][o][partial]; the last only when present.  An accumulated partial gradient is
// added in the L2 (red), so its old value never travels to the SM.  The last warp is the producer
// (it refills a stage when every compute warp has released it); the compute warps meet once per
// token to combine three partial sums.
struct P2Smem {
    float4 scr[2][16];                         // [token parity][warp]: partial sums A, B, C
    uint64_t full[RB_STAGES], empty[RB_STAGES], meet;
    int abort_flag;
};

template <int CPT>
__global__ void __launch_bounds__(416, CPT == 1 ? 2 : 1)
route_p2_bwd_kernel(const bf16* __restrict__ dxn, const bf16* __restrict__ o, const bf16* __restrict__ part,
                    const float* __restrict__ w, const bf16* __restrict__ n_w, const float* __restrict__ stats2,
                    bf16* __restrict__ dout, float* __restrict__ dlse, bf16* __restrict__ dpart, int dpart_acc,
                    float* __restrict__ dw_part, float* __restrict__ dnw_part, int N, int D, int stages, int* status) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ P2Smem sm;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ncw = (blockDim.x >> 5) - 1;                        // compute warps; the last warp is the producer
    const int nct = ncw * 32;                                     // compute threads
    const bool has_p = part != nullptr;
    const bool acc = has_p && dpart_acc;
    const int rows = 2 + (has_p ? 1 : 0);
    const uint32_t row_bytes = (uint32_t)D * 2;
    const int nchunks = D >> 3;
    const float invD = 1.f / (float)D;
    if (threadIdx.x == 0) {
        for (int i = 0; i < stages; ++i) {
            tc::mbar_init(&sm.full[i], 1);
            tc::mbar_init(&sm.empty[i], ncw);
        }
        tc::mbar_init(&sm.meet, ncw);
        sm.abort_flag = 0;
        tc::fence_barrier_init();
    }
    __syncthreads();
    const int my_tokens = blockIdx.x < N ? (N - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (warp == ncw) {
        if (lane == 0) {
            for (int it = 0; it < my_tokens; ++it) {
                const int st = it % stages;
                if (!tc::mbar_wait(&sm.empty[st], ((it / stages) & 1) ^ 1, &sm.abort_flag)) {
                    atomicMax(status, (int)KB_TIMEOUT_TMA);
                    break;
                }
                const size_t tok = (size_t)blockIdx.x + (size_t)it * gridDim.x;
                uint8_t* base = smem + (size_t)st * rows * row_bytes;
                tc::mbar_expect_tx(&sm.full[st], rows * row_bytes);
                bulk_g2s(base, dxn + tok * D, row_bytes, &sm.full[st]);
                bulk_g2s(base + row_bytes, o + tok * D, row_bytes, &sm.full[st]);
                if (has_p) bulk_g2s(base + 2 * row_bytes, part + tok * D, row_bytes, &sm.full[st]);
            }
        }
    } else {
        float nw[CPT][8], wv[CPT][8], dw_acc[CPT][8], dnw_acc[CPT][8];
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            const int c = threadIdx.x + k * nct;
#pragma unroll
            for (int i = 0; i < 8; ++i) nw[k][i] = wv[k][i] = dw_acc[k][i] = dnw_acc[k][i] = 0.f;
            if (c < nchunks) {
                unpack8(ld8(n_w + c * 8), nw[k]);
                if (has_p) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) wv[k][i] = w[c * 8 + i];
                }
            }
        }
        for (int it = 0; it < my_tokens; ++it) {
            const int st = it % stages, par = it & 1;
            const size_t tok = (size_t)blockIdx.x + (size_t)it * gridDim.x;
            const float4 sv = *reinterpret_cast<const float4*>(stats2 + tok * 4);   // pi, l_p, r_p, rstd
            if (!tc::mbar_wait(&sm.full[st], (it / stages) & 1, &sm.abort_flag)) {
                if (lane == 0) atomicMax(status, (int)KB_TIMEOUT_TMA);
                break;
            }
            const bf16* base = reinterpret_cast<const bf16*>(smem + (size_t)st * rows * row_bytes);
            const float pi = sv.x, lp = sv.y, rp = sv.z, rstd = sv.w;
            float gw[CPT][8], hn[CPT][8], dif[CPT][8];                              // g * n_w, h * rstd, o - p
            float A = 0.f, Bv = 0.f, Cv = 0.f;
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const int c = threadIdx.x + k * nct;
#pragma unroll
                for (int i = 0; i < 8; ++i) gw[k][i] = hn[k][i] = dif[k][i] = 0.f;
                if (c < nchunks) {
                    float g[8], of[8], pf[8];
                    unpack8(ld8(base + c * 8), g);
                    unpack8(ld8(base + D + c * 8), of);
                    if (has_p) unpack8(ld8(base + 2 * D + c * 8), pf);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        dif[k][i] = has_p ? of[i] - pf[i] : 0.f;
                        hn[k][i] = (of[i] - pi * dif[k][i]) * rstd;
                        gw[k][i] = g[i] * nw[k][i];
                        dnw_acc[k][i] += g[i] * hn[k][i];
                        A += gw[k][i] * hn[k][i];
                        Bv += gw[k][i] * dif[k][i];
                        Cv += hn[k][i] * dif[k][i];
                    }
                }
            }
            A = warp_sum(A);
            Bv = warp_sum(Bv);
            Cv = warp_sum(Cv);
            if (lane == 0) sm.scr[par][warp] = make_float4(A, Bv, Cv, 0.f);
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&sm.meet);
            if (!tc::mbar_wait(&sm.meet, it & 1, &sm.abort_flag)) {
                if (lane == 0) atomicMax(status, (int)KB_TIMEOUT_EPI);
                break;
            }
            float3 red = make_float3(0.f, 0.f, 0.f);
            for (int i = 0; i < ncw; ++i) {
                const float4 v = sm.scr[par][i];
                red.x += v.x;
                red.y += v.y;
                red.z += v.z;
            }
            const float m = red.x * invD;
            const float cdot = rstd * (red.y - m * red.z);                          // sum dh (o - p)
            const float dl = pi * (1.f - pi) * cdot;                                // dlse; dl_p = -dl
            const float c_w = -dl * rp;
            const float c_p = -dl * lp * rp * rp * invD;
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const int c = threadIdx.x + k * nct;
                if (c >= nchunks) continue;
                float dh[8], dov[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    dh[i] = rstd * (gw[k][i] - hn[k][i] * m);
                    dov[i] = (1.f - pi) * dh[i];
                }
                st8(dout + tok * D + (size_t)c * 8, pack8(dov));
                if (has_p) {
                    // o - p = dif and h = hn / rstd give p back without another shared-memory read
                    float dp[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float pf = hn[k][i] / rstd - (1.f - pi) * dif[k][i];
                        dp[i] = pi * dh[i] + c_w * wv[k][i] - c_p * pf;
                        dw_acc[k][i] += c_w * pf;
                    }
                    if (acc) red_add8(dpart + tok * D + (size_t)c * 8, pack8(dp));
                    else st8(dpart + tok * D + (size_t)c * 8, pack8(dp));
                }
            }
            if (threadIdx.x == 0) dlse[tok] = has_p ? dl : 0.f;
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&sm.empty[st]);
        }
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            const int c = threadIdx.x + k * nct;
            if (c < nchunks) {
                float* a = dnw_part + (size_t)blockIdx.x * D + (size_t)c * 8;
                float* b = dw_part + (size_t)blockIdx.x * D + (size_t)c * 8;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    a[i] = dnw_acc[k][i];
                    if (has_p) b[i] = dw_acc[k][i];
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && sm.abort_flag) {    // copies still in flight must land before shared memory is released
        for (int i = 0; i < stages; ++i) {
            const uint64_t t0 = global_timer_ns();
            while (!tc::mbar_try_wait(&sm.full[i], 0) && !tc::mbar_try_wait(&sm.full[i], 1) &&
                   global_timer_ns() - t0 < 2000000ull) {}
        }
    }
}

// ------------------------------------------------------------------------------------------------
// phase 1: tensor-core dot products over the rows of a ring stage
// ------------------------------------------------------------------------------------------------
struct P1Srcs {
    const bf16* p[MAXS];
};
struct P1Dsts {
    bf16* p[MAXS];
    unsigned acc_mask;
};

// Two 8x8 bf16 matrices: lanes 0-7 give the row addresses of the first, lanes 8-15 of the second.
__device__ __forceinline__ void ldsm_x2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
// c[16x8] += a[16x16] b[16x8]; rows 8..15 of a are zero here, so a1 = a3 = 0 and c[2], c[3] stay unused.
__device__ __forceinline__ void mma_16816(float* c, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    const uint32_t z = 0;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}
// Address a lane passes to ldsm_x2 for the 8 rows starting at `rows` (row pitch in bytes) and the
// 16 columns starting at `col`: rows past `nrows` alias row 0 (their products are never read).
__device__ __forceinline__ uint32_t frag_addr(uint32_t rows, uint32_t pitch, int nrows, int col, int lane) {
    const int rr = lane & 7;
    return rows + (rr < nrows ? rr : 0) * pitch + (uint32_t)(col + ((lane >> 3) & 1) * 8) * 2;
}

// Shared-memory bytes of one ring row: 16 bytes of padding keep the 8 row addresses of an
// ldmatrix on different banks.
__host__ __device__ __forceinline__ uint32_t p1_pitch(int D) { return (uint32_t)D * 2 + 16; }

// Shared skeleton of the two phase-1 kernels.  The last warp of the CTA is the producer: it
// streams one token's rows per ring stage and recycles a stage when every compute warp has
// released it (mbarrier, no CTA-wide barrier).  The compute warps meet once per token, after
// writing their partial dot products; each of them then finishes the token's small softmax
// algebra redundantly in registers, so nothing else has to be synchronised.
struct P1Smem {
    float scr[2][16][80];                      // [token parity][warp]: 64 partial dots [q][s], 8 partial squared norms
    __align__(16) float tab[16][3][64];        // per warp: coefficient tables [s][q] for the per-element pass
    uint64_t full[RB_STAGES], empty[RB_STAGES], meet;
    int abort_flag;
};

// Meeting point of the compute warps for token `it` (bounded wait; false = give up).
__device__ __forceinline__ bool p1_meet(P1Smem& sm, int it, int lane) {
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&sm.meet);
    return tc::mbar_wait(&sm.meet, it & 1, &sm.abort_flag);
}

// Sum over the compute warps of the partials this lane owns: dots (q = g, s = 2t, 2t+1) and the
// squared norms of the same two sources.
__device__ __forceinline__ void p1_gather(const P1Smem& sm, int par, int ncw, int g, int t, float2& dots, float2& ss) {
    dots = make_float2(0.f, 0.f);
    ss = make_float2(0.f, 0.f);
    for (int w = 0; w < ncw; ++w) {
        const float2 d = *reinterpret_cast<const float2*>(&sm.scr[par][w][g * 8 + 2 * t]);
        const float2 q = *reinterpret_cast<const float2*>(&sm.scr[par][w][64 + 2 * t]);
        dots.x += d.x; dots.y += d.y;
        ss.x += q.x; ss.y += q.y;
    }
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

template <int THREADS>
__global__ void __launch_bounds__(THREADS, 1)
route_p1_fwd_kernel(P1Srcs srcs, int S, int Q, const float* __restrict__ wf, bf16* __restrict__ o,
                    float* __restrict__ lse, float* __restrict__ r_g, float* __restrict__ logit_g, int N, int D,
                    float eps, int stages, int* status) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ P1Smem sm;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ncw = (blockDim.x >> 5) - 1;                        // compute warps; the last warp is the producer
    const int g = lane >> 2, t = lane & 3;
    const uint32_t pitch = p1_pitch(D);
    const uint32_t row_bytes = (uint32_t)D * 2;
    const int nchunks = D >> 3, nks = D >> 4;
    const float invD = 1.f / (float)D;
    if (threadIdx.x == 0) {
        for (int i = 0; i < stages; ++i) {
            tc::mbar_init(&sm.full[i], 1);
            tc::mbar_init(&sm.empty[i], ncw);
        }
        tc::mbar_init(&sm.meet, ncw);
        sm.abort_flag = 0;
        tc::fence_barrier_init();
    }
    __syncthreads();
    const int my_tokens = blockIdx.x < N ? (N - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (warp == ncw) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            for (int it = 0; it < my_tokens; ++it) {
                const int st = it % stages;
                if (!tc::mbar_wait(&sm.empty[st], ((it / stages) & 1) ^ 1, &sm.abort_flag)) {
                    atomicMax(status, (int)KB_TIMEOUT_TMA);
                    break;
                }
                const size_t tok = (size_t)blockIdx.x + (size_t)it * gridDim.x;
                uint8_t* base = smem + (size_t)st * S * pitch;
                tc::mbar_expect_tx(&sm.full[st], S * row_bytes);
                for (int q = 0; q < S; ++q) bulk_g2s(base + (size_t)q * pitch, srcs.p[q] + tok * D, row_bytes, &sm.full[st]);
            }
        }
    } else {
        // ------------------------------------------------------------ compute
        // the queries' A fragments for this warp's column slice stay in registers for the whole kernel
        uint32_t wa0[KSW], wa2[KSW];
#pragma unroll
        for (int i = 0; i < KSW; ++i) {
            const int ks = warp * KSW + i;
            wa0[i] = wa2[i] = 0;
            if (ks < nks && g < Q) {
                const float* wr = wf + (size_t)g * D + ks * 16 + 2 * t;
                const __nv_bfloat162 lo = __floats2bfloat162_rn(wr[0], wr[1]), hi = __floats2bfloat162_rn(wr[8], wr[9]);
                wa0[i] = *reinterpret_cast<const uint32_t*>(&lo);
                wa2[i] = *reinterpret_cast<const uint32_t*>(&hi);
            }
        }
        const int c = threadIdx.x;                                  // this thread's 8-column chunk
        const bool active = c < nchunks;
        float* tab = &sm.tab[warp][0][0];                           // probabilities [s][q]
        for (int it = 0; it < my_tokens; ++it) {
            const int st = it % stages, par = it & 1;
            const size_t tok = (size_t)blockIdx.x + (size_t)it * gridDim.x;
            if (!tc::mbar_wait(&sm.full[st], (it / stages) & 1, &sm.abort_flag)) {
                if (lane == 0) atomicMax(status, (int)KB_TIMEOUT_TMA);
                break;
            }
            const uint8_t* stage = smem + (size_t)st * S * pitch;
            const uint32_t rows = smem_u32(stage);
            float cd[4] = {0.f, 0.f, 0.f, 0.f}, cg[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < KSW; ++i) {
                const int ks = warp * KSW + i;
                if (ks < nks) {
                    uint32_t v0, v1;
                    ldsm_x2(v0, v1, frag_addr(rows, pitch, S, ks * 16, lane));
                    mma_16816(cd, wa0[i], wa2[i], v0, v1);        // dots[q = g][s = 2t, 2t + 1]
                    mma_16816(cg, v0, v1, v0, v1);                // gram[s = g][s' = 2t, 2t + 1]
                }
            }
            *reinterpret_cast<float2*>(&sm.scr[par][warp][g * 8 + 2 * t]) = make_float2(cd[0], cd[1]);
            if ((g >> 1) == t) sm.scr[par][warp][64 + g] = (g & 1) ? cg[1] : cg[0];
            if (!p1_meet(sm, it, lane)) {
                if (lane == 0) atomicMax(status, (int)KB_TIMEOUT_EPI);
                break;
            }
            // every warp finishes the token's softmax itself: lane (g, t) owns query g, sources 2t and 2t+1
            float2 dots, ss;
            p1_gather(sm, par, ncw, g, t, dots, ss);
            const int s0 = 2 * t, s1 = 2 * t + 1;
            const float r0 = rsqrtf(ss.x * invD + eps), r1 = rsqrtf(ss.y * invD + eps);
            const float l0 = s0 < S ? dots.x * r0 : -INFINITY, l1 = s1 < S ? dots.y * r1 : -INFINITY;
            const float mx = quad_max(fmaxf(l0, l1));
            const float e0 = __expf(l0 - mx), e1 = __expf(l1 - mx);
            const float den = quad_sum(e0 + e1);
            const float inv = 1.f / den;
            tab[s0 * 8 + g] = e0 * inv;
            tab[s1 * 8 + g] = e1 * inv;
            if (warp == 0 && g < Q) {                                 // one warp records the statistics
                if (s0 < S) logit_g[((size_t)g * N + tok) * S + s0] = l0;
                if (s1 < S) logit_g[((size_t)g * N + tok) * S + s1] = l1;
                if (t == 0) lse[(size_t)g * N + tok] = mx + __logf(den);
                if (g == 0) {
                    if (s0 < S) r_g[tok * S + s0] = r0;
                    if (s1 < S) r_g[tok * S + s1] = r1;
                }
            }
            __syncwarp();
            if (active) {
                float2 acc[MAXQ][4];
#pragma unroll
                for (int q = 0; q < MAXQ; ++q)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[q][i] = make_float2(0.f, 0.f);
#pragma unroll
                for (int q = 0; q < MAXS; ++q) {                    // q runs over sources here
                    if (q < S) {
                        float v[8];
                        unpack8(ld8(reinterpret_cast<const bf16*>(stage + (size_t)q * pitch) + c * 8), v);
                        const float4 p0 = *reinterpret_cast<const float4*>(tab + q * 8);
                        const float4 p1 = *reinterpret_cast<const float4*>(tab + q * 8 + 4);
                        const float pq[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
                        for (int k = 0; k < MAXQ; ++k)
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                acc[k][i] = __ffma2_rn(make_float2(pq[k], pq[k]), make_float2(v[2 * i], v[2 * i + 1]), acc[k][i]);
                    }
                }
#pragma unroll
                for (int k = 0; k < MAXQ; ++k)
                    if (k < Q) {
                        bf16x8 ov;
#pragma unroll
                        for (int i = 0; i < 4; ++i) ov.v[i] = __floats2bfloat162_rn(acc[k][i].x, acc[k][i].y);
                        st8(o + ((size_t)k * N + tok) * D + (size_t)c * 8, ov);
                    }
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&sm.empty[st]);          // this warp is done with the stage
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && sm.abort_flag) {     // copies still in flight must land before shared memory is released
        for (int i = 0; i < stages; ++i) {
            const uint64_t t0 = global_timer_ns();
            while (!tc::mbar_try_wait(&sm.full[i], 0) && !tc::mbar_try_wait(&sm.full[i], 1) &&
                   global_timer_ns() - t0 < 2000000ull) {}
        }
    }
}

// phase 1 backward (reference: kernels/phase_1.py:204-274), all Q queries of the block at once:
//   P_qs = e^{l_qs - lse_q}, a_qs = do_q . u_s, dl_qs = P_qs (dlse_q + a_qs - sum_s P_qs a_qs)
//   du_s += sum_q [P_qs do_q + dl_qs r_s w_q] - (sum_q dl_qs l_qs) r_s^2 u_s / D
// and cw[s][tok][q] = dl_qs r_s, from which route_dw_kernel forms dw_q = sum_tok sum_s cw u_s.
// stage rows: S sources, then Q gradient rows.
template <int THREADS>
__global__ void __launch_bounds__(THREADS, 1)
route_p1_bwd_kernel(P1Srcs srcs, P1Dsts dsts, int S, int Q, const float* __restrict__ wf,
                    const bf16* __restrict__ dout, const float* __restrict__ dlse, const float* __restrict__ lse,
                    const float* __restrict__ r_g, const float* __restrict__ logit_g, float* __restrict__ cw_g,
                    int N, int D, int stages, int* status) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ P1Smem sm;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ncw = (blockDim.x >> 5) - 1;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t pitch = p1_pitch(D);
    const uint32_t row_bytes = (uint32_t)D * 2;
    const int nchunks = D >> 3, nks = D >> 4;
    const float invD = 1.f / (float)D;
    const int rows_per_stage = S + Q;
    if (threadIdx.x == 0) {
        for (int i = 0; i < stages; ++i) {
            tc::mbar_init(&sm.full[i], 1);
            tc::mbar_init(&sm.empty[i], ncw);
        }
        tc::mbar_init(&sm.meet, ncw);
        sm.abort_flag = 0;
        tc::fence_barrier_init();
    }
    __syncthreads();
    const int my_tokens = blockIdx.x < N ? (N - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (warp == ncw) {
        if (lane == 0) {
            for (int it = 0; it < my_tokens; ++it) {
                const int st = it % stages;
                if (!tc::mbar_wait(&sm.empty[st], ((it / stages) & 1) ^ 1, &sm.abort_flag)) {
                    atomicMax(status, (int)KB_TIMEOUT_TMA);
                    break;
                }
                const size_t tok = (size_t)blockIdx.x + (size_t)it * gridDim.x;
                uint8_t* base = smem + (size_t)st * rows_per_stage * pitch;
                tc::mbar_expect_tx(&sm.full[st], rows_per_stage * row_bytes);
                for (int q = 0; q < S; ++q) bulk_g2s(base + (size_t)q * pitch, srcs.p[q] + tok * D, row_bytes, &sm.full[st]);
                for (int q = 0; q < Q; ++q)
                    bulk_g2s(base + (size_t)(S + q) * pitch, dout + ((size_t)q * N + tok) * D, row_bytes, &sm.full[st]);
            }
        }
    } else {
        const int c = threadIdx.x;
        const bool active = c < nchunks;
        float* tP = &sm.tab[warp][0][0];                            // [q][s]: P_qs
        float* tW = &sm.tab[warp][1][0];                            // [q][s]: dl_qs r_s
        float* tV = &sm.tab[warp][2][0];                            // [s]: (sum_q dl_qs l_qs) r_s^2 / D
        const int s0 = 2 * t, s1 = 2 * t + 1;
        const bool qv = g < Q;
        for (int it = 0; it < my_tokens; ++it) {
            const int st = it % stages, par = it & 1;
            const size_t tok = (size_t)blockIdx.x + (size_t)it * gridDim.x;
            // statistics of this lane's (query, two sources): requested before the wait, used after the dots
            const float ls = qv ? lse[(size_t)g * N + tok] : 0.f, dls = qv ? dlse[(size_t)g * N + tok] : 0.f;
            const float lg0 = qv && s0 < S ? logit_g[((size_t)g * N + tok) * S + s0] : -INFINITY;
            const float lg1 = qv && s1 < S ? logit_g[((size_t)g * N + tok) * S + s1] : -INFINITY;
            const float rr0 = s0 < S ? r_g[tok * S + s0] : 0.f, rr1 = s1 < S ? r_g[tok * S + s1] : 0.f;
            if (!tc::mbar_wait(&sm.full[st], (it / stages) & 1, &sm.abort_flag)) {
                if (lane == 0) atomicMax(status, (int)KB_TIMEOUT_TMA);
                break;
            }
            const uint8_t* stage = smem + (size_t)st * rows_per_stage * pitch;
            const uint32_t rows = smem_u32(stage);
            float ca[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < KSW; ++i) {
                const int ks = warp * KSW + i;
                if (ks < nks) {
                    uint32_t a0, a2, v0, v1;
                    ldsm_x2(a0, a2, frag_addr(rows + S * pitch, pitch, Q, ks * 16, lane));
                    ldsm_x2(v0, v1, frag_addr(rows, pitch, S, ks * 16, lane));
                    mma_16816(ca, a0, a2, v0, v1);                // a[q = g][s = 2t, 2t + 1]
                }
            }
            *reinterpret_cast<float2*>(&sm.scr[par][warp][g * 8 + 2 * t]) = make_float2(ca[0], ca[1]);
            if (!p1_meet(sm, it, lane)) {
                if (lane == 0) atomicMax(status, (int)KB_TIMEOUT_EPI);
                break;
            }
            float2 a = make_float2(0.f, 0.f);
            for (int w = 0; w < ncw; ++w) {
                const float2 d = *reinterpret_cast<const float2*>(&sm.scr[par][w][g * 8 + 2 * t]);
                a.x += d.x; a.y += d.y;
            }
            const float p0 = __expf(lg0 - ls), p1 = __expf(lg1 - ls);           // 0 for unused (query, source) pairs
            const float abar = quad_sum(p0 * a.x + p1 * a.y);
            const float dl0 = p0 * (dls + a.x - abar), dl1 = p1 * (dls + a.y - abar);
            *reinterpret_cast<float2*>(&tP[g * 8 + s0]) = make_float2(p0, p1);
            *reinterpret_cast<float2*>(&tW[g * 8 + s0]) = make_float2(dl0 * rr0, dl1 * rr1);
            // sum over the queries (lanes with the same t) of dl * l, scaled per source
            float v0 = s0 < S && qv ? dl0 * lg0 : 0.f, v1 = s1 < S && qv ? dl1 * lg1 : 0.f;
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                v0 += __shfl_xor_sync(0xffffffffu, v0, off);
                v1 += __shfl_xor_sync(0xffffffffu, v1, off);
            }
            if (g == 0) *reinterpret_cast<float2*>(&tV[s0]) = make_float2(v0 * rr0 * rr0 * invD, v1 * rr1 * rr1 * invD);
            if (warp == 0 && qv) {                                    // coefficients of the query gradients
                if (s0 < S) cw_g[((size_t)s0 * N + tok) * MAXQ + g] = dl0 * rr0;
                if (s1 < S) cw_g[((size_t)s1 * N + tok) * MAXQ + g] = dl1 * rr1;
            }
            __syncwarp();
            if (active) {
                float2 du[MAXS][4];
#pragma unroll
                for (int q = 0; q < MAXS; ++q)
#pragma unroll
                    for (int i = 0; i < 4; ++i) du[q][i] = make_float2(0.f, 0.f);
#pragma unroll
                for (int q = 0; q < MAXQ; ++q) {
                    if (q < Q) {
                        float gq[8];
                        unpack8(ld8(reinterpret_cast<const bf16*>(stage + (size_t)(S + q) * pitch) + c * 8), gq);
                        const float4 x0 = *reinterpret_cast<const float4*>(wf + (size_t)q * D + c * 8);
                        const float4 x1 = *reinterpret_cast<const float4*>(wf + (size_t)q * D + c * 8 + 4);
                        const float2 w2[4] = {make_float2(x0.x, x0.y), make_float2(x0.z, x0.w), make_float2(x1.x, x1.y),
                                              make_float2(x1.z, x1.w)};
                        const float4 pa = *reinterpret_cast<const float4*>(tP + q * 8), pb = *reinterpret_cast<const float4*>(tP + q * 8 + 4);
                        const float4 wa = *reinterpret_cast<const float4*>(tW + q * 8), wb = *reinterpret_cast<const float4*>(tW + q * 8 + 4);
                        const float ps[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
                        const float ws[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                        for (int k = 0; k < MAXS; ++k) {
                            if (k < S) {
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    du[k][i] = __ffma2_rn(make_float2(ps[k], ps[k]), make_float2(gq[2 * i], gq[2 * i + 1]), du[k][i]);
                                    du[k][i] = __ffma2_rn(make_float2(ws[k], ws[k]), w2[i], du[k][i]);
                                }
                            }
                        }
                    }
                }
#pragma unroll
                for (int k = 0; k < MAXS; ++k) {
                    if (k >= S) continue;
                    float v[8];
                    unpack8(ld8(reinterpret_cast<const bf16*>(stage + (size_t)k * pitch) + c * 8), v);
                    const float cv = -tV[k];
                    bf16x8 ov;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 d = __ffma2_rn(make_float2(cv, cv), make_float2(v[2 * i], v[2 * i + 1]), du[k][i]);
                        ov.v[i] = __floats2bfloat162_rn(d.x, d.y);
                    }
                    bf16* dst = dsts.p[k] + tok * D + (size_t)c * 8;
                    if (dsts.acc_mask >> k & 1u) red_add8(dst, ov);
                    else st8(dst, ov);
                }
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&sm.empty[st]);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && sm.abort_flag) {
        for (int i = 0; i < stages; ++i) {
            const uint64_t t0 = global_timer_ns();
            while (!tc::mbar_try_wait(&sm.full[i], 0) && !tc::mbar_try_wait(&sm.full[i], 1) &&
                   global_timer_ns() - t0 < 2000000ull) {}
        }
    }
}

// dw_part[cta][q][D] = sum over this CTA's tokens and all sources of cw[s][tok][q] * u_s[tok][:]
// (the query gradients of phase 1; a column sum over the CTAs finishes them).  Pure streaming: a
// thread owns 8 columns and reads its 16 bytes of every source row.
__global__ void __launch_bounds__(512)
route_dw_kernel(P1Srcs srcs, int S, int Q, const float* __restrict__ cw_g, float* __restrict__ dw_part, int N, int D) {
    const int c = threadIdx.x;
    const int nchunks = D >> 3;
    if (c >= nchunks) return;
    float2 acc[MAXQ][4];
#pragma unroll
    for (int q = 0; q < MAXQ; ++q)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[q][i] = make_float2(0.f, 0.f);
    for (size_t tok = blockIdx.x; tok < (size_t)N; tok += gridDim.x) {
#pragma unroll 2
        for (int s = 0; s < S; ++s) {
            float v[8];
            unpack8(ld8(srcs.p[s] + tok * D + (size_t)c * 8), v);
            const float4 c0 = *reinterpret_cast<const float4*>(cw_g + ((size_t)s * N + tok) * MAXQ);
            const float4 c1 = *reinterpret_cast<const float4*>(cw_g + ((size_t)s * N + tok) * MAXQ + 4);
            const float cq[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
            for (int q = 0; q < MAXQ; ++q)
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    acc[q][i] = __ffma2_rn(make_float2(cq[q], cq[q]), make_float2(v[2 * i], v[2 * i + 1]), acc[q][i]);
        }
    }
    for (int q = 0; q < Q; ++q) {
        float* b = dw_part + ((size_t)blockIdx.x * Q + q) * D + (size_t)c * 8;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            b[2 * i] = acc[q][i].x;
            b[2 * i + 1] = acc[q][i].y;
        }
    }
}

template <typename K>
int rb_ensure_smem(K kernel, size_t bytes, bool* done_for_device) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 7;
    if (!done_for_device[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RB_DYN_SMEM) != cudaSuccess) return 7;
        done_for_device[dev] = true;
    }
    return bytes <= (size_t)RB_DYN_SMEM ? 0 : 8;
}

}  // namespace

// w[Q*D] fp32 = q * rn_w (bf16 inputs), the folded query of the routing kernels.
__global__ void route_fold_w_kernel(const bf16* __restrict__ q, const bf16* __restrict__ rn, float* __restrict__ w, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) w[i] = __bfloat162float(q[i]) * __bfloat162float(rn[i]);
}
KB_API int kb_route_fold_w(const void* q, const void* rn, float* w, int n, cudaStream_t st) {
    route_fold_w_kernel<<<(n + 255) / 256, 256, 0, st>>>((const bf16*)q, (const bf16*)rn, w, n);
    return cudaGetLastError() == cudaSuccess ? 0 : 8;
}

// 1 when the blocked kernels cover this shape (else the caller uses the per-call kernels).
KB_API int kb_route_blocked_ok(int S, int D) {
    return S >= 1 && S <= MAXS && D % 16 == 0 && D >= 16 && D <= 4096 &&
           (size_t)(S + MAXQ) * p1_pitch(D) <= (size_t)RB_DYN_SMEM;
}

// Number of CTAs (= rows of the partial weight-gradient buffers) of the two backward kernels.
KB_API int kb_route_blocked_grid(int N, int which) {
    const int g = rb_num_sms() * (which == 2 ? 2 : 4);
    return N < g ? N : g;
}

KB_API int kb_route_p1_fwd(const void* const* srcs, int S, int Q, const float* wf, void* o, float* lse, float* r,
                           float* logit, int N, int D, float eps, int* status, cudaStream_t st) {
    if (!kb_route_blocked_ok(S, D) || Q < 1 || Q > MAXQ || N < 1) return 5;
    P1Srcs ps;
    for (int s = 0; s < MAXS; ++s) ps.p[s] = s < S ? (const bf16*)srcs[s] : nullptr;
    const size_t stage = (size_t)S * p1_pitch(D);
    int stages = (int)(RB_DYN_SMEM / stage);
    if (stages > RB_STAGES) stages = RB_STAGES;
    if (stages < 1) return 8;
    const size_t smem = stage * stages;
    const int grid = N < rb_num_sms() ? N : rb_num_sms();
    const int threads = ((D / 8 + 31) / 32) * 32 + 32;           // compute warps + the producer warp
    if (threads <= 416) {
        static bool attr[64] = {};
        int r_ = rb_ensure_smem(route_p1_fwd_kernel<416>, smem, attr);
        if (r_) return r_;
        route_p1_fwd_kernel<416><<<grid, threads, smem, st>>>(ps, S, Q, wf, (bf16*)o, lse, r, logit, N, D, eps, stages, status);
    } else {
        static bool attr[64] = {};
        int r_ = rb_ensure_smem(route_p1_fwd_kernel<544>, smem, attr);
        if (r_) return r_;
        route_p1_fwd_kernel<544><<<grid, threads, smem, st>>>(ps, S, Q, wf, (bf16*)o, lse, r, logit, N, D, eps, stages, status);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : 8;
}

// cw[S][N][8] fp32 workspace: coefficients of the query gradients, consumed by kb_route_dw.
KB_API int kb_route_p1_bwd(const void* const* srcs, void* const* dsts, unsigned acc_mask, int S, int Q, const float* wf,
                           const void* dout, const float* dlse, const float* lse, const float* r, const float* logit,
                           float* cw, int N, int D, int* status, cudaStream_t st) {
    if (!kb_route_blocked_ok(S, D) || Q < 1 || Q > MAXQ || N < 1) return 5;
    P1Srcs ps;
    P1Dsts pd;
    for (int s = 0; s < MAXS; ++s) {
        ps.p[s] = s < S ? (const bf16*)srcs[s] : nullptr;
        pd.p[s] = s < S ? (bf16*)dsts[s] : nullptr;
    }
    pd.acc_mask = acc_mask;
    const size_t stage = (size_t)(S + Q) * p1_pitch(D);
    int stages = (int)(RB_DYN_SMEM / stage);
    if (stages > RB_STAGES) stages = RB_STAGES;
    if (stages < 1) return 8;
    const size_t smem = stage * stages;
    const int grid = N < rb_num_sms() ? N : rb_num_sms();
    const int threads = ((D / 8 + 31) / 32) * 32 + 32;
    if (threads <= 416) {
        static bool attr[64] = {};
        int r_ = rb_ensure_smem(route_p1_bwd_kernel<416>, smem, attr);
        if (r_) return r_;
        route_p1_bwd_kernel<416><<<grid, threads, smem, st>>>(ps, pd, S, Q, wf, (const bf16*)dout, dlse, lse, r, logit, cw,
                                                              N, D, stages, status);
    } else {
        static bool attr[64] = {};
        int r_ = rb_ensure_smem(route_p1_bwd_kernel<544>, smem, attr);
        if (r_) return r_;
        route_p1_bwd_kernel<544><<<grid, threads, smem, st>>>(ps, pd, S, Q, wf, (const bf16*)dout, dlse, lse, r, logit, cw,
                                                              N, D, stages, status);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : 8;
}

// dw_part[grid][Q][D] (grid = kb_route_blocked_grid(N, 1) rows) from cw and the sources.
KB_API int kb_route_dw(const void* const* srcs, int S, int Q, const float* cw, float* dw_part, int N, int D,
                       cudaStream_t st) {
    if (S < 1 || S > MAXS || Q < 1 || Q > MAXQ || D % 8 != 0 || D > 4096 || N < 1) return 5;
    P1Srcs ps;
    for (int s = 0; s < MAXS; ++s) ps.p[s] = s < S ? (const bf16*)srcs[s] : nullptr;
    const int threads = ((D / 8 + 31) / 32) * 32;
    route_dw_kernel<<<kb_route_blocked_grid(N, 1), threads, 0, st>>>(ps, S, Q, cw, dw_part, N, D);
    return cudaGetLastError() == cudaSuccess ? 0 : 8;
}

KB_API int kb_route_p2_fwd(const void* o, const float* lse, const void* part, const float* w, const void* n_w, void* xn,
                           float* stats2, int N, int D, float eps, cudaStream_t st) {
    if (D % 8 != 0 || D < 8 || D > 8192 || N < 1) return 5;
    const int nch = (D / 8 + 31) / 32;
    const int ctas = (N + 7) / 8;
    const int grid = ctas < rb_num_sms() * 8 ? ctas : rb_num_sms() * 8;
#define P2F(NCH_)                                                                                              \
    route_p2_fwd_kernel<NCH_><<<grid, 256, 0, st>>>((const bf16*)o, lse, (const bf16*)part, w, (const bf16*)n_w, \
                                                    (bf16*)xn, stats2, N, D, eps)
    if (nch <= 1) P2F(1);
    else if (nch <= 2) P2F(2);
    else if (nch <= 4) P2F(4);
    else if (nch <= 8) P2F(8);
    else if (nch <= 12) P2F(12);
    else if (nch <= 16) P2F(16);
    else P2F(32);
#undef P2F
    return cudaGetLastError() == cudaSuccess ? 0 : 8;
}

KB_API int kb_route_p2_bwd(const void* dxn, const void* o, const void* part, const float* w, const void* n_w,
                           const float* stats2, void* dout, float* dlse, void* dpart, int dpart_acc, float* dw_part,
                           float* dnw_part, int N, int D, int* status, cudaStream_t st) {
    if (D % 8 != 0 || D < 8 || D > 8192 || N < 1) return 5;
    const int nchunks = D / 8;
    const int cpt = (nchunks + 383) / 384;                                   // one chunk per thread up to D = 3072
    const int threads = ((nchunks + cpt - 1) / cpt + 31) / 32 * 32 + 32;     // compute warps + the producer warp
    const int rows = 2 + (part ? 1 : 0);
    const size_t stage = (size_t)rows * D * 2;
    const int ctas_per_sm = 2;
    int stages = (int)((200 * 1024 / ctas_per_sm) / stage);
    if (stages > RB_STAGES) stages = RB_STAGES;
    if (stages < 1) return 8;
    const size_t smem = stage * stages;
    const int grid = kb_route_blocked_grid(N, 2);
#define P2B(CPT_)                                                                                                  \
    {                                                                                                              \
        static bool attr[64] = {};                                                                                 \
        int r_ = rb_ensure_smem(route_p2_bwd_kernel<CPT_>, smem, attr);                                            \
        if (r_) return r_;                                                                                         \
        route_p2_bwd_kernel<CPT_><<<grid, threads, smem, st>>>((const bf16*)dxn, (const bf16*)o, (const bf16*)part, w, \
                                                                (const bf16*)n_w, stats2, (bf16*)dout, dlse,       \
                                                                (bf16*)dpart, dpart_acc, dw_part, dnw_part, N, D,  \
                                                                stages, status);                                   \
    }
    if (cpt == 1) P2B(1)
    else if (cpt == 2) P2B(2)
    else if (cpt == 3) P2B(3)
    else return 5;
#undef P2B
    return cudaGetLastError() == cudaSuccess ? 0 : 8;
}
