// Serving kernels: paged KV cache append, split-KV paged decode attention (GQA), greedy argmax.
//
// Cache layout: k_pages / v_pages [num_pages, n_kv, PAGE, hd] bf16 with PAGE = 16 tokens: the 16 rows
// of one (page, kv head) are 4 KB (hd 128) of contiguous memory, which is what the decode kernel
// streams; keys are stored post QK-norm and post RoPE (as the reference caches them,
// src/model/llama.py:333-337).  A request's pages are listed in page_table[req][i].
#include <stdlib.h>

#include "tc.cuh"

typedef __nv_bfloat16 bf16;
constexpr int PAGE = 16;

// k, v: [N, n_kv*hd] rows with the given strides; slot[n] = page * PAGE + offset in page, or < 0 to skip.
// A slot at or past `num_slots` (pages * PAGE) is recorded as KB_BAD_INDEX and skipped.
__global__ void kv_append_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v, long long k_stride,
                                 long long v_stride, bf16* __restrict__ k_pages, bf16* __restrict__ v_pages,
                                 const long long* __restrict__ slot, int N, int row_elems, int hd, long long num_slots,
                                 int* __restrict__ status) {
    kb_dep_trigger();
    kb_dep_wait();
    const int chunks = row_elems >> 3;
    const int n_kv = row_elems / hd;
    const long long total = (long long)N * chunks;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(i / chunks), c = (int)(i % chunks);
        const long long s = slot[n];
        if (s < 0) continue;
        if (s >= num_slots) {
            if (c == 0 && status) atomicMax(status, (int)KB_BAD_INDEX);
            continue;
        }
        const int kvh = (c * 8) / hd, d = (c * 8) % hd;
        const size_t dst = (((size_t)(s / PAGE) * n_kv + kvh) * PAGE + (size_t)(s % PAGE)) * hd + d;
        st8(k_pages + dst, ld8(k + (size_t)n * k_stride + (size_t)c * 8));
        st8(v_pages + dst, ld8(v + (size_t)n * v_stride + (size_t)c * 8));
    }
}
KB_API int kb_kv_append(const void* k, const void* v, long long k_stride, long long v_stride, void* k_pages,
                        void* v_pages, const long long* slot, int N, int row_elems, int hd, long long num_slots,
                        int* status, cudaStream_t st) {
    if (row_elems % 8 || k_stride % 8 || v_stride % 8 || hd % 8 || row_elems % hd) return 5;
    long long blocks = ((long long)N * (row_elems / 8) + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 4096) blocks = 4096;
    return kb_launch_dep(kv_append_kernel, dim3((unsigned)blocks), dim3(256), 0, st, (const bf16*)k, (const bf16*)v, k_stride,
                         v_stride, (bf16*)k_pages, (bf16*)v_pages, slot, N, row_elems, hd, num_slots, status);
}

// One CTA per (request, kv head, split of SPLIT tokens).  G = query heads per kv head.
// Phase 1: scores (8 lanes per token, 16 elements each for hd=128; 4 lanes x 16 for hd=64).
// Phase 2: softmax statistics over the split.  Phase 3: thread d accumulates sum_t p[t] V[t][d].
template <int HD, int G>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const bf16* __restrict__ q, long long q_stride, const bf16* __restrict__ k_pages,
                    const bf16* __restrict__ v_pages, const int* __restrict__ page_table, int max_pages,
                    const int* __restrict__ ctx_lens, int n_kv, int split_tokens, float scale,
                    float* __restrict__ part_o, float* __restrict__ part_ml, int nsplit) {
    extern __shared__ float sm[];
    float* sc = sm;                       // [G][split_tokens]
    __shared__ float qs[G][HD];
    __shared__ float red[2][G][4];
    __shared__ int spage[2048 / PAGE];    // page numbers of this split (split_tokens <= 2048)
    // kv head is the fastest-varying block index: the CTAs that read the eight 256-byte head slices of
    // the same token rows are launched together
    const int kvh = blockIdx.x, req = blockIdx.y, sp = blockIdx.z;
    const int ctx = ctx_lens[req];
    const int t0 = sp * split_tokens;
    const int nt = min(split_tokens, ctx - t0);
    const int H = n_kv * G;
    const size_t pbase = ((size_t)(req * n_kv + kvh) * nsplit + sp);
    if (nt <= 0) {
        if (threadIdx.x < G) {
            part_ml[(pbase * G + threadIdx.x) * 2] = -INFINITY;
            part_ml[(pbase * G + threadIdx.x) * 2 + 1] = 0.f;
        }
        return;
    }
    for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i % HD;
        qs[g][d] = __bfloat162float(q[(size_t)req * q_stride + (size_t)(kvh * G + g) * HD + d]) * scale;
    }
    for (int i = threadIdx.x; i < (nt + PAGE - 1) / PAGE; i += blockDim.x)
        spage[i] = page_table[(size_t)req * max_pages + t0 / PAGE + i];
    __syncthreads();
    constexpr int LPT = HD / 16;          // lanes per token
    constexpr int TPW = 32 / LPT;         // tokens per warp iteration
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LPT, tw = lane / LPT;
    // K pass.  Bandwidth here is set by the loads in flight, so every thread issues the 32-byte loads
    // of KU tokens before it touches any of them, and page numbers come from shared memory (a
    // dependent global load per token would double the latency of every step).
    constexpr int KU = 4;
    constexpr int KSTEP = 4 * TPW;        // tokens covered by the CTA per unrolled slot
    for (int tb = warp * TPW + tw; tb < ((nt + KSTEP * KU - 1) / (KSTEP * KU)) * (KSTEP * KU); tb += KSTEP * KU) {
        bf16x8 kr[KU][2];
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            const int t = tb + u * KSTEP;
            if (t < nt) {
                const int tok = t0 + t;
                const bf16* kp = k_pages + (((size_t)spage[t / PAGE] * n_kv + kvh) * PAGE + tok % PAGE) * HD + sub * 16;
                kr[u][0] = ld8(kp);
                kr[u][1] = ld8(kp + 8);
            }
        }
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            const int t = tb + u * KSTEP;
            float acc[G];
#pragma unroll
            for (int g = 0; g < G; ++g) acc[g] = 0.f;
            if (t < nt) {
                float kf[16];
                unpack8(kr[u][0], kf);
                unpack8(kr[u][1], kf + 8);
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[g] += kf[i] * qs[g][sub * 16 + i];
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
#pragma unroll
                for (int o = LPT / 2; o > 0; o >>= 1) acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], o);
                if (sub == 0 && t < nt) sc[g * split_tokens + t] = acc[g];
            }
        }
    }
    __syncthreads();
    // softmax statistics per query head
    float mx[G], sum[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float m = -INFINITY;
        for (int t = threadIdx.x; t < nt; t += blockDim.x) m = fmaxf(m, sc[g * split_tokens + t]);
        m = warp_max(m);
        if (lane == 0) red[0][g][warp] = m;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
        mx[g] = fmaxf(fmaxf(red[0][g][0], red[0][g][1]), fmaxf(red[0][g][2], red[0][g][3]));
        float s = 0.f;
        for (int t = threadIdx.x; t < nt; t += blockDim.x) {
            const float p = __expf(sc[g * split_tokens + t] - mx[g]);
            sc[g * split_tokens + t] = p;
            s += p;
        }
        s = warp_sum(s);
        if (lane == 0) red[1][g][warp] = s;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) sum[g] = red[1][g][0] + red[1][g][1] + red[1][g][2] + red[1][g][3];
    // weighted sum of V: thread (c, tg) owns the 8-element chunk c of the head dimension for tokens
    // tg, tg + NTG, ...; 16-byte loads, then the NTG partial rows are summed through shared memory
    {
        constexpr int NCH = HD / 8;            // chunks per row: 16 (hd 128) or 8 (hd 64)
        constexpr int NTG = 128 / NCH;         // token groups: 8 or 16
        const int c = threadIdx.x % NCH, tg = threadIdx.x / NCH;
        float o[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int i = 0; i < 8; ++i) o[g][i] = 0.f;
        constexpr int VU = 8;
        for (int tb = tg; tb < nt; tb += NTG * VU) {
            bf16x8 vr[VU];
#pragma unroll
            for (int u = 0; u < VU; ++u) {
                const int t = tb + u * NTG;
                if (t < nt) {
                    const int tok = t0 + t;
                    vr[u] = ld8(v_pages + (((size_t)spage[t / PAGE] * n_kv + kvh) * PAGE + tok % PAGE) * HD + c * 8);
                }
            }
#pragma unroll
            for (int u = 0; u < VU; ++u) {
                const int t = tb + u * NTG;
                if (t < nt) {
                    float vf[8];
                    unpack8(vr[u], vf);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float pw = sc[g * split_tokens + t];
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[g][i] += pw * vf[i];
                    }
                }
            }
        }
        __syncthreads();                       // scores are dead from here: reuse their space? no: separate buffer
        __shared__ float vred[128 / NCH][G][HD];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int i = 0; i < 8; ++i) vred[tg][g][c * 8 + i] = o[g][i];
        __syncthreads();
        for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
            const int g = i / HD, d = i % HD;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < NTG; ++j) acc += vred[j][g][d];
            part_o[(pbase * G + g) * HD + d] = acc;
        }
    }
    if (threadIdx.x < G) {
        part_ml[(pbase * G + threadIdx.x) * 2] = mx[threadIdx.x];
        part_ml[(pbase * G + threadIdx.x) * 2 + 1] = sum[threadIdx.x];
    }
    (void)H;
}

// Streaming variant of the split kernel: one pass over the tokens with an online softmax, K and V
// of a step loaded together, no score buffer and no block-wide barrier inside the loop.
// Lane layout: 8 lanes per token (8 elements of each half of the head row), 4 tokens per warp and step; every lane
// keeps running (max, sum) and its 16-element slice of the output for the tokens of its lane
// group; groups and warps are merged at the end.  Scores are kept in log2 units.
template <int HD, int G, int U>
__global__ void __launch_bounds__(128, U >= 4 ? 2 : 3)
paged_decode_stream_kernel(const bf16* __restrict__ q, long long q_stride, const bf16* __restrict__ k_pages,
                           const bf16* __restrict__ v_pages, const int* __restrict__ page_table, int max_pages,
                           const int* __restrict__ ctx_lens, int n_kv, int split_tokens, float scale,
                           float* __restrict__ part_o, float* __restrict__ part_ml, int nsplit) {
    constexpr int LPT = HD / 16, TPW = 32 / LPT, STEP = 4 * TPW;
    __shared__ float qs[G][HD];
    __shared__ int spage[2048 / PAGE];
    __shared__ float wo[4][G][HD];
    __shared__ float wml[4][G][2];
    const int kvh = blockIdx.x, req = blockIdx.y, sp = blockIdx.z;
    const int ctx = ctx_lens[req];
    const int t0 = sp * split_tokens;
    const int nt = min(split_tokens, ctx - t0);
    const size_t pbase = ((size_t)(req * n_kv + kvh) * nsplit + sp);
    if (nt <= 0) {
        if (threadIdx.x < G) {
            part_ml[(pbase * G + threadIdx.x) * 2] = -INFINITY;
            part_ml[(pbase * G + threadIdx.x) * 2 + 1] = 0.f;
        }
        return;
    }
    const float qscale = scale * 1.4426950408889634f;
    for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i % HD;
        qs[g][d] = __bfloat162float(q[(size_t)req * q_stride + (size_t)(kvh * G + g) * HD + d]) * qscale;
    }
    for (int i = threadIdx.x; i < (nt + PAGE - 1) / PAGE; i += blockDim.x)
        spage[i] = page_table[(size_t)req * max_pages + t0 / PAGE + i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LPT, tw = lane / LPT;
    float qr[G][16], o[G][16], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            qr[g][i] = qs[g][(i < 8 ? 0 : HD / 2) + sub * 8 + (i & 7)];
            o[g][i] = 0.f;
        }
    }
    const int span = STEP * U;
    for (int tb = warp * TPW + tw; tb < ((nt + span - 1) / span) * span; tb += span) {
        bf16x8 kr[U][2], vr[U][2];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = tb + u * STEP;
            if (t < nt) {
                // lane `sub` owns elements [8 sub, 8 sub + 8) of each half of the row, so the eight lanes of
                // a token read 128 contiguous bytes per instruction (whole sectors)
                const size_t off = (((size_t)spage[t / PAGE] * n_kv + kvh) * PAGE + (t0 + t) % PAGE) * HD + sub * 8;
                kr[u][0] = ld8(k_pages + off);
                kr[u][1] = ld8(k_pages + off + HD / 2);
                vr[u][0] = ld8(v_pages + off);
                vr[u][1] = ld8(v_pages + off + HD / 2);
            }
        }
        float sc[U][G];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool valid = tb + u * STEP < nt;
            float kf[16];
            if (valid) {
                unpack8(kr[u][0], kf);
                unpack8(kr[u][1], kf + 8);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float a = 0.f;
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) a += kf[i] * qr[g][i];
                }
#pragma unroll
                for (int x = LPT / 2; x > 0; x >>= 1) a += __shfl_xor_sync(0xffffffffu, a, x);
                sc[u][g] = valid ? a : -INFINITY;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float mn = m[g];
#pragma unroll
            for (int u = 0; u < U; ++u) mn = fmaxf(mn, sc[u][g]);
            if (mn == -INFINITY) continue;          // no valid token for this lane group yet
            const float f = exp2f(m[g] - mn);
            m[g] = mn;
            l[g] *= f;
#pragma unroll
            for (int i = 0; i < 16; ++i) o[g][i] *= f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (tb + u * STEP < nt) {
                float vf[16];
                unpack8(vr[u][0], vf);
                unpack8(vr[u][1], vf + 8);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pw = exp2f(sc[u][g] - m[g]);
                    l[g] += pw;
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[g][i] += pw * vf[i];
                }
            }
        }
    }
    // merge the lane groups of the warp (lanes with equal `sub`)
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float mg = m[g];
#pragma unroll
        for (int x = LPT; x < 32; x <<= 1) mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, x));
        const float f = mg == -INFINITY ? 0.f : exp2f(m[g] - mg);
        float lg = l[g] * f;
#pragma unroll
        for (int x = LPT; x < 32; x <<= 1) lg += __shfl_xor_sync(0xffffffffu, lg, x);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float v = o[g][i] * f;
#pragma unroll
            for (int x = LPT; x < 32; x <<= 1) v += __shfl_xor_sync(0xffffffffu, v, x);
            if (tw == 0) wo[warp][g][(i < 8 ? 0 : HD / 2) + sub * 8 + (i & 7)] = v;
        }
        if (lane == 0) {
            wml[warp][g][0] = mg;
            wml[warp][g][1] = lg;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i % HD;
        float mx = fmaxf(fmaxf(wml[0][g][0], wml[1][g][0]), fmaxf(wml[2][g][0], wml[3][g][0]));
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w)
            if (wml[w][g][0] != -INFINITY) acc += wo[w][g][d] * exp2f(wml[w][g][0] - mx);
        part_o[(pbase * G + g) * HD + d] = acc;
    }
    if (threadIdx.x < G) {
        const int g = threadIdx.x;
        const float mx = fmaxf(fmaxf(wml[0][g][0], wml[1][g][0]), fmaxf(wml[2][g][0], wml[3][g][0]));
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w)
            if (wml[w][g][0] != -INFINITY) sum += wml[w][g][1] * exp2f(wml[w][g][0] - mx);
        part_ml[(pbase * G + g) * 2] = mx * 0.6931471805599453f;       // back to natural-log units for the merge
        part_ml[(pbase * G + g) * 2 + 1] = sum;
    }
}

// Merge the splits: out[req][head][d] = sum_s e^{m_s - M} o_s[d] / sum_s e^{m_s - M} l_s
template <int HD>
__global__ void paged_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                   bf16* __restrict__ out, long long out_stride, int n_kv, int G, int nsplit) {
    kb_dep_trigger();
    kb_dep_wait();
    const int req = blockIdx.x, head = blockIdx.y;
    const int kvh = head / G, g = head % G;
    const int d = threadIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) {
        const size_t pb = ((size_t)(req * n_kv + kvh) * nsplit + s);
        M = fmaxf(M, part_ml[(pb * G + g) * 2]);
    }
    float num = 0.f, den = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const size_t pb = ((size_t)(req * n_kv + kvh) * nsplit + s);
        const float m = part_ml[(pb * G + g) * 2], l = part_ml[(pb * G + g) * 2 + 1];
        if (l <= 0.f) continue;
        const float w = __expf(m - M);
        den += w * l;
        if (d < HD) num += w * part_o[(pb * G + g) * HD + d];
    }
    if (d < HD) out[(size_t)req * out_stride + (size_t)head * HD + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
}

// Bulk-copy variant of the streaming kernel (the default for head_dim 128): with the head-major page layout
// the 16 K rows (and the 16 V rows) of one page are one contiguous 4 KB block, so one thread streams
// pages into a shared-memory ring with cp.async.bulk + mbarrier transaction counts and all threads
// compute from shared memory.  Bytes in flight are set by the ring (64 KB per CTA), not by registers.
// A stage holds two pages (K0 K1 V0 V1); waits are bounded: on a timeout the split contributes
// nothing and kb_decode_status() reports it.
__device__ int g_decode_status = 0;

__device__ __forceinline__ void bulk_g2s_dec(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

template <int HD, int G>
__global__ void __launch_bounds__(128, 3)
paged_decode_bulk_kernel(const bf16* __restrict__ q, long long q_stride, const bf16* __restrict__ k_pages,
                         const bf16* __restrict__ v_pages, const int* __restrict__ page_table, int max_pages,
                         const int* __restrict__ ctx_lens, int n_kv, int split_tokens, float scale,
                         float* __restrict__ part_o, float* __restrict__ part_ml, int nsplit) {
    constexpr int LPT = HD / 16, TPW = 32 / LPT, NST = 4;
    constexpr int PG = PAGE * HD;                       // elements of one (page, head) block
    extern __shared__ __align__(128) uint8_t ring_raw[];
    bf16* ring = reinterpret_cast<bf16*>(ring_raw);     // [NST][4][PG]: K0 K1 V0 V1
    __shared__ float qs[G][HD];
    __shared__ int spage[2048 / PAGE];
    __shared__ float wo[4][G][HD];
    __shared__ float wml[4][G][2];
    __shared__ uint64_t full[NST];
    __shared__ int abort_flag;
    const int kvh = blockIdx.x, req = blockIdx.y, sp = blockIdx.z;
    const int ctx = ctx_lens[req];
    const int t0 = sp * split_tokens;
    const int nt = min(split_tokens, ctx - t0);
    const size_t pbase = ((size_t)(req * n_kv + kvh) * nsplit + sp);
    if (nt <= 0) {
        if (threadIdx.x < G) {
            part_ml[(pbase * G + threadIdx.x) * 2] = -INFINITY;
            part_ml[(pbase * G + threadIdx.x) * 2 + 1] = 0.f;
        }
        return;
    }
    const int npages = (nt + PAGE - 1) / PAGE, niter = (npages + 1) / 2;
    const float qscale = scale * 1.4426950408889634f;
    for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i % HD;
        qs[g][d] = __bfloat162float(q[(size_t)req * q_stride + (size_t)(kvh * G + g) * HD + d]) * qscale;
    }
    for (int i = threadIdx.x; i < npages; i += blockDim.x)
        spage[i] = page_table[(size_t)req * max_pages + t0 / PAGE + i];
    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) tc::mbar_init(&full[s], 1);
        abort_flag = 0;
        tc::fence_barrier_init();
    }
    __syncthreads();
    auto issue = [&](int it) {
        const int st = it % NST;
        const int np = min(2, npages - 2 * it);
        tc::mbar_expect_tx(&full[st], (uint32_t)(np * 2 * PG * 2));
        for (int j = 0; j < np; ++j) {
            const size_t src = ((size_t)spage[2 * it + j] * n_kv + kvh) * PG;
            bulk_g2s_dec(ring + ((size_t)st * 4 + j) * PG, k_pages + src, PG * 2, &full[st]);
            bulk_g2s_dec(ring + ((size_t)st * 4 + 2 + j) * PG, v_pages + src, PG * 2, &full[st]);
        }
    };
    if (threadIdx.x == 0)
        for (int it = 0; it < NST && it < niter; ++it) issue(it);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LPT, tw = lane / LPT;
    float qr[G][16], o[G][16], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            qr[g][i] = qs[g][(i < 8 ? 0 : HD / 2) + sub * 8 + (i & 7)];
            o[g][i] = 0.f;
        }
    }
    bool ok = true;
    for (int it = 0; it < niter; ++it) {
        const int st = it % NST;
        if (!tc::mbar_wait(&full[st], (uint32_t)(it / NST) & 1u, &abort_flag)) {
            ok = false;
            break;
        }
        const int tin = warp * TPW + tw;                 // token within a page (HD 128: 4 warps x 4 = 16)
        float sc[2][G];
        bf16x8 vr[2][2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const bool valid = tin < PAGE && (2 * it + u) * PAGE + tin < nt;
            float kf[16];
            if (valid) {
                const bf16* kp = ring + ((size_t)st * 4 + u) * PG + (size_t)tin * HD + sub * 8;
                unpack8(ld8(kp), kf);
                unpack8(ld8(kp + HD / 2), kf + 8);
                const bf16* vp = ring + ((size_t)st * 4 + 2 + u) * PG + (size_t)tin * HD + sub * 8;
                vr[u][0] = ld8(vp);
                vr[u][1] = ld8(vp + HD / 2);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float a = 0.f;
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) a += kf[i] * qr[g][i];
                }
#pragma unroll
                for (int x = LPT / 2; x > 0; x >>= 1) a += __shfl_xor_sync(0xffffffffu, a, x);
                sc[u][g] = valid ? a : -INFINITY;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float mn = fmaxf(m[g], fmaxf(sc[0][g], sc[1][g]));
            if (mn == -INFINITY) continue;
            const float f = exp2f(m[g] - mn);
            m[g] = mn;
            l[g] *= f;
#pragma unroll
            for (int i = 0; i < 16; ++i) o[g][i] *= f;
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (tin < PAGE && (2 * it + u) * PAGE + tin < nt) {
                float vf[16];
                unpack8(vr[u][0], vf);
                unpack8(vr[u][1], vf + 8);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pw = exp2f(sc[u][g] - m[g]);
                    l[g] += pw;
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[g][i] += pw * vf[i];
                }
            }
        }
        __syncthreads();                                 // every thread is done with this stage
        if (threadIdx.x == 0 && it + NST < niter) issue(it + NST);
    }
    if (!ok) {
        // a copy did not arrive in time: report, contribute nothing, and let copies in flight land
        if (threadIdx.x == 0) {
            atomicMax(&g_decode_status, (int)KB_TIMEOUT_TMA);
            const uint64_t t_0 = global_timer_ns();
            while (global_timer_ns() - t_0 < 2000000ull) {}
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < G; ++g) { m[g] = -INFINITY; l[g] = 0.f; }
    }
    // merge the lane groups of the warp, then the warps (same as the streaming kernel)
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float mg = m[g];
#pragma unroll
        for (int x = LPT; x < 32; x <<= 1) mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, x));
        const float f = (mg == -INFINITY || m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mg);
        float lg = l[g] * f;
#pragma unroll
        for (int x = LPT; x < 32; x <<= 1) lg += __shfl_xor_sync(0xffffffffu, lg, x);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float v = o[g][i] * f;
#pragma unroll
            for (int x = LPT; x < 32; x <<= 1) v += __shfl_xor_sync(0xffffffffu, v, x);
            if (tw == 0) wo[warp][g][(i < 8 ? 0 : HD / 2) + sub * 8 + (i & 7)] = v;
        }
        if (lane == 0) {
            wml[warp][g][0] = mg;
            wml[warp][g][1] = lg;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i % HD;
        const float mx = fmaxf(fmaxf(wml[0][g][0], wml[1][g][0]), fmaxf(wml[2][g][0], wml[3][g][0]));
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w)
            if (wml[w][g][0] != -INFINITY) acc += wo[w][g][d] * exp2f(wml[w][g][0] - mx);
        part_o[(pbase * G + g) * HD + d] = acc;
    }
    if (threadIdx.x < G) {
        const int g = threadIdx.x;
        const float mx = fmaxf(fmaxf(wml[0][g][0], wml[1][g][0]), fmaxf(wml[2][g][0], wml[3][g][0]));
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w)
            if (wml[w][g][0] != -INFINITY) sum += wml[w][g][1] * exp2f(wml[w][g][0] - mx);
        part_ml[(pbase * G + g) * 2] = mx == -INFINITY ? -INFINITY : mx * 0.6931471805599453f;
        part_ml[(pbase * G + g) * 2 + 1] = sum;
    }
}
// Tensor-core variant (head_dim 128): the G query heads of a KV head are the first G rows of a
// 16-row `mma.sync.m16n8k16` A operand, so one page (16 tokens) costs 16 MMAs for Q K^T and 16 for
// P V instead of ~400 scalar FMAs and bf16 unpacks per lane - the scalar kernels are bound by
// instruction issue at 0.46 of the copy bandwidth, not by memory.  Every warp owns its own ring of
// pages (page w, w + 4, ... of the split): its 32 lanes each issue one 256-byte cp.async.bulk per
// K / V row into rows of 272 bytes (the 16-byte pad makes the ldmatrix reads conflict-free), so
// there is no block-wide barrier in the loop.  Waits are bounded as in the bulk kernel.
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// d += a * b, m16n8k16, bf16 inputs; rows 8..15 of A are zero here (a1 = a3 = 0)
__device__ __forceinline__ void mma_16816(float* d, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    const uint32_t z = 0;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// A staged (page, head) block of K or V is two 128-byte-swizzled half tiles [16 rows][64 elements]
// (2 KB each), written by one TMA tensor copy each: four copies per page instead of 32 row copies -
// the per-copy cost of the copy engine was what bounded the first version of this kernel.
constexpr int MMA_HALF = PAGE * 128;                 // bytes of one half tile
constexpr int MMA_PAGE = 2 * MMA_HALF;               // one staged (page, head) block of K or V
constexpr int MMA_NST = 2;                           // pages in flight per warp
constexpr int MMA_SMEM = 4 * MMA_NST * 2 * MMA_PAGE + 1024;

__device__ __forceinline__ void tma_load_2d_dec(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// byte offset of 16-byte chunk `chunk` (0..15 over the 256-byte row) of row `row` inside a staged block
__device__ __forceinline__ uint32_t swz_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * MMA_HALF + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// Merge of the splits inside the decode kernel: the CTA that finishes last for a (request, kv head) pair -
// elected through a counter that it leaves at zero for the next call - combines the pair's partial results
// exactly as paged_merge_kernel does (thread d = head dimension d, HD = blockDim.x = 128).  Every CTA of the
// pair calls this, also the ones whose split is empty.
template <int G>
__device__ __forceinline__ void merge_by_last_cta(const float* part_o, const float* part_ml, bf16* __restrict__ out,
                                                  long long out_stride, unsigned* counters, int req, int kvh, int n_kv,
                                                  int nsplit) {
    constexpr int HD = 128;
    __shared__ int s_last;
    __threadfence();                                     // this thread's partial results, device-wide
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(&counters[req * n_kv + kvh], 1u);
        s_last = prev == (unsigned)nsplit - 1u;
        if (s_last) counters[req * n_kv + kvh] = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int d = threadIdx.x;
    const size_t pb0 = (size_t)(req * n_kv + kvh) * nsplit;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float M = -INFINITY;
        for (int sidx = 0; sidx < nsplit; ++sidx) M = fmaxf(M, __ldcg(part_ml + ((pb0 + sidx) * G + g) * 2));
        float num = 0.f, den = 0.f;
        for (int sidx = 0; sidx < nsplit; ++sidx) {
            const size_t pb = pb0 + sidx;
            const float m = __ldcg(part_ml + (pb * G + g) * 2), l = __ldcg(part_ml + (pb * G + g) * 2 + 1);
            if (l <= 0.f) continue;
            const float w = __expf(m - M);
            den += w * l;
            num += w * __ldcg(part_o + (pb * G + g) * HD + d);
        }
        out[(size_t)req * out_stride + (size_t)(kvh * G + g) * HD + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
    }
}

template <int G>
__global__ void __launch_bounds__(128, 3)
paged_decode_mma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const bf16* __restrict__ q, long long q_stride, const int* __restrict__ page_table, int max_pages,
                        const int* __restrict__ ctx_lens, int n_kv, int split_tokens, float scale,
                        float* part_o, float* part_ml, int nsplit, bf16* __restrict__ out, long long out_stride,
                        unsigned* merge_counters) {
    constexpr int HD = 128;
    extern __shared__ uint8_t ring_unaligned[];
    uint8_t* ring_raw = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ring_unaligned) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(16) bf16 qs[G][HD];
    __shared__ int spage[2048 / PAGE];
    __shared__ float wml[4][G][2];
    __shared__ uint64_t full[4][MMA_NST];
    __shared__ int abort_flag;
    const int kvh = blockIdx.x, req = blockIdx.y, sp = blockIdx.z;
    kb_dep_trigger();
    kb_dep_wait();                      // the rows appended to the pages and the queries come from the kernels before
    const int ctx = ctx_lens[req];
    const int t0 = sp * split_tokens;
    const int nt = min(split_tokens, ctx - t0);
    const size_t pbase = ((size_t)(req * n_kv + kvh) * nsplit + sp);
    if (nt <= 0) {
        if (threadIdx.x < G) {
            part_ml[(pbase * G + threadIdx.x) * 2] = -INFINITY;
            part_ml[(pbase * G + threadIdx.x) * 2 + 1] = 0.f;
        }
        if (merge_counters) merge_by_last_cta<G>(part_o, part_ml, out, out_stride, merge_counters, req, kvh, n_kv, nsplit);
        return;
    }
    const int npages = (nt + PAGE - 1) / PAGE;
    const float qscale = scale * 1.4426950408889634f;
    for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i % HD;
        qs[g][d] = __float2bfloat16(__bfloat162float(q[(size_t)req * q_stride + (size_t)(kvh * G + g) * HD + d]) * qscale);
    }
    for (int i = threadIdx.x; i < npages; i += blockDim.x)
        spage[i] = page_table[(size_t)req * max_pages + t0 / PAGE + i];
    if (threadIdx.x == 0) {
        for (int w = 0; w < 4; ++w)
            for (int s = 0; s < MMA_NST; ++s) tc::mbar_init(&full[w][s], 1);
        abort_flag = 0;
        tc::fence_barrier_init();
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t* ring = ring_raw + (size_t)warp * MMA_NST * 2 * MMA_PAGE;
    const int my_pages = warp < npages ? (npages - warp + 3) / 4 : 0;       // pages warp, warp + 4, ...
    auto issue = [&](int i) {                                               // i-th page of this warp
        if (lane == 0) {
            const int st = i % MMA_NST;
            uint8_t* dst = ring + (size_t)(st * 2) * MMA_PAGE;
            const int row0 = (spage[warp + 4 * i] * n_kv + kvh) * PAGE;     // row of the [pages * heads * 16, 128] view
            tc::mbar_expect_tx(&full[warp][st], 2 * MMA_PAGE);
            tma_load_2d_dec(dst, &tmK, &full[warp][st], 0, row0);
            tma_load_2d_dec(dst + MMA_HALF, &tmK, &full[warp][st], 64, row0);
            tma_load_2d_dec(dst + MMA_PAGE, &tmV, &full[warp][st], 0, row0);
            tma_load_2d_dec(dst + MMA_PAGE + MMA_HALF, &tmV, &full[warp][st], 64, row0);
        }
    };
    for (int i = 0; i < MMA_NST && i < my_pages; ++i) issue(i);

    // Q fragments: row g = lane / 4 of the A operand (zero for g >= G), k = 16 ks + 2 (lane % 4) [+ 8]
    const int g_row = lane >> 2, qd = lane & 3;
    uint32_t qa0[8], qa2[8];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        qa0[ks] = g_row < G ? *reinterpret_cast<const uint32_t*>(&qs[g_row < G ? g_row : 0][ks * 16 + 2 * qd]) : 0u;
        qa2[ks] = g_row < G ? *reinterpret_cast<const uint32_t*>(&qs[g_row < G ? g_row : 0][ks * 16 + 8 + 2 * qd]) : 0u;
    }
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    // ldmatrix lane addressing: K matrices are (tokens 0-7 | 8-15) x (k 0-7 | 8-15) of a 16-wide k step, V
    // matrices (tokens 0-7 | 8-15) x (head dims 0-7 | 8-15) of a 16-wide column step
    const int k_row = (lane & 7) + (lane >> 4) * 8, k_sub = (lane >> 3) & 1;
    const int v_row = (lane & 7) + ((lane >> 3) & 1) * 8, v_sub = lane >> 4;
    for (int i = 0; i < my_pages; ++i) {
        const int st = i % MMA_NST;
        if (!tc::mbar_wait(&full[warp][st], (uint32_t)(i / MMA_NST) & 1u, &abort_flag)) {
            ok = false;
            break;
        }
        const uint32_t kb = smem_u32(ring + (size_t)(st * 2) * MMA_PAGE), vb = kb + MMA_PAGE;
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t b00, b01, b10, b11;
            ldsm_x4(kb + swz_off(k_row, ks * 2 + k_sub), b00, b01, b10, b11);
            mma_16816(s0, qa0[ks], qa2[ks], b00, b01);
            mma_16816(s1, qa0[ks], qa2[ks], b10, b11);
        }
        // online softmax on row g_row: this lane holds tokens 2 qd, 2 qd + 1, 8 + 2 qd, 9 + 2 qd of the page
        const int tok0 = (warp + 4 * i) * PAGE + 2 * qd;
        const float v00 = tok0 < nt ? s0[0] : -INFINITY, v01 = tok0 + 1 < nt ? s0[1] : -INFINITY;
        const float v10 = tok0 + 8 < nt ? s1[0] : -INFINITY, v11 = tok0 + 9 < nt ? s1[1] : -INFINITY;
        float mx = fmaxf(fmaxf(v00, v01), fmaxf(v10, v11));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float mn = fmaxf(m, mx);                   // finite: the first token of a staged page is always valid
        const float f = exp2f(m - mn);
        m = mn;
        const float p00 = exp2f(v00 - mn), p01 = exp2f(v01 - mn), p10 = exp2f(v10 - mn), p11 = exp2f(v11 - mn);
        l = l * f + (p00 + p01) + (p10 + p11);
        const uint32_t pa0 = pack2_bf16(p00, p01), pa2 = pack2_bf16(p10, p11);
#pragma unroll
        for (int j = 0; j < 16; ++j) { o[j][0] *= f; o[j][1] *= f; }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_trans(vb + swz_off(v_row, j * 2 + v_sub), b0, b1, b2, b3);
            mma_16816(o[2 * j], pa0, pa2, b0, b1);
            mma_16816(o[2 * j + 1], pa0, pa2, b2, b3);
        }
        __syncwarp();                                    // every lane has read this stage
        if (i + MMA_NST < my_pages) {
            tc::fence_proxy_async();
            issue(i + MMA_NST);
        }
    }
    if (!ok) {
        // a copy did not arrive in time: report, contribute nothing, and let copies in flight land
        if (lane == 0) {
            atomicMax(&g_decode_status, (int)KB_TIMEOUT_TMA);
            const uint64_t t_0 = global_timer_ns();
            while (global_timer_ns() - t_0 < 2000000ull) {}
        }
        __syncwarp();
        m = -INFINITY;
        l = 0.f;
    }
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    // the warp's partial output goes to the start of its own (now idle) ring: [G][HD] floats
    __syncwarp();
    float* wo_w = reinterpret_cast<float*>(ring);
    if (g_row < G) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            wo_w[g_row * HD + 8 * j + 2 * qd] = m == -INFINITY ? 0.f : o[j][0];
            wo_w[g_row * HD + 8 * j + 2 * qd + 1] = m == -INFINITY ? 0.f : o[j][1];
        }
        if (qd == 0) {
            wml[warp][g_row][0] = m;
            wml[warp][g_row][1] = l;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i % HD;
        const float mxx = fmaxf(fmaxf(wml[0][g][0], wml[1][g][0]), fmaxf(wml[2][g][0], wml[3][g][0]));
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w)
            if (wml[w][g][0] != -INFINITY)
                acc += reinterpret_cast<const float*>(ring_raw + (size_t)w * MMA_NST * 2 * MMA_PAGE)[g * HD + d] *
                       exp2f(wml[w][g][0] - mxx);
        part_o[(pbase * G + g) * HD + d] = acc;
    }
    if (threadIdx.x < G) {
        const int g = threadIdx.x;
        const float mxx = fmaxf(fmaxf(wml[0][g][0], wml[1][g][0]), fmaxf(wml[2][g][0], wml[3][g][0]));
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w)
            if (wml[w][g][0] != -INFINITY) sum += wml[w][g][1] * exp2f(wml[w][g][0] - mxx);
        part_ml[(pbase * G + g) * 2] = mxx == -INFINITY ? -INFINITY : mxx * 0.6931471805599453f;
        part_ml[(pbase * G + g) * 2 + 1] = sum;
    }
    if (merge_counters) merge_by_last_cta<G>(part_o, part_ml, out, out_stride, merge_counters, req, kvh, n_kv, nsplit);
}

// Reads the decode status word and clears it, so that one timeout is reported once.
KB_API int kb_decode_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int));
    }
    return v;
}

typedef CUresult (*EncodeTiledFnDec)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// pages [num_pages][n_kv][16][128] bf16 seen as rows of 128 elements; a box is half a (page, head) block
static int make_page_tmap(CUtensorMap* m, const void* base, long long rows) {
    static EncodeTiledFnDec enc = nullptr;
    if (!enc) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return 100;
        enc = reinterpret_cast<EncodeTiledFnDec>(ptr);
    }
    cuuint64_t dims[2] = {128, (cuuint64_t)rows};
    cuuint64_t strides[1] = {256};
    cuuint32_t box[2] = {64, PAGE};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 200 + (int)r;
}

// Which decode attention kernel kb_paged_decode launches: -1 = read KB_DECODE_KERNEL on the first call,
// 0 phases, 1 stream, 2 bulk, 3 mma.  kb_set_decode_kernel lets one process compare them.
static int g_decode_kernel = -1;
KB_API void kb_set_decode_kernel(int which) { g_decode_kernel = which; }

// Workspace sizes (floats) for B requests: part_o = B*n_kv*nsplit*G*hd, part_ml = B*n_kv*nsplit*G*2.
// `num_pages`: pages in k_pages / v_pages (the tensor-core kernel addresses them through a tensor map).
static int paged_decode_impl(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                             const int* page_table, int max_pages, const int* ctx_lens, int B, int n_q, int n_kv, int hd,
                             int max_ctx, int split_tokens, float scale, float* part_o, float* part_ml, void* out,
                             long long out_stride, int num_pages, unsigned* merge_counters, cudaStream_t st) {
    const int G = n_q / n_kv;
    bool merged = false;                 // the decode kernel merged the splits itself
    if (n_q % n_kv || split_tokens % PAGE || split_tokens > 2048) return 5;
    const int nsplit = (max_ctx + split_tokens - 1) / split_tokens;
    dim3 grid(n_kv, B, nsplit);
    const size_t smem = (size_t)G * split_tokens * sizeof(float);
    // KB_DECODE_KERNEL: "mma" (default for head_dim 128: tensor-core tiles, per-warp page rings), "bulk"
    // (scalar FMA from a block-wide cp.async.bulk ring; the default for other head sizes), "stream" (online
    // softmax from registers) or "phases" (three-phase kernel with the scores in shared memory)
    int& streaming = g_decode_kernel;
    static int unroll = 2;
    if (streaming < 0) {
        const char* e = getenv("KB_DECODE_KERNEL");
        streaming = (e && e[0] == 'p') ? 0 : (e && e[0] == 's') ? 1 : (e && e[0] == 'b') ? 2 : 3;   // phases | stream | bulk | mma (default)
        // tokens per lane group and iteration: 2 (default: 168 registers, three CTAs per SM; measured
        // 0.136 ms against 0.155 ms for 4, which needs 237 registers and leaves two CTAs per SM)
        const char* u = getenv("KB_DECODE_UNROLL");
        if (u && atoi(u) == 4) unroll = 4;
    }
#define DEC(HD_, G_)                                                                                          \
    if (streaming == 3 && (HD_) == 128 && num_pages > 0) {                                                     \
        static bool mma_flags[64] = {};                                                                        \
        bool* attr = kb_device_flag(mma_flags);                                                                \
        if (!attr) return 7;                                                                                   \
        if (!*attr) {                                                                                          \
            if (cudaFuncSetAttribute(paged_decode_mma_kernel<G_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                     MMA_SMEM) != cudaSuccess) return 7;                                       \
            *attr = true;                                                                                      \
        }                                                                                                      \
        CUtensorMap tmK, tmV;                                                                                  \
        const long long page_rows = (long long)num_pages * n_kv * PAGE;                                        \
        int tr = make_page_tmap(&tmK, k_pages, page_rows);                                                     \
        if (!tr) tr = make_page_tmap(&tmV, v_pages, page_rows);                                                \
        if (tr) return tr;                                                                                     \
        const int lr = kb_launch_dep(paged_decode_mma_kernel<G_>, grid, dim3(128), MMA_SMEM, st,               \
            tmK, tmV, (const bf16*)q, q_stride, page_table, max_pages, ctx_lens,                               \
            n_kv, split_tokens, scale, part_o, part_ml, nsplit, (bf16*)out, out_stride, merge_counters);       \
        if (lr) return lr;                                                                                     \
        merged = merge_counters != nullptr;                                                                    \
    } else if (streaming >= 2 && (HD_) == 128 && (G_) <= 4) {                                                         \
        static bool attr_flags[64] = {};                                                                       \
        bool* attr = kb_device_flag(attr_flags);                                                               \
        if (!attr) return 7;                                                                                   \
        if (!*attr) {                                                                                          \
            if (cudaFuncSetAttribute(paged_decode_bulk_kernel<HD_, G_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                     4 * 4 * PAGE * (HD_) * 2) != cudaSuccess) return 7;                       \
            *attr = true;                                                                                      \
        }                                                                                                      \
        paged_decode_bulk_kernel<HD_, G_><<<grid, 128, 4 * 4 * PAGE * (HD_) * 2, st>>>(                        \
            (const bf16*)q, q_stride, (const bf16*)k_pages, (const bf16*)v_pages, page_table, max_pages, ctx_lens, \
            n_kv, split_tokens, scale, part_o, part_ml, nsplit);                                               \
    } else if (streaming && (G_) <= 4 && unroll == 4)                                                          \
        paged_decode_stream_kernel<HD_, G_, 4><<<grid, 128, 0, st>>>((const bf16*)q, q_stride, (const bf16*)k_pages, \
                                                              (const bf16*)v_pages, page_table, max_pages, ctx_lens, \
                                                              n_kv, split_tokens, scale, part_o, part_ml, nsplit); \
    else if (streaming && (G_) <= 4)                                                                           \
        paged_decode_stream_kernel<HD_, G_, 2><<<grid, 128, 0, st>>>((const bf16*)q, q_stride, (const bf16*)k_pages, \
                                                              (const bf16*)v_pages, page_table, max_pages, ctx_lens, \
                                                              n_kv, split_tokens, scale, part_o, part_ml, nsplit); \
    else                                                                                                       \
        paged_decode_kernel<HD_, G_><<<grid, 128, smem, st>>>((const bf16*)q, q_stride, (const bf16*)k_pages,  \
                                                              (const bf16*)v_pages, page_table, max_pages, ctx_lens, \
                                                              n_kv, split_tokens, scale, part_o, part_ml, nsplit)
    if (hd == 128) {
        switch (G) {
            case 1: DEC(128, 1); break;
            case 2: DEC(128, 2); break;
            case 3: DEC(128, 3); break;
            case 4: DEC(128, 4); break;
            case 8: DEC(128, 8); break;
            default: return 5;
        }
        if (kb_launch_status()) return KB_LAUNCH_FAILED;
        if (merged) return 0;
        return kb_launch_dep(paged_merge_kernel<128>, dim3(B, n_q), dim3(128), 0, st, (const float*)part_o, (const float*)part_ml,
                             (bf16*)out, out_stride, n_kv, G, nsplit);
    } else if (hd == 64) {
        switch (G) {
            case 1: DEC(64, 1); break;
            case 2: DEC(64, 2); break;
            case 3: DEC(64, 3); break;
            case 4: DEC(64, 4); break;
            case 8: DEC(64, 8); break;
            default: return 5;
        }
        if (kb_launch_status()) return KB_LAUNCH_FAILED;
        return kb_launch_dep(paged_merge_kernel<64>, dim3(B, n_q), dim3(64), 0, st, (const float*)part_o, (const float*)part_ml,
                             (bf16*)out, out_stride, n_kv, G, nsplit);
    } else {
        return 5;
    }
    return kb_launch_status();
}
KB_API int kb_paged_decode(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                           const int* page_table, int max_pages, const int* ctx_lens, int B, int n_q, int n_kv, int hd,
                           int max_ctx, int split_tokens, float scale, float* part_o, float* part_ml, void* out,
                           long long out_stride, int num_pages, cudaStream_t st) {
    return paged_decode_impl(q, q_stride, k_pages, v_pages, page_table, max_pages, ctx_lens, B, n_q, n_kv, hd, max_ctx,
                             split_tokens, scale, part_o, part_ml, out, out_stride, num_pages, nullptr, st);
}
// The same in one launch where the tensor-core kernel runs (head_dim 128, `num_pages` > 0): the last CTA of a
// (request, kv head) pair merges the pair's splits.  `merge_counters`: B * n_kv zero-initialised words owned by
// the caller; the kernel leaves them at zero.  Calls that share the counters must not overlap in time.
KB_API int kb_paged_decode_merged(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                  const int* page_table, int max_pages, const int* ctx_lens, int B, int n_q, int n_kv,
                                  int hd, int max_ctx, int split_tokens, float scale, float* part_o, float* part_ml,
                                  void* out, long long out_stride, int num_pages, unsigned* merge_counters,
                                  cudaStream_t st) {
    return paged_decode_impl(q, q_stride, k_pages, v_pages, page_table, max_pages, ctx_lens, B, n_q, n_kv, hd, max_ctx,
                             split_tokens, scale, part_o, part_ml, out, out_stride, num_pages, merge_counters, st);
}

// Greedy sampling: out[row] = argmax_j logits[row][j] (first index on ties).
__global__ void argmax_kernel(const bf16* __restrict__ logits, long long stride, int V, long long* __restrict__ out) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const bf16* lg = logits + (size_t)blockIdx.x * stride;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
        const float v = __bfloat162float(lg[j]);
        if (v > best || (v == best && j < idx)) { best = v; idx = j; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = lane < (blockDim.x >> 5) ? bv[lane] : -INFINITY;
        idx = lane < (blockDim.x >> 5) ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx;
    }
}
KB_API int kb_argmax(const void* logits, long long stride, int rows, int V, long long* out, cudaStream_t st) {
    argmax_kernel<<<rows, 512, 0, st>>>((const bf16*)logits, stride, V, out);
    return kb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of kb_paged_decode (declared and documented in no_alloc.h): the
// split-KV partial results live in a fixed device array owned by this file.
#include <stdio.h>

#include <mutex>

#include "no_alloc.h"

static __device__ __align__(256) float g_noalloc_scratch[KB_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device.  In host code the array's name is
// only a handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress.
float* noalloc_scratch_for_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
        float* p = nullptr;
        const cudaError_t rc = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
        if (rc != cudaSuccess || p == nullptr) {
            fprintf(stderr, "kb_paged_decode_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev,
                    cudaGetErrorString(rc));
            return nullptr;
        }
        g_noalloc_ptr[dev] = p;
    }
    return g_noalloc_ptr[dev];
}
}  // namespace

KB_API int kb_paged_decode_noalloc(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                   const int* page_table, int max_pages, const int* ctx_lens, int B, int n_q,
                                   int n_kv, int hd, int max_ctx, int split_tokens, float scale, void* out,
                                   long long out_stride, cudaStream_t stream) {
    if (B <= 0 || n_q <= 0 || n_kv <= 0 || hd <= 0 || max_ctx <= 0 || split_tokens <= 0) return 5;
    const long long nsplit = (max_ctx + split_tokens - 1) / split_tokens;
    const long long need_o = (long long)B * n_q * nsplit * hd;       // partial outputs
    const long long need_ml = (long long)B * n_q * nsplit * 2;       // running max and sum per split
    if (need_o + need_ml > (long long)KB_NOALLOC_SCRATCH_FLOATS) {
        fprintf(stderr,
                "kb_paged_decode_noalloc: request needs %lld floats of scratch (B=%d heads=%d splits=%lld hd=%d) "
                "but the built-in array holds %d; use kb_paged_decode with caller workspaces, a larger "
                "split_tokens, or a smaller batch\n",
                need_o + need_ml, B, n_q, nsplit, hd, KB_NOALLOC_SCRATCH_FLOATS);
        return KB_NOALLOC_TOO_LARGE;
    }
    float* scratch = noalloc_scratch_for_current_device();
    if (scratch == nullptr) return KB_NOALLOC_SETUP_FAILED;
    // part_ml starts on a 256-byte boundary after part_o
    const long long ml_off = (need_o + 63) / 64 * 64;
    if (ml_off + need_ml > (long long)KB_NOALLOC_SCRATCH_FLOATS) {
        fprintf(stderr, "kb_paged_decode_noalloc: request needs %lld floats of scratch but the built-in array holds %d\n",
                ml_off + need_ml, KB_NOALLOC_SCRATCH_FLOATS);
        return KB_NOALLOC_TOO_LARGE;
    }
    return kb_paged_decode(q, q_stride, k_pages, v_pages, page_table, max_pages, ctx_lens, B, n_q, n_kv, hd, max_ctx,
                           split_tokens, scale, scratch, scratch + ml_off, out, out_stride, /*num_pages=*/0, stream);
}
