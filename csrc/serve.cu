// Serving kernels: paged KV cache append, split-KV paged decode attention (GQA), greedy argmax.
//
// Cache layout: k_pages / v_pages [num_pages, PAGE, n_kv, hd] bf16 with PAGE = 16 tokens;
// keys are stored post QK-norm and post RoPE (as the reference caches them,
// src/model/llama.py:333-337).  A request's pages are listed in page_table[req][i].
#include "common.cuh"

typedef __nv_bfloat16 bf16;
constexpr int PAGE = 16;

// k, v: [N, n_kv*hd] rows with the given strides; slot[n] = page * PAGE + offset in page, or < 0 to skip.
__global__ void kv_append_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v, long long k_stride,
                                 long long v_stride, bf16* __restrict__ k_pages, bf16* __restrict__ v_pages,
                                 const long long* __restrict__ slot, int N, int row_elems) {
    const int chunks = row_elems >> 3;
    const long long total = (long long)N * chunks;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(i / chunks), c = (int)(i % chunks);
        const long long s = slot[n];
        if (s < 0) continue;
        st8(k_pages + s * row_elems + (size_t)c * 8, ld8(k + (size_t)n * k_stride + (size_t)c * 8));
        st8(v_pages + s * row_elems + (size_t)c * 8, ld8(v + (size_t)n * v_stride + (size_t)c * 8));
    }
}
KB_API int kb_kv_append(const void* k, const void* v, long long k_stride, long long v_stride, void* k_pages,
                        void* v_pages, const long long* slot, int N, int row_elems, cudaStream_t st) {
    if (row_elems % 8 || k_stride % 8 || v_stride % 8) return 5;
    long long blocks = ((long long)N * (row_elems / 8) + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 4096) blocks = 4096;
    kv_append_kernel<<<(int)blocks, 256, 0, st>>>((const bf16*)k, (const bf16*)v, k_stride, v_stride, (bf16*)k_pages,
                                                  (bf16*)v_pages, slot, N, row_elems);
    return 0;
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
    const int req = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z;
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
    const int row = n_kv * HD;
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
                const bf16* kp = k_pages + ((size_t)spage[t / PAGE] * PAGE + tok % PAGE) * row + (size_t)kvh * HD + sub * 16;
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
                    vr[u] = ld8(v_pages + ((size_t)spage[t / PAGE] * PAGE + tok % PAGE) * row + (size_t)kvh * HD + c * 8);
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

// Merge the splits: out[req][head][d] = sum_s e^{m_s - M} o_s[d] / sum_s e^{m_s - M} l_s
template <int HD>
__global__ void paged_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                   bf16* __restrict__ out, long long out_stride, int n_kv, int G, int nsplit) {
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

// Workspace sizes (floats) for B requests: part_o = B*n_kv*nsplit*G*hd, part_ml = B*n_kv*nsplit*G*2.
KB_API int kb_paged_decode(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                           const int* page_table, int max_pages, const int* ctx_lens, int B, int n_q, int n_kv, int hd,
                           int max_ctx, int split_tokens, float scale, float* part_o, float* part_ml, void* out,
                           long long out_stride, cudaStream_t st) {
    const int G = n_q / n_kv;
    if (n_q % n_kv || split_tokens % PAGE || split_tokens > 2048) return 5;
    const int nsplit = (max_ctx + split_tokens - 1) / split_tokens;
    dim3 grid(B, n_kv, nsplit);
    const size_t smem = (size_t)G * split_tokens * sizeof(float);
#define DEC(HD_, G_)                                                                                          \
    paged_decode_kernel<HD_, G_><<<grid, 128, smem, st>>>((const bf16*)q, q_stride, (const bf16*)k_pages,      \
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
        paged_merge_kernel<128><<<dim3(B, n_q), 128, 0, st>>>(part_o, part_ml, (bf16*)out, out_stride, n_kv, G, nsplit);
    } else if (hd == 64) {
        switch (G) {
            case 1: DEC(64, 1); break;
            case 2: DEC(64, 2); break;
            case 3: DEC(64, 3); break;
            case 4: DEC(64, 4); break;
            case 8: DEC(64, 8); break;
            default: return 5;
        }
        paged_merge_kernel<64><<<dim3(B, n_q), 64, 0, st>>>(part_o, part_ml, (bf16*)out, out_stride, n_kv, G, nsplit);
    } else {
        return 5;
    }
    return 0;
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
    return 0;
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
                           split_tokens, scale, scratch, scratch + ml_off, out, out_stride, stream);
}
