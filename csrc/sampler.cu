// Batched token sampler on the device, in the reference's order (serve.py:266-304): repetition
// penalty -> temperature -> top-k -> top-p -> multinomial, greedy at temperature 0.  One CTA per
// request row; every request carries its own parameters, seed and draw counter, so a mixed batch
// (greedy next to nucleus sampling) is one launch and no logits leave the device.
//
//   repetition penalty   a bitmap of the request's prompt and generated tokens (one bit per
//                        vocabulary id) selects the logits to damp; the sampled token is added to it
//   top-k                exact k-th largest value by a 4-pass radix select over order-preserving keys
//                        (ties at the threshold are kept, as the reference's `lg < kth` does)
//   top-p                the same radix descent over probability mass: the smallest key whose
//                        higher-keyed mass does not exceed top_p stays, everything below goes
//   multinomial          u = hash(seed, counter) in [0, 1); inverse CDF over the kept items in
//                        vocabulary order (block-wide prefix sum)
// The row (L2-resident) is re-read by each pass instead of being held per thread.
#include "common.cuh"

typedef __nv_bfloat16 bf16;

namespace {

constexpr int SAMP_THREADS = 1024;

__device__ __forceinline__ uint32_t order_key(float x) {      // larger float <-> larger key
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// splitmix64 of (seed, counter) -> 24 random bits -> [0, 1)
__host__ __device__ __forceinline__ float uniform01(unsigned long long seed, unsigned int counter) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * ((unsigned long long)counter + 1ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

struct BlockScratch {
    float f[32];
    int i[32];
    union {
        unsigned int cnt[256];
        float mass[256];
    } hist;
    unsigned int sel_prefix;
    unsigned int sel_k;
    float sel_acc;
    int chosen;
};

__device__ __forceinline__ float block_max(float v, BlockScratch& s) {
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s.f[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = s.f[threadIdx.x & 31];
    return warp_max(r);
}
__device__ __forceinline__ float block_sumf(float v, BlockScratch& s) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s.f[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = s.f[threadIdx.x & 31];
    return warp_sum(r);
}

template <typename T>
__device__ __forceinline__ float load_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float load_logit<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }

template <typename T>
__global__ void __launch_bounds__(SAMP_THREADS)
sample_kernel(const T* __restrict__ logits, long long row_stride, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ rep_penalty,
              const long long* __restrict__ seeds, const int* __restrict__ counters, unsigned int* __restrict__ seen,
              int seen_words, const int* __restrict__ slots, long long* __restrict__ out) {
    __shared__ BlockScratch s;
    const int row = blockIdx.x, tid = threadIdx.x;
    const int ipt = (V + SAMP_THREADS - 1) / SAMP_THREADS;     // items per thread, contiguous: vocabulary order = thread order
    const int lo = min(tid * ipt, V), hi = min(lo + ipt, V);
    const float T_ = temperature[row], rp = rep_penalty[row], tp = top_p[row];
    const float invT = T_ > 0.f ? 1.f / T_ : 1.f;
    const int k = top_k[row];
    unsigned int* bits = seen ? seen + (size_t)slots[row] * seen_words : nullptr;
    const bool penal = rp != 1.f && bits != nullptr;
    const T* lg = logits + (size_t)row * row_stride;
    // The row (96 KB at most, L2-resident) is re-read by every pass; nothing per-item is kept in
    // registers.  v(i): logit after repetition penalty and temperature.
    auto val = [&](int idx) -> float {
        float v = load_logit<T>(lg, idx);
        if (penal && (bits[idx >> 5] >> (idx & 31) & 1u)) v = v > 0.f ? v / rp : v * rp;
        return v * invT;
    };

    float mx = -INFINITY;
    int amax = 0x7fffffff;
    for (int idx = lo; idx < hi; ++idx) {
        const float v = val(idx);
        if (v > mx) { mx = v; amax = idx; }
    }
    const float gmax = block_max(mx, s);
    if (T_ <= 0.f) {
        // greedy: lowest index among the maxima
        int cand = mx == gmax ? amax : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
        __syncthreads();
        if ((tid & 31) == 0) s.i[tid >> 5] = cand;
        __syncthreads();
        int r = s.i[tid & 31];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) r = min(r, __shfl_xor_sync(0xffffffffu, r, o));
        if (tid == 0) {
            out[row] = r;
            if (bits) atomicOr(&bits[r >> 5], 1u << (r & 31));
        }
        return;
    }

    // ---- top-k: radix select of the k-th largest key
    unsigned int thr_key = 0;                                    // keep key >= thr_key
    if (k > 0 && k < V) {
        if (tid == 0) { s.sel_prefix = 0; s.sel_k = (unsigned int)k; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int b = tid; b < 256; b += SAMP_THREADS) s.hist.cnt[b] = 0;
            __syncthreads();
            const unsigned int prefix = s.sel_prefix;
            for (int idx = lo; idx < hi; ++idx) {
                const unsigned int key = order_key(val(idx));
                if (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&s.hist.cnt[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned int need = s.sel_k, b = 255;
                for (;; --b) {
                    const unsigned int c = s.hist.cnt[b];
                    if (c >= need || b == 0) break;
                    need -= c;
                }
                s.sel_prefix = prefix | (b << shift);
                s.sel_k = need;
            }
            __syncthreads();
        }
        thr_key = s.sel_prefix;
    }

    // ---- softmax weights of the kept items: w(i) = e^{v - max} when key >= threshold, else 0
    unsigned int pkey = 0;                                       // top-p threshold key (0: keep all)
    auto weight = [&](int idx) -> float {
        const float v = val(idx);
        const unsigned int key = order_key(v);
        return (key >= thr_key && key >= pkey) ? __expf(v - gmax) : 0.f;
    };
    float loc = 0.f;
    for (int idx = lo; idx < hi; ++idx) loc += weight(idx);
    float Z = block_sumf(loc, s);

    // ---- top-p: radix descent over probability mass
    if (tp > 0.f && tp < 1.f) {
        const float limit = tp * Z;
        if (tid == 0) { s.sel_prefix = 0; s.sel_acc = 0.f; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int b = tid; b < 256; b += SAMP_THREADS) s.hist.mass[b] = 0.f;
            __syncthreads();
            const unsigned int prefix = s.sel_prefix;
            for (int idx = lo; idx < hi; ++idx) {
                const float v = val(idx);
                const unsigned int key = order_key(v);
                if (key >= thr_key && (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8))))
                    atomicAdd(&s.hist.mass[(key >> shift) & 255u], __expf(v - gmax));
            }
            __syncthreads();
            if (tid == 0) {
                float acc = s.sel_acc;
                unsigned int b = 255;
                for (;; --b) {
                    const float m = s.hist.mass[b];
                    if (acc + m > limit || b == 0) break;       // the crossing happens inside this bin
                    acc += m;
                }
                s.sel_prefix = prefix | (b << shift);
                s.sel_acc = acc;
            }
            __syncthreads();
        }
        pkey = s.sel_prefix;
        loc = 0.f;
        for (int idx = lo; idx < hi; ++idx) loc += weight(idx);
        Z = block_sumf(loc, s);
    }

    // ---- multinomial: inverse CDF in vocabulary order
    const float target = uniform01((unsigned long long)seeds[row], (unsigned int)counters[row]) * Z;
    const int lane = tid & 31, warp = tid >> 5;
    float incl = loc;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    __syncthreads();
    if (lane == 31) s.f[warp] = incl;
    if (tid == 0) s.chosen = -1;
    __syncthreads();
    float wbase = 0.f;
    for (int w = 0; w < warp; ++w) wbase += s.f[w];
    const float excl = wbase + incl - loc;
    int last_kept = -1;
    if (loc > 0.f) {
        float run = excl;
        int pick = -1;
        for (int idx = lo; idx < hi; ++idx) {
            const float w = weight(idx);
            if (w > 0.f) {
                last_kept = idx;
                if (pick < 0 && target >= excl && target < run + w) pick = idx;
                run += w;
            }
        }
        if (pick < 0 && target >= excl && target < excl + loc) pick = last_kept;   // rounding inside this thread's range
        if (pick >= 0) atomicMax(&s.chosen, pick);
    }
    __syncthreads();
    if (s.chosen < 0) {
        // rounding left the target at or past the total: the last kept item of the row takes it
        if (last_kept >= 0) atomicMax(&s.chosen, last_kept);
        __syncthreads();
    }
    if (tid == 0) {
        const int r = s.chosen < 0 ? 0 : s.chosen;
        out[row] = r;
        if (bits) atomicOr(&bits[r >> 5], 1u << (r & 31));
    }
}

}  // namespace

// logits[B, V] (dtype 0 = bf16, 1 = fp32; `row_stride` elements between rows); per-row parameter
// arrays on the device; `seen` = bitmaps [*, seen_words] of 32-bit words, row `slots[b]` belongs to
// request b (null: no repetition penalty and nothing recorded).  out[B] int64.
KB_API int kb_sample(const void* logits, int dtype, long long row_stride, int B, int V, const float* temperature,
                     const int* top_k, const float* top_p, const float* rep_penalty, const long long* seeds,
                     const int* counters, unsigned int* seen, int seen_words, const int* slots, long long* out,
                     cudaStream_t st) {
    if (B < 1 || V < 1 || (seen && (long long)seen_words * 32 < V)) return 5;
    if (dtype == 0)
        sample_kernel<bf16><<<B, SAMP_THREADS, 0, st>>>((const bf16*)logits, row_stride, V, temperature, top_k, top_p,
                                                        rep_penalty, seeds, counters, seen, seen_words, slots, out);
    else if (dtype == 1)
        sample_kernel<float><<<B, SAMP_THREADS, 0, st>>>((const float*)logits, row_stride, V, temperature, top_k, top_p,
                                                         rep_penalty, seeds, counters, seen, seen_words, slots, out);
    else
        return 5;
    return kb_launch_status();
}
