// Quantisers for the block-scaled fp8 path (e4m3, fp32 scales; scale = amax / 448 per tile, or the
// next power of two above it in `pow2` mode, which the hardware block-scaled GEMM requires).
//
//   kb_quant_rows     x [M,K] bf16 -> q [M,K],  s[K/128][M]      1x128 tiles along K (activations; the
//                                                                 scale array is stored K-block-major so
//                                                                 the GEMM epilogue reads it coalesced)
//   kb_quant_blocks   w [N,K] bf16 -> q [N,K],  s[K/128][N/128]  128x128 blocks (weights), and optionally
//                                   qt [K,N],  st[N/128][K/128]  the transposed copy for the data gradient
//   kb_quant_cols_t   x [M,N] bf16 -> qt [N,M], s[M/128][N]      128x1 tiles along M, written transposed:
//                                                                 both operands of the weight gradient
//                                                                 contract over tokens
// The reference relies on torchao's per-tensor dynamic scaling (src/training/train.py:301-312).
#include <cuda_fp8.h>

#include "common.cuh"

namespace {

constexpr float FP8_MAX = 448.f;

// Scale of a tile: amax / 448, or with `pow2` the next power of two at or above it (an exact
// 8-bit exponent, which the hardware block-scaled MMA takes as the scale factor; values then use
// at least half of the e4m3 range instead of all of it).
__device__ __forceinline__ float tile_scale(float amax, int pow2) {
    float s = fmaxf(amax, 1e-12f) / FP8_MAX;
    if (pow2) {
        uint32_t b = __float_as_uint(s);
        if (b & 0x007FFFFFu) b = (b & 0x7F800000u) + 0x00800000u;
        s = __uint_as_float(b);
    }
    return s;
}

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

__device__ __forceinline__ uint2 pack8_e4m3(const float* v, float inv) {
    return make_uint2(pack4_e4m3(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv),
                      pack4_e4m3(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv));
}

// Sixteen lanes per (row, K block): a lane holds 8 consecutive elements (one 16-byte load, one 8-byte
// store), so a warp covers two K blocks per step; U steps are in flight per thread.
template <int U>
__global__ void __launch_bounds__(256)
quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                  float* __restrict__ s, int M, int kblocks, int pow2) {
    const int sub = threadIdx.x & 15;
    const long long half_global = ((long long)blockIdx.x * 256 + threadIdx.x) >> 4;     // which 16-lane group
    const long long groups = (long long)gridDim.x * 16;
    const long long total = (long long)M * kblocks;
    for (long long w0 = half_global; (w0 & ~1LL) < total; w0 += groups * U) {      // both groups of a warp iterate together (shuffles)
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long w = w0 + (long long)u * groups;
            if (w < total) {
                const long long row = w / kblocks;
                const int kb = (int)(w - row * kblocks);
                raw[u] = *reinterpret_cast<const uint4*>(x + row * ldx + kb * 128 + sub * 8);
            } else {
                raw[u] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long w = w0 + (long long)u * groups;
            float v[8];
            unpack8(*reinterpret_cast<const bf16x8*>(&raw[u]), v);
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (w < total) {
                const long long row = w / kblocks;
                const int kb = (int)(w - row * kblocks);
                const float scale = tile_scale(amax, pow2), inv = 1.f / scale;
                *reinterpret_cast<uint2*>(q + row * ldq + kb * 128 + sub * 8) = pack8_e4m3(v, inv);
                if (sub == 0) s[(long long)kb * M + row] = scale;
            }
        }
    }
}

// one CTA (256 threads) per 128x128 block; thread t: row t/2, columns (t%2)*64 .. +64
__global__ void __launch_bounds__(256)
quant_blocks_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, uint8_t* __restrict__ q, float* __restrict__ s,
                    uint8_t* __restrict__ qt, float* __restrict__ st, int N, int K, int pow2) {
    __shared__ float red[8];
    __shared__ __align__(16) uint8_t tile[128][128 + 16];
    const int nb = blockIdx.y, kb = blockIdx.x;
    const int r = threadIdx.x >> 1, c0 = (threadIdx.x & 1) * 64;
    const int row = nb * 128 + r;
    float v[64];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float t[8];
        if (row < N) unpack8(ld8(w + row * ldw + kb * 128 + c0 + j * 8), t);
        else {
#pragma unroll
            for (int i = 0; i < 8; ++i) t[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[j * 8 + i] = t[i];
            amax = fmaxf(amax, fabsf(t[i]));
        }
    }
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
    const float scale = tile_scale(amax, pow2), inv = 1.f / scale;
    if (threadIdx.x == 0) {
        s[(long long)kb * gridDim.y + nb] = scale;
        if (st) st[(long long)nb * gridDim.x + kb] = scale;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint4 o;
        uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            op[i] = pack4_e4m3(v[j * 16 + i * 4] * inv, v[j * 16 + i * 4 + 1] * inv, v[j * 16 + i * 4 + 2] * inv,
                               v[j * 16 + i * 4 + 3] * inv);
        if (row < N) *reinterpret_cast<uint4*>(q + (long long)row * K + kb * 128 + c0 + j * 16) = o;
        if (qt) *reinterpret_cast<uint4*>(&tile[r][c0 + j * 16]) = o;
    }
    if (qt) {
        __syncthreads();
        // transposed write: output row = k (kb*128 + kk), 128 contiguous bytes along n
        const int kk = threadIdx.x >> 1, n0 = (threadIdx.x & 1) * 64;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint4 o;
            uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
            for (int i = 0; i < 16; ++i) ob[i] = tile[n0 + j * 16 + i][kk];
            if (nb * 128 + n0 + j * 16 < N)
                *reinterpret_cast<uint4*>(qt + (long long)(kb * 128 + kk) * N + nb * 128 + n0 + j * 16) = o;
        }
    }
}

// one CTA (256 threads) per 128 (rows of x, the M / token dim) x 128 (columns of x) tile.
__global__ void __launch_bounds__(256)
quant_cols_t_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ qt, float* __restrict__ s,
                    int M, int N, int pow2) {
    __shared__ __nv_bfloat16 tile[128][128 + 8];
    __shared__ float cmax[2][128];
    const int mb = blockIdx.x, nb = blockIdx.y;
    // load: thread t reads row t/2, 64 columns
    {
        const int r = threadIdx.x >> 1, c0 = (threadIdx.x & 1) * 64;
        const int row = mb * 128 + r;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int col = nb * 128 + c0 + j * 8;
            bf16x8 v;
            if (row < M && col < N) v = ld8(x + row * ldx + col);
            else {
#pragma unroll
                for (int i = 0; i < 4; ++i) v.v[i] = __floats2bfloat162_rn(0.f, 0.f);
            }
            *reinterpret_cast<uint4*>(&tile[r][c0 + j * 8]) = *reinterpret_cast<const uint4*>(&v);
        }
    }
    __syncthreads();
    // column amax: thread t handles column t%128, rows (t/128)*64 .. +64
    {
        const int c = threadIdx.x & 127, r0 = (threadIdx.x >> 7) * 64;
        float amax = 0.f;
#pragma unroll 8
        for (int r = 0; r < 64; ++r) amax = fmaxf(amax, fabsf(__bfloat162float(tile[r0 + r][c])));
        cmax[threadIdx.x >> 7][c] = amax;
    }
    __syncthreads();
    // write: thread t handles column (output row) t/2, token range (t%2)*64 .. +64
    {
        const int c = threadIdx.x >> 1, m0 = (threadIdx.x & 1) * 64;
        const int col = nb * 128 + c;
        const float scale = tile_scale(fmaxf(cmax[0][c], cmax[1][c]), pow2), inv = 1.f / scale;
        if (col < N) {
            if (m0 == 0) s[(long long)mb * N + col] = scale;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 o;
                uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = m0 + j * 16 + i * 4;
                    op[i] = pack4_e4m3(__bfloat162float(tile[m][c]) * inv, __bfloat162float(tile[m + 1][c]) * inv,
                                       __bfloat162float(tile[m + 2][c]) * inv, __bfloat162float(tile[m + 3][c]) * inv);
                }
                *reinterpret_cast<uint4*>(qt + (long long)col * M + mb * 128 + m0 + j * 16) = o;
            }
        }
    }
}

}  // namespace

KB_API int kb_quant_rows(const void* x, long long ldx, void* q, long long ldq, float* s, int M, int K, int pow2,
                         cudaStream_t st) {
    if (M <= 0 || K <= 0 || (K & 127) || (ldx & 7) || (ldq & 7) || ((uintptr_t)x & 15) || ((uintptr_t)q & 7)) return 5;
    const long long groups = (long long)M * (K / 128);
    long long blocks = (groups + 16 * 4 - 1) / (16 * 4);          // 16 groups per block, 4 steps each
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    quant_rows_kernel<4><<<(int)blocks, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, s, M, K / 128, pow2);
    return kb_launch_status();
}
KB_API int kb_quant_blocks(const void* w, long long ldw, void* q, float* s, void* qt, float* st_, int N, int K,
                           int pow2, cudaStream_t st) {
    if (N <= 0 || K <= 0 || (K & 127) || (N & 15) || (ldw & 7)) return 5;
    dim3 grid(K / 128, (N + 127) / 128);
    quant_blocks_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)w, ldw, (uint8_t*)q, s, (uint8_t*)qt, st_, N, K, pow2);
    return kb_launch_status();
}
KB_API int kb_quant_cols_t(const void* x, long long ldx, void* qt, float* s, int M, int N, int pow2, cudaStream_t st) {
    if (M <= 0 || N <= 0 || (M & 127) || (N & 7) || (ldx & 7)) return 5;
    dim3 grid(M / 128, (N + 127) / 128);
    quant_cols_t_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)qt, s, M, N, pow2);
    return kb_launch_status();
}
