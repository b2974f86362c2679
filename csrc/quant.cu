// Quantisers for the block-scaled fp8 path (e4m3, scale = amax / 448 per tile, fp32 scales).
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

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

// one warp per (row, K block): lane l holds elements [4l, 4l+4)
__global__ void __launch_bounds__(256)
quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                  float* __restrict__ s, int M, int kblocks) {
    const int lane = threadIdx.x & 31;
    const long long warp_global = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long total = (long long)M * kblocks;
    for (long long w = warp_global; w < total; w += (long long)gridDim.x * 8) {
        const int row = (int)(w / kblocks), kb = (int)(w % kblocks);
        const uint2 raw = *reinterpret_cast<const uint2*>(x + row * ldx + kb * 128 + lane * 4);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
        amax = warp_max(amax);
        const float scale = fmaxf(amax, 1e-12f) / FP8_MAX, inv = 1.f / scale;
        *reinterpret_cast<uint32_t*>(q + row * ldq + kb * 128 + lane * 4) = pack4_e4m3(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
        if (lane == 0) s[(long long)kb * M + row] = scale;
    }
}

// one CTA (256 threads) per 128x128 block; thread t: row t/2, columns (t%2)*64 .. +64
__global__ void __launch_bounds__(256)
quant_blocks_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, uint8_t* __restrict__ q, float* __restrict__ s,
                    uint8_t* __restrict__ qt, float* __restrict__ st, int N, int K) {
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
    const float scale = fmaxf(amax, 1e-12f) / FP8_MAX, inv = 1.f / scale;
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
                    int M, int N) {
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
        const float scale = fmaxf(fmaxf(cmax[0][c], cmax[1][c]), 1e-12f) / FP8_MAX, inv = 1.f / scale;
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

KB_API int kb_quant_rows(const void* x, long long ldx, void* q, long long ldq, float* s, int M, int K,
                         cudaStream_t st) {
    if (M <= 0 || K <= 0 || (K & 127) || (ldx & 3) || (ldq & 3)) return 5;
    const long long warps = (long long)M * (K / 128);
    long long blocks = (warps + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    quant_rows_kernel<<<(int)blocks, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, s, M, K / 128);
    return kb_launch_status();
}
KB_API int kb_quant_blocks(const void* w, long long ldw, void* q, float* s, void* qt, float* st_, int N, int K,
                           cudaStream_t st) {
    if (N <= 0 || K <= 0 || (K & 127) || (N & 15) || (ldw & 7)) return 5;
    dim3 grid(K / 128, (N + 127) / 128);
    quant_blocks_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)w, ldw, (uint8_t*)q, s, (uint8_t*)qt, st_, N, K);
    return kb_launch_status();
}
KB_API int kb_quant_cols_t(const void* x, long long ldx, void* qt, float* s, int M, int N, cudaStream_t st) {
    if (M <= 0 || N <= 0 || (M & 127) || (N & 7) || (ldx & 7)) return 5;
    dim3 grid(M / 128, (N + 127) / 128);
    quant_cols_t_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)qt, s, M, N);
    return kb_launch_status();
}
