// Shared pieces of the flash-attention kernels (forward, dQ, dK/dV): tensor maps over token-major
// matrices, tile constants, the shared-memory operand descriptors of the four product shapes
// and the score arithmetic.
//
// Operands are token-major matrices [rows = tokens, heads side by side]; a tile is 128 tokens
// x head_dim, stored by TMA as head_dim/64 column halves of 128 rows x 128 bytes (128-byte
// swizzle).  The same stored tile serves as
//   * a K-major operand (rows = M or N, head_dim = K): products with the transpose of the tile
//   * an MN-major B operand (rows = K, head_dim = N): products that contract over tokens
#pragma once
#include <cuda.h>

#include "tc.cuh"

namespace attn {

constexpr int BT = 128;                            // tokens per tile, both for queries and keys
constexpr int HALF_BYTES = BT * 64 * 2;            // one 64-column half of a tile: 16 KB
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

template <int HD>
struct Tile {
    static constexpr int HALVES = HD / 64;
    static constexpr int BYTES = HALVES * HALF_BYTES;
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// rows x cols bf16 matrix with the given row stride (elements); box = 64 columns x 128 rows.
// Rows past the end read as zero.
inline int make_rows_tmap(CUtensorMap* m, const void* base, long long rows, long long cols, long long row_stride) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return 100;
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, 1};
    cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2, (cuuint64_t)rows * row_stride * 2};
    cuuint32_t box[3] = {64, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 200 + (int)r;
}

// Host-side check shared by the launchers: strides in elements, column offsets of head 0.
inline bool operand_ok(const void* p, long long stride, int col0) {
    return !((uintptr_t)p & 15) && !(stride & 7) && !(col0 & 7);
}

// One tile (128 tokens starting at `row`, head columns starting at `col`) -> shared memory.
template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int col, int row) {
#pragma unroll
    for (int h = 0; h < HD / 64; ++h) tc::tma_load_3d(dst + h * HALF_BYTES, m, bar, col + h * 64, row, 0);
}

// acc[128 x 128] (+)= A B^T with both tiles K-major over head_dim: A rows -> accumulator lanes,
// B rows -> accumulator columns.  One descriptor pair is built per call; each contraction step
// only adds a constant to the low words, so the issuing thread stays ahead of the tensor pipe.
template <int HD>
__device__ __forceinline__ void mma_nt_tiles(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, uint32_t idesc) {
    const tc::DescHalves a = tc::smem_desc_halves(a_addr, 16, 1024), b = tc::smem_desc_halves(b_addr, 16, 1024);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
        const uint32_t off = ((k >> 2) * HALF_BYTES + (k & 3) * 32) >> 4;
        tc::mma_f16_h(d_tmem, a.lo + off, a.hi, b.lo + off, b.hi, idesc, k != 0);
    }
}

// acc[128 x 128] = A B^T with A = 128 x HD bf16 held in tensor memory (8 columns per 16-wide
// contraction step) and B a stored tile, K-major over head_dim.  Reading only B from shared
// memory halves the shared-memory traffic of the product, which is what bounds the all-shared
// form of a 128 x 128 tile.
template <int HD>
__device__ __forceinline__ void mma_tn_tile(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr, uint32_t idesc) {
    const tc::DescHalves b = tc::smem_desc_halves(b_addr, 16, 1024);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
        const uint32_t off = ((k >> 2) * HALF_BYTES + (k & 3) * 32) >> 4;
        tc::mma_f16_ts_h(d_tmem, a_tmem + 8 * k, b.lo + off, b.hi, idesc, k != 0);
    }
}

// acc[128 x HD] (+)= A B with A = 128 x 128 bf16 in tensor memory and B a stored tile read as
// [K = 128 tokens, N = HD] (MN-major).  The packed A operand (8 columns per 16-wide contraction
// step) is either one run of 64 columns (QUARTERS false) or four runs of 16 columns, one at the
// start of each 32-column quarter of the fp32 tile it overwrites (QUARTERS true: every thread of
// a row writes its packed result inside the columns it read).
template <int HD, bool QUARTERS>
__device__ __forceinline__ void mma_ts_tile(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr, uint32_t idesc,
                                            bool accumulate) {
    const tc::DescHalves b = tc::smem_desc_halves(b_addr, HALF_BYTES, 1024);
    const uint32_t acc = accumulate ? 1u : 0u;
#pragma unroll
    for (int k = 0; k < BT / 16; ++k) {
        const uint32_t a = a_tmem + (QUARTERS ? 32 * (k >> 1) + 8 * (k & 1) : 8 * k);
        tc::mma_f16_ts_h(d_tmem, a, b.lo + k * (2048 >> 4), b.hi, idesc, k == 0 ? acc : 1u);
    }
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Two floats -> packed bf16 by keeping the upper halves (one byte-permute on the integer pipe).
// The fp32 -> bf16 conversion instruction shares the special-function pipe with the exponentials,
// which is the busiest pipe of these kernels.  Callers pre-multiply the values by TRUNC_BIAS
// (folded into a constant they apply anyway), which turns truncation into rounding to within a
// quarter of a bf16 step on average.
constexpr float TRUNC_BIAS = 1.001953125f;         // 1 + 2^-9
constexpr float TRUNC_BIAS_LOG2 = 0.0028150156f;   // log2(1 + 2^-9)
__device__ __forceinline__ uint32_t pack_bf16_trunc(float a, float b) {
    return __byte_perm(__float_as_uint(a), __float_as_uint(b), 0x7632);
}

// max of three (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x for a pair of x <= 0 on the FMA pipe with packed two-wide instructions: the integer part
// comes from a round-down add of 1.5 * 2^23 (its low mantissa bits then hold floor(x)), the
// fraction goes through a degree-3 minimax polynomial on [0, 1) (relative error 7.5e-5, below
// the bf16 rounding of the probabilities it feeds), and the exponent is added with integer
// arithmetic.  Used for a share of the elements so that the special-function unit is not the
// only source of exponentials.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
    const float M = 12582912.f;
    x.x = fmaxf(x.x, -126.f);
    x.y = fmaxf(x.y, -126.f);
    const float2 t = __fadd2_rd(x, make_float2(M, M));
    const float2 fl = __fadd2_rn(t, make_float2(-M, -M));
    const float2 f = __ffma2_rn(fl, make_float2(-1.f, -1.f), x);
    float2 p = __ffma2_rn(f, make_float2(0.07802403f, 0.07802403f), make_float2(0.22606707f, 0.22606707f));
    p = __ffma2_rn(p, f, make_float2(0.69583399f, 0.69583399f));
    p = __ffma2_rn(p, f, make_float2(0.99992513f, 0.99992513f));
    p.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
    p.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
    return p;
}

// 2^x for a pair: pair number `i` of a row decides between the special-function unit and the
// polynomial (EMU of every 4 pairs are emulated).
template <int EMU>
__device__ __forceinline__ float2 exp2_pair(float2 x, int i) {
    if ((i & 3) < EMU) return exp2_poly2(x);
    return make_float2(exp2f(x.x), exp2f(x.y));
}

}  // namespace attn
