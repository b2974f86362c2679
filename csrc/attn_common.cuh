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
// B rows -> accumulator columns.
template <int HD>
__device__ __forceinline__ void mma_nt_tiles(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, uint32_t idesc) {
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
        const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
        tc::mma_f16(d_tmem, tc::smem_desc_sw128(a_addr + off, 16, 1024), tc::smem_desc_sw128(b_addr + off, 16, 1024),
                    idesc, k != 0);
    }
}

// acc[128 x HD] (+)= A B with A = 128 x 128 bf16 in tensor memory and B a stored tile read as
// [K = 128 tokens, N = HD] (MN-major).  The packed A operand lives in two runs of 32 columns:
// contraction steps 0..3 at `a_tmem`, steps 4..7 at `a_tmem + a_hi`.
template <int HD>
__device__ __forceinline__ void mma_ts_tile(uint32_t d_tmem, uint32_t a_tmem, uint32_t a_hi, uint32_t b_addr,
                                            uint32_t idesc, bool accumulate) {
#pragma unroll
    for (int k = 0; k < BT / 16; ++k) {
        const uint32_t a = a_tmem + (k < 4 ? k * 8 : a_hi + (k - 4) * 8);
        tc::mma_f16_ts(d_tmem, a, tc::smem_desc_sw128(b_addr + k * 2048, HALF_BYTES, 1024), idesc,
                       accumulate || k != 0);
    }
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// 2^x for x <= 0 on the FMA pipe (Cody-Waite split, degree-3 minimax on [0,1)); relative error
// about 1e-4, below the bf16 rounding of the probabilities it feeds.  Used for a share of the
// elements so that the special-function unit is not the only exponent source.
__device__ __forceinline__ float exp2_poly(float x) {
    x = fmaxf(x, -126.f);
    const float fl = floorf(x);
    const float f = x - fl;
    float p = fmaf(f, 0.07802403f, 0.22606707f);
    p = fmaf(p, f, 0.69583399f);
    p = fmaf(p, f, 0.99992513f);
    return __int_as_float(__float_as_int(p) + ((int)fl << 23));
}

}  // namespace attn
