// Causal GQA flash-attention forward for sm_100a (head_dim 128, bf16).
//
// One CTA per (128-row query tile, head, batch); two CTAs share an SM so that one CTA's
// softmax overlaps the other's tensor-core work.  Per key/value tile of 128 tokens:
//   S = Q K^T      tcgen05.mma, both operands K-major in shared memory (TMA, 128-byte swizzle),
//                  fp32 scores in tensor memory (128 lanes x 128 columns)
//   softmax        thread = query row: tcgen05.ld the row, online max / sum in base 2, write
//                  P as packed bf16 back into the score columns (tcgen05.st)
//   O += P V       tcgen05.mma with the A operand read from tensor memory and V as an MN-major
//                  shared-memory operand; O stays in tensor memory for the whole row of tiles
// The running maximum is refreshed lazily: O (in tensor memory) and the running sum are rescaled
// only when a row's maximum grows by more than 2^8, which is rare after the first tiles.
// Every wait is bounded (status word on timeout).
#include <cuda.h>

#include "tc.cuh"

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int TILE_BYTES = BQ * HD * 2;            // 32 KB, stored as two 64-column halves of 16 KB
constexpr int HALF_BYTES = BQ * 64 * 2;
constexpr int SMEM_BYTES = 3 * TILE_BYTES + 1024 + 128;
constexpr float RESCALE_THRESHOLD = 8.0f;          // in log2 units

struct FlashParams {
    int B, T, H, KV;
    float scale_log2;                              // softmax scale * log2(e)
    __nv_bfloat16* out;                            // [B, T, H, HD]
    float* lse;                                    // [B, H, T], natural log
    int q_col0, k_col0, v_col0;                    // first column of head 0 inside each operand's rows
    int* status;
};

__global__ void __launch_bounds__(160, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = smem + TILE_BYTES;
    uint8_t* sV = smem + 2 * TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * TILE_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;
    uint64_t* v_full = bars + 2;
    uint64_t* s_full = bars + 3;
    uint64_t* p_ready = bars + 4;
    uint64_t* o_done = bars + 5;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;       // heavy tiles first
    const int head = blockIdx.y, b = blockIdx.z;
    const int kvh = head / (p.H / p.KV);
    const int n_tiles = qt + 1;
    const int row0 = b * p.T + qt * BQ;                        // first token row of this query tile

    if (threadIdx.x == 0) {
        tc::mbar_init(q_full, 1);
        tc::mbar_init(k_full, 1);
        tc::mbar_init(v_full, 1);
        tc::mbar_init(s_full, 1);
        tc::mbar_init(p_ready, 4);
        tc::mbar_init(o_done, 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    if (warp == 4) {
        tc::tmem_alloc(tmem_slot, 256);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_s = *tmem_slot;            // scores / probabilities
    const uint32_t tmem_o = tmem_s + 128;          // output accumulator

    if (warp == 4) {
        // ------------------------------------------------------------ TMA + MMA issue (one thread)
        if (lane == 0) {
            tc::prefetch_tmap(&tmQ);
            tc::prefetch_tmap(&tmK);
            tc::prefetch_tmap(&tmV);
            const int qx = p.q_col0 + head * HD, kx = p.k_col0 + kvh * HD, vx = p.v_col0 + kvh * HD;
            tc::mbar_expect_tx(q_full, TILE_BYTES);
            tc::tma_load_3d(sQ, &tmQ, q_full, qx, row0, 0);
            tc::tma_load_3d(sQ + HALF_BYTES, &tmQ, q_full, qx + 64, row0, 0);
            auto load_k = [&](int j) {
                tc::mbar_expect_tx(k_full, TILE_BYTES);
                tc::tma_load_3d(sK, &tmK, k_full, kx, b * p.T + j * BKV, 0);
                tc::tma_load_3d(sK + HALF_BYTES, &tmK, k_full, kx + 64, b * p.T + j * BKV, 0);
            };
            auto load_v = [&](int j) {
                tc::mbar_expect_tx(v_full, TILE_BYTES);
                tc::tma_load_3d(sV, &tmV, v_full, vx, b * p.T + j * BKV, 0);
                tc::tma_load_3d(sV + HALF_BYTES, &tmV, v_full, vx + 64, b * p.T + j * BKV, 0);
            };
            load_k(0);
            load_v(0);
            const uint32_t idesc_s = tc::instr_desc_f16(BQ, BKV, 1, 1, 0, 0);
            const uint32_t idesc_o = tc::instr_desc_f16(BQ, HD, 1, 1, 0, 1);
            const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
            bool ok = tc::mbar_wait(q_full, 0, abort_flag);
            if (!ok) atomicMax(p.status, (int)KB_TIMEOUT_TMA);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const uint32_t ph = j & 1;
                if (!tc::mbar_wait(k_full, ph, abort_flag)) { atomicMax(p.status, (int)KB_TIMEOUT_TMA); break; }
                tc::tc_fence_after();
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
                    tc::mma_f16(tmem_s, tc::smem_desc_sw128(q_addr + off, 16, 1024),
                                tc::smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, k != 0);
                }
                tc::tc_commit(s_full);
                // K may be overwritten once the score MMAs have read it
                if (!tc::mbar_wait(s_full, ph, abort_flag)) { atomicMax(p.status, (int)KB_TIMEOUT_MMA); break; }
                if (j + 1 < n_tiles) load_k(j + 1);
                if (!tc::mbar_wait(p_ready, ph, abort_flag)) { atomicMax(p.status, (int)KB_TIMEOUT_MMA); break; }
                if (!tc::mbar_wait(v_full, ph, abort_flag)) { atomicMax(p.status, (int)KB_TIMEOUT_TMA); break; }
                tc::tc_fence_after();
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k) {
                    // A: 16 bf16 = 8 packed columns per step; B: V as [kv rows][hd], MN-major, 16 rows per step
                    tc::mma_f16_ts(tmem_o, tmem_s + k * 8, tc::smem_desc_sw128(v_addr + k * 2048, HALF_BYTES, 1024),
                                   idesc_o, (j | k) != 0);
                }
                tc::tc_commit(o_done);
                if (j + 1 < n_tiles) {
                    if (!tc::mbar_wait(o_done, ph, abort_flag)) { atomicMax(p.status, (int)KB_TIMEOUT_MMA); break; }
                    load_v(j + 1);
                }
            }
        }
    } else {
        // ------------------------------------------------------------ softmax: thread = query row
        const int r = warp * 32 + lane;                            // row inside the tile
        const uint32_t lane_base = ((uint32_t)(warp * 32) << 16);
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const uint32_t ph = j & 1;
            if (!tc::mbar_wait(s_full, ph, abort_flag)) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                ok = false;
                break;
            }
            tc::tc_fence_after();
            float s[BKV];
#pragma unroll
            for (int c = 0; c < BKV; c += 32) tc::tmem_ld32(tmem_s + lane_base + c, reinterpret_cast<uint32_t*>(s + c));
            tc::tmem_ld_wait();
            float mx = -INFINITY;
            if (j == qt) {                                          // diagonal tile: causal mask
#pragma unroll
                for (int c = 0; c < BKV; ++c) {
                    s[c] = c <= r ? s[c] * p.scale_log2 : -INFINITY;
                    mx = fmaxf(mx, s[c]);
                }
            } else {
#pragma unroll
                for (int c = 0; c < BKV; ++c) {
                    s[c] *= p.scale_log2;
                    mx = fmaxf(mx, s[c]);
                }
            }
            const bool grow = mx > m_used + RESCALE_THRESHOLD;      // first tile: m_used = -inf -> true
            if (__any_sync(0xffffffffu, grow) && j > 0) {
                // O holds sums of p * v with p relative to m_used: move it to the new maximum
                if (!tc::mbar_wait(o_done, (j - 1) & 1, abort_flag)) {
                    if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                    ok = false;
                    break;
                }
                tc::tc_fence_after();
                const float m_new = fmaxf(m_used, mx);
                const float f = exp2f(m_used - m_new);
#pragma unroll 1
                for (int c = 0; c < HD; c += 32) {
                    uint32_t o[32];
                    tc::tmem_ld32(tmem_o + lane_base + c, o);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                    tc::tmem_st32(tmem_o + lane_base + c, o);
                }
                tc::tmem_st_wait();
                l *= f;
                m_used = m_new;
            } else if (j == 0) {
                m_used = mx;
            }
            float sum = 0.f;
#pragma unroll
            for (int half = 0; half < 2; ++half) {                  // 64 scores -> 32 packed columns at a time
                uint32_t pk[32];
#pragma unroll
                for (int c = 0; c < 64; c += 2) {
                    const float p0 = exp2f(s[half * 64 + c] - m_used), p1 = exp2f(s[half * 64 + c + 1] - m_used);
                    sum += p0 + p1;
                    const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    pk[c >> 1] = *reinterpret_cast<const uint32_t*>(&h);
                }
                tc::tmem_st32(tmem_s + lane_base + half * 32, pk);
            }
            l += sum;
            tc::tmem_st_wait();
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(p_ready);
        }
        if (ok && tc::mbar_wait(o_done, (n_tiles - 1) & 1, abort_flag)) {
            tc::tc_fence_after();
            const float inv = 1.f / l;
            // T need not be a multiple of the tile: rows past the end of this sequence (zero-filled by
            // TMA, or the first rows of the next sequence) are computed but never stored; for the valid
            // rows the causal mask already excludes every key at or beyond the end
            const bool valid = qt * BQ + r < p.T;
            __nv_bfloat16* dst = p.out + ((size_t)(row0 + r) * p.H + head) * HD;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
                uint32_t o[32];
                tc::tmem_ld32(tmem_o + lane_base + c, o);
                tc::tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        float f8[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) f8[e] = __uint_as_float(o[i + e]) * inv;
                        st8(dst + c + i, pack8(f8));
                    }
                }
            }
            if (valid) p.lse[((size_t)b * p.H + head) * p.T + qt * BQ + r] = (m_used + log2f(l)) * 0.6931471805599453f;
        } else if (ok && lane == 0) {
            atomicMax(p.status, (int)KB_TIMEOUT_EPI);
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_s, 256);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_attn() {
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

// rows x cols bf16 matrix with the given row stride; box = 64 columns x 128 rows
int make_rows_tmap(CUtensorMap* m, const void* base, long long rows, long long cols, long long row_stride) {
    EncodeTiledFn enc = get_encode_attn();
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

}  // namespace

// q/k/v: token-major matrices [B*T, *] whose rows hold the heads side by side (row strides in
// elements; *_col0 = column of head 0).  out [B,T,H,128] bf16, lse [B,H,T] fp32.
KB_API int kb_flash_fwd(const void* q, long long q_stride, int q_cols, int q_col0, const void* k, long long k_stride,
                        int k_cols, int k_col0, const void* v, long long v_stride, int v_cols, int v_col0, void* out,
                        float* lse, int B, int T, int H, int KV, int hd, float scale, int* status, cudaStream_t st) {
    if (hd != HD || T < 1 || H % KV != 0) return 5;
    if ((q_stride & 7) || (k_stride & 7) || (v_stride & 7) || (q_col0 & 63) || (k_col0 & 63) || (v_col0 & 63)) return 6;
    if (((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15)) return 6;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
            return 7;
        attr_set = true;
    }
    CUtensorMap tmQ, tmK, tmV;
    int r = make_rows_tmap(&tmQ, q, (long long)B * T, q_cols, q_stride);
    if (r) return r;
    r = make_rows_tmap(&tmK, k, (long long)B * T, k_cols, k_stride);
    if (r) return r;
    r = make_rows_tmap(&tmV, v, (long long)B * T, v_cols, v_stride);
    if (r) return r;
    FlashParams p;
    p.B = B; p.T = T; p.H = H; p.KV = KV;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out = (__nv_bfloat16*)out;
    p.lse = lse;
    p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
    p.status = status;
    dim3 grid((T + BQ - 1) / BQ, H, B);
    flash_fwd_kernel<<<grid, 160, SMEM_BYTES, st>>>(tmQ, tmK, tmV, p);
    return 0;
}
