// Persistent warp-specialised GEMM for sm_100a:  C[b] = alpha * A[b] x B[b]^T + beta * Cin[b].
//
//   TMA (128-byte swizzle) -> 4-stage shared-memory ring -> tcgen05.mma (128x256x16, fp32
//   accumulators in tensor memory, two accumulator buffers) -> tcgen05.ld epilogue that
//   overlaps the next tile's main loop.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2-5 = epilogue (one TMEM lane quarter each).
// Operands are 16-bit (bf16 or fp16).  Each may be K-major (row = M/N index, K contiguous)
// or MN-major (row = K index, M/N contiguous), so forward, data-gradient and weight-gradient
// products run without explicit transposes.  A batch dimension (same-shape matrices with a
// fixed stride) serves the batched Newton-Schulz of Muon.
// The epilogue computes alpha*acc + beta*Cin with Cin of the output type: residual adds,
// gradient accumulation and the Newton-Schulz polynomials are all fused here.
#include <cuda.h>

#include "tc.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_STAGE = BM * BK * 2, B_STAGE = BN * BK * 2;
constexpr int SMEM_BYTES = STAGES * (A_STAGE + B_STAGE) + 1024 /*align*/ + 256 /*barriers*/;
constexpr int GROUP_M = 8;

struct GemmParams {
    int M, N, K, batch;
    int a_mn, b_mn;            // operand majors
    int a_fmt, b_fmt;          // 0 fp16, 1 bf16
    int out_type;              // 0 fp16, 1 bf16, 2 fp32
    float alpha, beta;
    void* C;
    const void* Cin;           // may be null (beta ignored) or alias C
    long long ldc, c_batch_stride;
    long long ldcin, cin_batch_stride;
    int* status;
    int split_k;               // > 1: each tile's K range is cut into split_k parts, fp32 atomic accumulation
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& b, int& tm, int& tn) {
    const int per_batch = tiles_m * tiles_n;
    b = tile / per_batch;
    int t = tile % per_batch;
    const int group = GROUP_M * tiles_n;
    const int g = t / group;
    const int first_m = g * GROUP_M;
    const int gm = min(GROUP_M, tiles_m - first_m);
    t -= g * group;
    tm = first_m + t % gm;
    tn = t / gm;
}

template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* dst, const OutT* cin, const uint32_t* acc, float alpha, float beta,
                                            int ncols);

template <>
__device__ __forceinline__ void store_row32<float>(float* dst, const float* cin, const uint32_t* acc, float alpha,
                                                   float beta, int ncols) {
    // ncols < 0 encodes "32 columns, 16-byte aligned": vector path
    if (ncols < 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float4 v;
            v.x = alpha * __uint_as_float(acc[4 * j]);
            v.y = alpha * __uint_as_float(acc[4 * j + 1]);
            v.z = alpha * __uint_as_float(acc[4 * j + 2]);
            v.w = alpha * __uint_as_float(acc[4 * j + 3]);
            if (cin) {
                const float4 c = *reinterpret_cast<const float4*>(cin + 4 * j);
                v.x += beta * c.x; v.y += beta * c.y; v.z += beta * c.z; v.w += beta * c.w;
            }
            *reinterpret_cast<float4*>(dst + 4 * j) = v;
        }
    } else {
        for (int j = 0; j < ncols; ++j) {
            float v = alpha * __uint_as_float(acc[j]);
            if (cin) v += beta * cin[j];
            dst[j] = v;
        }
    }
}

template <typename T>
__device__ __forceinline__ float h2f(T x);
template <> __device__ __forceinline__ float h2f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float h2f<__half>(__half x) { return __half2float(x); }
template <typename T>
__device__ __forceinline__ T f2h(float x);
template <> __device__ __forceinline__ __nv_bfloat16 f2h<__nv_bfloat16>(float x) { return __float2bfloat16(x); }
template <> __device__ __forceinline__ __half f2h<__half>(float x) { return __float2half(x); }

template <typename T>
__device__ __forceinline__ void store_row32_16(T* dst, const T* cin, const uint32_t* acc, float alpha, float beta,
                                               int ncols, bool vec_ok) {
    if (ncols == 32 && vec_ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = alpha * __uint_as_float(acc[8 * j + i]);
            if (cin) {
                const uint4 raw = *reinterpret_cast<const uint4*>(cin + 8 * j);
                const T* c = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += beta * h2f<T>(c[i]);
            }
            uint4 o;
            T* op = reinterpret_cast<T*>(&o);
#pragma unroll
            for (int i = 0; i < 8; ++i) op[i] = f2h<T>(v[i]);
            *reinterpret_cast<uint4*>(dst + 8 * j) = o;
        }
    } else {
        for (int j = 0; j < ncols; ++j) {
            float v = alpha * __uint_as_float(acc[j]);
            if (cin) v += beta * h2f<T>(cin[j]);
            dst[j] = f2h<T>(v);
        }
    }
}

__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE + B_STAGE));
    uint64_t* full = bars;                 // [STAGES]  TMA -> MMA
    uint64_t* empty = bars + STAGES;       // [STAGES]  MMA -> TMA
    uint64_t* acc_full = bars + 2 * STAGES;      // [2] MMA -> epilogue
    uint64_t* acc_empty = bars + 2 * STAGES + 2; // [2] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n * p.batch * p.split_k;   // work items (tile, k-part)
    const int kblocks_total = (p.K + BK - 1) / BK;
    const int kb_per = (kblocks_total + p.split_k - 1) / p.split_k;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(&acc_full[b], 1);
            tc::mbar_init(&acc_empty[b], 4);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, 512);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tc::prefetch_tmap(&tmA);
            tc::prefetch_tmap(&tmB);
            int stage = 0;
            uint32_t phase = 0;
            int issued = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int b, tm, tn;
                tile_coords(tile / p.split_k, tiles_m, tiles_n, b, tm, tn);
                const int kb0 = (tile % p.split_k) * kb_per, kb1 = min(kblocks_total, kb0 + kb_per);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
                        atomicMax(p.status, (int)KB_TIMEOUT_TMA);
                        ok = false;
                        break;
                    }
                    tc::mbar_expect_tx(&full[stage], A_STAGE + B_STAGE);
                    uint8_t* a_dst = sA + stage * A_STAGE;
                    uint8_t* b_dst = sB + stage * B_STAGE;
                    if (p.a_mn) {
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c)
                            tc::tma_load_3d(a_dst + c * (64 * BK * 2), &tmA, &full[stage], tm * BM + c * 64, kb * BK, b);
                    } else {
                        tc::tma_load_3d(a_dst, &tmA, &full[stage], kb * BK, tm * BM, b);
                    }
                    if (p.b_mn) {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c)
                            tc::tma_load_3d(b_dst + c * (64 * BK * 2), &tmB, &full[stage], tn * BN + c * 64, kb * BK, b);
                    } else {
                        tc::tma_load_3d(b_dst, &tmB, &full[stage], kb * BK, tn * BN, b);
                    }
                    ++issued;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // let copies already in flight land before the block can exit
                const int inflight = issued < STAGES ? issued : STAGES;
                for (int i = 0; i < inflight; ++i) {
                    int s = stage - 1 - i;
                    uint32_t ph = phase;
                    if (s < 0) { s += STAGES; ph ^= 1; }
                    const uint64_t t0 = global_timer_ns();
                    while (!tc::mbar_try_wait(&full[s], ph) && global_timer_ns() - t0 < 2000000ull) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = tc::instr_desc_f16(BM, BN, p.a_fmt, p.b_fmt, p.a_mn, p.b_mn);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                const int buf = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!tc::mbar_wait(&acc_empty[buf], acc_phase ^ 1, abort_flag)) {
                    atomicMax(p.status, (int)KB_TIMEOUT_MMA);
                    ok = false;
                    break;
                }
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const int kb0 = (tile % p.split_k) * kb_per, kb1 = min(kblocks_total, kb0 + kb_per);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!tc::mbar_wait(&full[stage], phase, abort_flag)) {
                        atomicMax(p.status, (int)KB_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    tc::tc_fence_after();
                    const uint32_t a_addr = smem_u32(sA + stage * A_STAGE);
                    const uint32_t b_addr = smem_u32(sB + stage * B_STAGE);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = p.a_mn ? tc::smem_desc_sw128(a_addr + k * 2048, 64 * BK * 2, 1024)
                                                   : tc::smem_desc_sw128(a_addr + k * 32, 16, 1024);
                        const uint64_t bd = p.b_mn ? tc::smem_desc_sw128(b_addr + k * 2048, 64 * BK * 2, 1024)
                                                   : tc::smem_desc_sw128(b_addr + k * 32, 16, 1024);
                        tc::mma_f16(d_tmem, ad, bd, idesc, ((kb - kb0) | k) != 0);
                    }
                    tc::tc_commit(&empty[stage]);   // stage reusable once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc::tc_commit(&acc_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;   // TMEM lanes [32*quarter, 32*quarter+32)
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
            int b, tm, tn;
            tile_coords(tile / p.split_k, tiles_m, tiles_n, b, tm, tn);
            const bool has_k = (tile % p.split_k) * kb_per < kblocks_total;
            const int buf = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            if (!tc::mbar_wait(&acc_full[buf], acc_phase, abort_flag)) {
                if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                ok = false;
                break;
            }
            tc::tc_fence_after();
            const int row = tm * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t acc[32];
                tc::tmem_ld32(taddr + c0, acc);
                tc::tmem_ld_wait();
                const int col = tn * BN + c0;
                const int ncols = min(32, p.N - col);
                if (p.split_k > 1) {
                    if (row < p.M && ncols > 0 && has_k) {
                        float* dst = reinterpret_cast<float*>(p.C) + (long long)b * p.c_batch_stride +
                                     (long long)row * p.ldc + col;
                        for (int j = 0; j < ncols; ++j) atomicAdd(dst + j, p.alpha * __uint_as_float(acc[j]));
                    }
                } else if (row < p.M && ncols > 0) {
                    const long long off = (long long)b * p.c_batch_stride + (long long)row * p.ldc + col;
                    const long long offin = (long long)b * p.cin_batch_stride + (long long)row * p.ldcin + col;
                    if (p.out_type == 2) {
                        float* dst = reinterpret_cast<float*>(p.C) + off;
                        const float* cin = p.Cin ? reinterpret_cast<const float*>(p.Cin) + offin : nullptr;
                        const bool vec = ((p.ldc | p.ldcin | col) & 3) == 0 && ncols == 32;
                        store_row32<float>(dst, cin, acc, p.alpha, p.beta, vec ? -1 : ncols);
                    } else {
                        const bool vec = ((p.ldc | p.ldcin | col) & 7) == 0;
                        if (p.out_type == 1) {
                            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
                            const __nv_bfloat16* cin =
                                p.Cin ? reinterpret_cast<const __nv_bfloat16*>(p.Cin) + offin : nullptr;
                            store_row32_16<__nv_bfloat16>(dst, cin, acc, p.alpha, p.beta, ncols, vec);
                        } else {
                            __half* dst = reinterpret_cast<__half*>(p.C) + off;
                            const __half* cin = p.Cin ? reinterpret_cast<const __half*>(p.Cin) + offin : nullptr;
                            store_row32_16<__half>(dst, cin, acc, p.alpha, p.beta, ncols, vec);
                        }
                    }
                }
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, 512);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
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

// 16-bit matrix [rows, cols] (cols contiguous, leading dimension ld elements) x batch.
int make_tmap(CUtensorMap* m, const void* base, int fmt, long long cols, long long rows, long long ld,
              long long batch, long long batch_stride, int box_cols, int box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return 100;
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch > 1 ? batch_stride : rows * ld) * 2};
    cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(m, fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                           const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 200 + (int)r;
}

}  // namespace

// C[b][M,N] = alpha * op(A[b]) * op(B[b])^T + beta * Cin[b].
//   a_mn = 0: A is [M,K] (lda = row stride);  a_mn = 1: A is stored [K,M].
//   b_mn = 0: B is [N,K];                      b_mn = 1: B is stored [K,N].
//   fmt: 0 fp16, 1 bf16.  out_type: 0 fp16, 1 bf16, 2 fp32.  status: device int, set on a wait timeout.
// Requirements: 16-byte aligned bases, lda/ldb multiples of 8 elements.
KB_API int kb_gemm(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, int batch,
                   long long lda, long long ldb, long long ldc, long long ldcin, long long a_bs, long long b_bs,
                   long long c_bs, long long cin_bs, int a_mn, int b_mn, int a_fmt, int b_fmt, int out_type,
                   float alpha, float beta, int* status, int max_ctas, int split_k, cudaStream_t st) {
    if (split_k < 1) split_k = 1;
    if (split_k > 1 && out_type != 2) return 5;
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 5;
    if ((lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return 6;
    if (batch > 1 && ((a_bs & 7) || (b_bs & 7))) return 6;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
            cudaSuccess)
            return 7;
        attr_set = true;
    }
    CUtensorMap tmA, tmB;
    int r;
    if (a_mn) r = make_tmap(&tmA, A, a_fmt, M, K, lda, batch, a_bs, 64, BK);
    else r = make_tmap(&tmA, A, a_fmt, K, M, lda, batch, a_bs, BK, BM);
    if (r) return r;
    if (b_mn) r = make_tmap(&tmB, B, b_fmt, N, K, ldb, batch, b_bs, 64, BK);
    else r = make_tmap(&tmB, B, b_fmt, K, N, ldb, batch, b_bs, BK, BN);
    if (r) return r;
    GemmParams p;
    p.M = M; p.N = N; p.K = K; p.batch = batch;
    p.a_mn = a_mn; p.b_mn = b_mn; p.a_fmt = a_fmt; p.b_fmt = b_fmt; p.out_type = out_type;
    p.alpha = alpha; p.beta = beta; p.C = C; p.Cin = Cin;
    p.ldc = ldc; p.c_batch_stride = c_bs; p.ldcin = ldcin; p.cin_batch_stride = cin_bs;
    p.status = status;
    p.split_k = split_k;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * batch * split_k;
    const int grid = tiles < sms ? tiles : sms;
    gemm_tcgen05_kernel<<<grid, 192, SMEM_BYTES, st>>>(tmA, tmB, p);
    return 0;
}
