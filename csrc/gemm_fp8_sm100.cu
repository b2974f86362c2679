// Block-scaled fp8 (e4m3) GEMM for sm_100a:  C = alpha * (A x B^T) + beta * Cin  with fine-grained scales.
//
//   A [M,K] e4m3, K contiguous, one fp32 scale per row and 128-wide K block     (sa[K/128][M])
//   B [N,K] e4m3, K contiguous, one fp32 scale per `b_gran` rows and K block    (sb[K/128][N/b_gran])
//       b_gran = 128: 128x128 weight blocks;  b_gran = 1: per-row scales (both operands are
//       activations, as in the weight-gradient product, where K is the token dimension)
//
//   TMA (128-byte swizzle; one 128-byte row = one K block = one scale block) -> 4-stage ring ->
//   tcgen05.mma kind::f8f6f4 (128x256x32, four per K block) into a *fresh* TMEM buffer per K block
//   -> the epilogue warps read each partial sum from TMEM, multiply by sa*sb and add it to fp32
//   accumulators in registers (per-K-block promotion), while the tensor core already works on the
//   next K block in the other TMEM buffer.
//
// Roles (320 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2-9 =
// promotion + epilogue (two warps per TMEM lane quarter, 128 columns each, so every scheduler has
// two warps to hide the TMEM load latency; a thread owns half an output row of the tile).
// All waits are bounded (status word).  The reference gets fp8 from torchao's per-tensor dynamic
// scaling (src/training/train.py:301-312); block scaling is the recipe this framework adds.
#include <cuda.h>
#include <cuda_fp8.h>
#include <string.h>

#include "tc.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 128, STAGES = 4, NBUF = 2;
constexpr int A_STAGE = BM * BK, B_STAGE = BN * BK;     // bytes (1 byte per element)
constexpr int EPI_WARPS = 8, EPI_COLS = BN / 2;          // two warps per TMEM lane quarter, 64 columns each
constexpr int SB_BYTES = EPI_WARPS * 2 * EPI_COLS * 4;   // staged B scales: per epilogue warp, double-buffered
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int SMEM_BYTES = STAGES * (A_STAGE + B_STAGE) + 1024 + 256 + SB_BYTES;

struct Fp8Params {
    int M, N, K;
    const float* sa;     // [K/128][M]
    const float* sb;     // [K/128][ceil(N/b_gran)]
    int b_gran, sb_ld;
    int out_type;        // 1 bf16, 2 fp32
    float alpha, beta;
    void* C;
    const void* Cin;
    long long ldc;
    int* status;
};

__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// kind::f8f6f4 instruction descriptor: e4m3 x e4m3 (format code 0), fp32 accumulate, K-major operands.
__device__ __forceinline__ uint32_t instr_desc_f8(int m, int n) {
    uint32_t d = 0;
    d |= 1u << 4;
    d |= (uint32_t)((n >> 3) & 0x3F) << 17;
    d |= (uint32_t)((m >> 4) & 0x1F) << 24;
    return d;
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Fp8Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE + B_STAGE));
    uint64_t* full = bars;                          // [STAGES] TMA -> MMA
    uint64_t* empty = bars + STAGES;                // [STAGES] MMA -> TMA
    uint64_t* part_full = bars + 2 * STAGES;        // [NBUF]   MMA -> promotion
    uint64_t* part_empty = bars + 2 * STAGES + NBUF;  // [NBUF] promotion -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * NBUF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* sbs = reinterpret_cast<float*>(smem + STAGES * (A_STAGE + B_STAGE) + 256);   // [EPI_WARPS][2][EPI_COLS]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int kblocks = p.K / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            tc::mbar_init(&part_full[b], 1);
            tc::mbar_init(&part_empty[b], EPI_WARPS);
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
    constexpr int GROUP_M = 16;

    auto coords = [&](int tile, int& tm, int& tn) {
        const int group = GROUP_M * tiles_n;
        const int g = tile / group;
        const int first_m = g * GROUP_M;
        const int gm = min(GROUP_M, tiles_m - first_m);
        const int t = tile - g * group;
        tm = first_m + t % gm;
        tn = t / gm;
    };

    if (warp == 0) {
        if (lane == 0) {
            tc::prefetch_tmap(&tmA);
            tc::prefetch_tmap(&tmB);
            int stage = 0, issued = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int tm, tn;
                coords(tile, tm, tn);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
                        atomicMax(p.status, (int)KB_TIMEOUT_TMA);
                        ok = false;
                        break;
                    }
                    tc::mbar_expect_tx(&full[stage], A_STAGE + B_STAGE);
                    tc::tma_load_3d(sA + stage * A_STAGE, &tmA, &full[stage], kb * BK, tm * BM, 0);
                    tc::tma_load_3d(sB + stage * B_STAGE, &tmB, &full[stage], kb * BK, tn * BN, 0);
                    ++issued;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
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
        if (lane == 0) {
            const uint32_t idesc = instr_desc_f8(BM, BN);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t it = 0;                     // K blocks issued so far: selects the TMEM buffer
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int buf = it % NBUF;
                    const uint32_t bphase = (it / NBUF) & 1;
                    if (!tc::mbar_wait(&part_empty[buf], bphase ^ 1, abort_flag) ||
                        !tc::mbar_wait(&full[stage], phase, abort_flag)) {
                        atomicMax(p.status, (int)KB_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    tc::tc_fence_after();
                    const uint32_t a_addr = smem_u32(sA + stage * A_STAGE);
                    const uint32_t b_addr = smem_u32(sB + stage * B_STAGE);
                    const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k) {
                        const uint64_t ad = tc::smem_desc_sw128(a_addr + k * 32, 16, 1024);
                        const uint64_t bd = tc::smem_desc_sw128(b_addr + k * 32, 16, 1024);
                        mma_f8(d_tmem, ad, bd, idesc, k != 0);
                    }
                    tc::tc_commit(&empty[stage]);
                    tc::tc_commit(&part_full[buf]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else {
        const int quarter = warp & 3;                 // TMEM lanes [32*quarter, +32)
        const int half = (warp - 2) >> 2;             // columns [64*half, +64) of the tile
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            int tm, tn;
            coords(tile, tm, tn);
            const int row = tm * BM + quarter * 32 + lane;
            const int rowc = min(row, p.M - 1);
            const int colbase = tn * BN + half * EPI_COLS;
            float acc[EPI_COLS];
#pragma unroll
            for (int j = 0; j < EPI_COLS; ++j) acc[j] = 0.f;
            for (int kb = 0; kb < kblocks && ok; ++kb, ++it) {
                const int buf = it % NBUF;
                const uint32_t bphase = (it / NBUF) & 1;
                const float a_scale = __ldg(p.sa + (long long)kb * p.M + rowc);
                float b_scale = 0.f;
                // per-column scales are staged per warp (no cross-warp barrier: every wait here must
                // stay bounded), double-buffered so a fast lane never overwrites what a slow one reads
                float* sbk = sbs + ((warp - 2) * 2 + (kb & 1)) * EPI_COLS;
                if (p.b_gran == 1) {
#pragma unroll
                    for (int j = 0; j < EPI_COLS / 32; ++j) {
                        const int col = colbase + j * 32 + lane;
                        sbk[j * 32 + lane] = col < p.N ? __ldg(p.sb + (long long)kb * p.sb_ld + col) : 0.f;
                    }
                    __syncwarp();
                } else {
                    b_scale = __ldg(p.sb + (long long)kb * p.sb_ld + colbase / p.b_gran) * a_scale;
                }
                if (!tc::mbar_wait(&part_full[buf], bphase, abort_flag)) {
                    if (lane == 0) atomicMax(p.status, (int)KB_TIMEOUT_EPI);
                    ok = false;
                    break;
                }
                tc::tc_fence_after();
                const uint32_t taddr = tmem_base + buf * BN + half * EPI_COLS + ((uint32_t)(quarter * 32) << 16);
                const float sc = b_scale;
#pragma unroll
                for (int c = 0; c < EPI_COLS / 16; ++c) {      // 16-column chunks: 128 accumulators leave few registers
                    uint32_t v[16];
                    tc::tmem_ld16(taddr + c * 16, v);
                    tc::tmem_ld_wait();
                    if (p.b_gran == 1) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            acc[c * 16 + j] = fmaf(__uint_as_float(v[j]), a_scale * sbk[c * 16 + j], acc[c * 16 + j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[c * 16 + j] = fmaf(__uint_as_float(v[j]), sc, acc[c * 16 + j]);
                    }
                }
                tc::tc_fence_before();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&part_empty[buf]);
            }
            if (!ok) break;
            if (row < p.M && colbase < p.N) {
                const int ncols = min(EPI_COLS, p.N - colbase);
                const long long off = (long long)row * p.ldc + colbase;
                if (p.out_type == 2) {
                    float* dst = reinterpret_cast<float*>(p.C) + off;
                    const float* cin = p.Cin ? reinterpret_cast<const float*>(p.Cin) + off : nullptr;
                    if (ncols == EPI_COLS && ((p.ldc | colbase) & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < EPI_COLS; j += 4) {
                            float4 o = make_float4(p.alpha * acc[j], p.alpha * acc[j + 1], p.alpha * acc[j + 2],
                                                   p.alpha * acc[j + 3]);
                            if (cin) {
                                const float4 ci = *reinterpret_cast<const float4*>(cin + j);
                                o.x += p.beta * ci.x; o.y += p.beta * ci.y; o.z += p.beta * ci.z; o.w += p.beta * ci.w;
                            }
                            *reinterpret_cast<float4*>(dst + j) = o;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < EPI_COLS; ++j)
                            if (j < ncols) dst[j] = p.alpha * acc[j] + (cin ? p.beta * cin[j] : 0.f);
                    }
                } else {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
                    const __nv_bfloat16* cin = p.Cin ? reinterpret_cast<const __nv_bfloat16*>(p.Cin) + off : nullptr;
                    if (ncols == EPI_COLS && ((p.ldc | colbase) & 7) == 0) {
#pragma unroll
                        for (int j = 0; j < EPI_COLS; j += 8) {
                            float o[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) o[i] = p.alpha * acc[j + i];
                            if (cin) {
                                float ci[8];
                                unpack8(ld8(cin + j), ci);
#pragma unroll
                                for (int i = 0; i < 8; ++i) o[i] += p.beta * ci[i];
                            }
                            st8(dst + j, pack8(o));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < EPI_COLS; ++j)
                            if (j < ncols)
                                dst[j] = __float2bfloat16(p.alpha * acc[j] + (cin ? p.beta * __bfloat162float(cin[j]) : 0.f));
                    }
                }
            }
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
// 8-bit matrix [rows, cols], cols contiguous, row stride ld bytes.
int make_tmap8(CUtensorMap* m, const void* base, long long cols, long long rows, long long ld, int box_cols,
               int box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return 100;
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, 1};
    cuuint64_t strides[2] = {(cuuint64_t)ld, (cuuint64_t)(rows * ld)};
    cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 200 + (int)r;
}

}  // namespace

// C[M,N] = alpha * sum_kb (A_kb x B_kb^T) * sa[kb][m] * sb[kb][n / b_gran]  + beta * Cin.
// A [M,K], B [N,K] e4m3 with K contiguous (lda/ldb in elements = bytes, multiples of 16);
// K a multiple of 128; sa is [K/128][M]; sb is [K/128][sb_ld]; b_gran is 128 (block scales) or 1.
// out_type 1 = bf16, 2 = fp32; Cin (nullable, may alias C) has C's type and layout.
KB_API int kb_gemm_fp8(const void* A, const void* B, const float* sa, const float* sb, void* C, const void* Cin,
                       int M, int N, int K, long long lda, long long ldb, long long ldc, int b_gran, int sb_ld,
                       int out_type, float alpha, float beta, int* status, int max_ctas, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0 || (K % BK) != 0) return 5;
    if (b_gran != 1 && b_gran != 128) return 5;
    if (out_type != 1 && out_type != 2) return 5;
    if ((lda & 15) || (ldb & 15) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return 6;
    static bool attr_flags[64] = {};
    bool* attr_set_p = kb_device_flag(attr_flags);
    if (!attr_set_p) return 7;
    if (!*attr_set_p) {
        if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
            return 7;
        *attr_set_p = true;
    }
    CUtensorMap tmA, tmB;
    int r = make_tmap8(&tmA, A, K, M, lda, BK, BM);
    if (r) return r;
    r = make_tmap8(&tmB, B, K, N, ldb, BK, BN);
    if (r) return r;
    Fp8Params p;
    memset(&p, 0, sizeof(p));
    p.M = M; p.N = N; p.K = K; p.sa = sa; p.sb = sb; p.b_gran = b_gran; p.sb_ld = sb_ld; p.out_type = out_type;
    p.alpha = alpha; p.beta = beta; p.C = C; p.Cin = Cin; p.ldc = ldc; p.status = status;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    gemm_fp8_kernel<<<tiles < sms ? tiles : sms, THREADS, SMEM_BYTES, st>>>(tmA, tmB, p);
    const cudaError_t le = cudaGetLastError();
    return le == cudaSuccess ? 0 : 300 + (int)le;
}
