// Shared device helpers for the sm_100a kernels: vector bf16 access, reductions, the
// status-word convention of bounded waits, and thin wrappers over the PTX used by the
// tensor-core kernels (mbarrier, TMA, tcgen05/TMEM).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#define KB_API extern "C" __attribute__((visibility("default")))

// Status codes written to a status word by kernels whose waits are bounded.
enum KbStatus : int { KB_OK = 0, KB_TIMEOUT_TMA = 1, KB_TIMEOUT_MMA = 2, KB_TIMEOUT_EPI = 3, KB_TIMEOUT_PEER = 4,
                      KB_BAD_ARG = 5, KB_BAD_INDEX = 6 };   // 6: an index read from data (token id, label, cache slot) was out of range; the access was skipped

// Launcher return code for "the launch itself was refused" (bad grid, shared-memory attribute, ...).
#define KB_LAUNCH_FAILED 9
// After a <<<>>>: 0, or KB_LAUNCH_FAILED when the runtime rejected the launch.
static inline int kb_launch_status() { return cudaGetLastError() == cudaSuccess ? 0 : KB_LAUNCH_FAILED; }
// Function attributes (dynamic shared memory opt-in) belong to one device: `flags[64]` remembers
// which devices have been set up.  Returns the flag of the current device, or null.
static inline bool* kb_device_flag(bool* flags) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return flags + dev;
}

// ---- programmatic dependent launch (overlap of a kernel's launch and prologue with its predecessor's tail)
// A kernel launched through kb_launch_dep() may start as soon as every CTA of the kernel before it on the
// stream has executed kb_dep_trigger() (or exited); it must execute kb_dep_wait() before it reads anything
// an earlier kernel wrote and before it writes anything an earlier kernel may still read.  The wait returns
// once the predecessor has completed and its writes are visible; in a kernel launched the ordinary way both
// instructions do nothing.  Every thread of such a kernel executes the wait (before any early return), so
// that "this grid has completed" keeps implying "everything before it has completed".
__device__ __forceinline__ void kb_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void kb_dep_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Process-wide switch (kb_set_dependent_launch; defined in elementwise.cu): 0 = ordinary launches everywhere.
extern int g_kb_dependent_launch;
template <typename... KArgs, typename... Args>
static inline int kb_launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = g_kb_dependent_launch ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...) != cudaSuccess) {
        cudaGetLastError();
        return KB_LAUNCH_FAILED;
    }
    return 0;
}

struct __align__(16) bf16x8 {
    __nv_bfloat162 v[4];
};

// 16-byte accesses go through uint4: a copy of the struct itself is member-wise (the bf16x2 type
// has user-provided copy operations) and was measured to become four 4-byte memory instructions,
// i.e. four times the requests and, for strided rows, eight times the sectors.
__device__ __forceinline__ bf16x8 ld8(const __nv_bfloat16* p) {
    bf16x8 r;
    *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
    return r;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const bf16x8& x) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&x);
}
// p[0..8) += x, rounded to bf16 in the L2 (one 16-byte reduction: no read latency on the issuing
// thread, unlike load-add-store).
__device__ __forceinline__ void red_add8(__nv_bfloat16* p, const bf16x8& x) {
    const uint4 v = *reinterpret_cast<const uint4*>(&x);
    asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ void unpack8(const bf16x8& x, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(x.v[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ bf16x8 pack8(const float* f) {
    bf16x8 r;
#pragma unroll
    for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum NV values across the block; every thread gets the totals.  `scratch` holds
// NV * 32 floats.  Contains two __syncthreads, so it may be reused back to back.
template <int NV>
__device__ __forceinline__ void block_sum(float* vals, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int i = 0; i < NV; ++i) vals[i] = warp_sum(vals[i]);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) scratch[i * 32 + warp] = vals[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        float v = lane < nwarp ? scratch[i * 32 + lane] : 0.f;
        vals[i] = warp_sum(v);
    }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
