// In-kernel collectives over NVLink peer memory (symmetric heap: the same buffer mapped at a
// per-rank address on every GPU).  Data moves by plain loads/stores on peer pointers; ordering
// is by epoch flags written with release semantics after a system fence and polled with
// acquire loads.  Every poll is bounded by a time limit; a wait that runs out records
// KB_TIMEOUT_PEER in the status word and the kernel returns normally, so the context survives
// and the host can raise.  Epochs only grow: flags are never reset.
//
//   kb_flag_signal      this rank raises flag[slot][rank] on every peer
//   kb_flag_wait        wait until flag[slot][r] >= epoch for every r (local memory)
//   kb_reduce_to_owner  owner sums a gradient range over all ranks (fp32), scales, stores bf16
//   kb_allreduce_slices two-shot all-reduce: each rank reduces its slice, stores it to every peer
//   kb_scalar_allreduce sum of one float per rank (also a full barrier)
//   kb_packed_allreduce sum of up to 8 floats per rank in one launch (tensor-parallel loss and norm terms)
//   kb_ag_push          all-gather producer: this rank's shard into every peer's staging slot, then
//                       the shard's ready flag (consumed by kb_gemm_ag's TMA producer)
//   kb_rs_reduce        reduce-scatter consumer: waits for the arrival counters that kb_gemm_rs's
//                       epilogue raises, sums the per-source slabs (+ residual), frees the slabs
//   kb_allreduce_oneshot small all-reduce for decode: every rank reads every peer's partial
//   kb_allreduce_multimem the same small all-reduce with the sum done in NVSwitch (multimem.ld_reduce)
//   kb_muon_apply_bcast p_new = p*decay - alpha*orth written into every rank's parameter arena
//                       (the all-gather of the updated matrix is the parameter write itself)
#include "common.cuh"

typedef __nv_bfloat16 bf16;

struct PeerPtrs {
    void* p[8];
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Bounded poll on a local flag.  Returns false on timeout.  The loop polls with relaxed loads
// and a growing sleep, and fences once at the end: a tight loop of system-scope acquire loads
// from a kernel that waits on a side stream was measured to slow concurrently running GEMMs
// by 1.5x at 4 and 8 ranks.
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, uint64_t limit_ns) {
    if (ld_acquire_sys(flag) >= epoch) return true;
    const uint64_t t0 = global_timer_ns();
    unsigned sleep_ns = 128;
    while (ld_relaxed_sys(flag) < epoch) {
        if (global_timer_ns() - t0 > limit_ns) return false;
        __nanosleep(sleep_ns);
        if (sleep_ns < 2048) sleep_ns <<= 1;
    }
    __threadfence_system();
    return ld_acquire_sys(flag) >= epoch;
}

// flags layout on every rank: int flags[slots][8]
__global__ void flag_signal_kernel(PeerPtrs flags, int world, int rank, int slot, int epoch) {
    if (threadIdx.x < world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + slot * 8 + rank, epoch);
    }
}
__global__ void flag_wait_kernel(const int* flags, int world, int slot, int epoch, unsigned long long limit_ns,
                                 int* status) {
    if (threadIdx.x < world) {
        if (!wait_flag(flags + slot * 8 + threadIdx.x, epoch, limit_ns)) atomicMax(status, (int)KB_TIMEOUT_PEER);
    }
}

KB_API int kb_flag_signal(void* const* peer_flags, int world, int rank, int slot, int epoch, cudaStream_t st) {
    if (world < 1 || world > 8) return 5;
    PeerPtrs pp;
    for (int i = 0; i < 8; ++i) pp.p[i] = i < world ? peer_flags[i] : nullptr;
    flag_signal_kernel<<<1, 32, 0, st>>>(pp, world, rank, slot, epoch);
    return kb_launch_status();
}
KB_API int kb_flag_wait(const int* flags, int world, int slot, int epoch, double limit_s, int* status,
                        cudaStream_t st) {
    if (world < 1 || world > 8) return 5;
    flag_wait_kernel<<<1, 32, 0, st>>>(flags, world, slot, epoch, (unsigned long long)(limit_s * 1e9), status);
    return kb_launch_status();
}

// out[i] = scale * sum_r peer[r][offset + i]  for i in [0, n); out is this rank's own buffer range.
template <int U>
__device__ __forceinline__ void reduce_vecs(const PeerPtrs& bufs, int world, long long offset, long long i0,
                                            long long stride, long long nvec, float scale, bf16* __restrict__ out) {
    // U independent 16-byte loads per rank are issued before any is consumed: NVLink reads are
    // latency-bound, so bytes in flight per thread set the bandwidth.
    uint4 raw[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (r < world && i < nvec)
                raw[u][r] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(bufs.p[r]) + offset) + i);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i >= nvec) continue;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < world) {
                float t[8];
                unpack8(*reinterpret_cast<const bf16x8*>(&raw[u][r]), t);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += t[j];
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= scale;
        st8(out + i * 8, pack8(acc));
    }
}

__global__ void __launch_bounds__(256)
reduce_to_owner_kernel(PeerPtrs bufs, int world, long long offset, long long n, float scale,
                       bf16* __restrict__ out) {
    const long long nvec = n >> 3;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += 2 * stride)
        reduce_vecs<2>(bufs, world, offset, i, stride, nvec, scale, out);
    // tail (n not a multiple of 8)
    for (long long i = (nvec << 3) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        float a = 0.f;
        for (int r = 0; r < world; ++r) a += __bfloat162float(reinterpret_cast<const bf16*>(bufs.p[r])[offset + i]);
        out[i] = __float2bfloat16(a * scale);
    }
}
KB_API int kb_reduce_to_owner(void* const* peer_bufs, int world, long long offset, long long n, float scale,
                              void* out, int max_ctas, cudaStream_t st) {
    if (world < 1 || world > 8 || (offset & 7)) return 5;
    PeerPtrs pp;
    for (int i = 0; i < 8; ++i) pp.p[i] = i < world ? peer_bufs[i] : nullptr;
    long long blocks = ((n >> 3) + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > max_ctas) blocks = max_ctas;
    reduce_to_owner_kernel<<<(int)blocks, 256, 0, st>>>(pp, world, offset, n, scale, (bf16*)out);
    return kb_launch_status();
}

// Two-shot all-reduce of [offset, offset+n): rank r owns the r-th of `world` equal slices
// (8-element granularity), reduces it over all ranks and stores the result to every rank.
__global__ void allreduce_slices_kernel(PeerPtrs bufs, int world, int rank, long long offset, long long n,
                                        float scale) {
    const long long nvec = (n + 7) >> 3;                 // caller pads the range to a multiple of 8
    const long long per = (nvec + world - 1) / world;
    const long long lo = per * rank, hi = min(nvec, lo + per);
    for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi;
         i += (long long)gridDim.x * blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int r = 0; r < world; ++r) {
            const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(bufs.p[r]) + offset) + i);
            float t[8];
            unpack8(*reinterpret_cast<const bf16x8*>(&raw), t);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += t[j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= scale;
        const bf16x8 o = pack8(acc);
        for (int r = 0; r < world; ++r)
            st8(reinterpret_cast<bf16*>(bufs.p[r]) + offset + i * 8, o);
    }
}
KB_API int kb_allreduce_slices(void* const* peer_bufs, int world, int rank, long long offset, long long n,
                               float scale, int max_ctas, cudaStream_t st) {
    if (world < 1 || world > 8 || (offset & 7) || (n & 7)) return 5;
    PeerPtrs pp;
    for (int i = 0; i < 8; ++i) pp.p[i] = i < world ? peer_bufs[i] : nullptr;
    long long blocks = ((n >> 3) / world + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > max_ctas) blocks = max_ctas;
    allreduce_slices_kernel<<<(int)blocks, 256, 0, st>>>(pp, world, rank, offset, n, scale);
    return kb_launch_status();
}

// Sum of one float per rank; doubles as a barrier.  vals layout on every rank: float vals[2][8]
// (double-buffered by epoch parity), flags as above.
__global__ void scalar_allreduce_kernel(PeerPtrs vals, PeerPtrs flags, int world, int rank, int slot, int epoch,
                                        const float* __restrict__ in, float* __restrict__ out,
                                        unsigned long long limit_ns, int* status) {
    __shared__ int ok;
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    const int par = epoch & 1;
    if (threadIdx.x < world) {
        if (in) reinterpret_cast<float*>(vals.p[threadIdx.x])[par * 8 + rank] = in[0];
        __threadfence_system();
        st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + slot * 8 + rank, epoch);
        if (!wait_flag(reinterpret_cast<const int*>(flags.p[rank]) + slot * 8 + threadIdx.x, epoch, limit_ns)) {
            atomicMax(status, (int)KB_TIMEOUT_PEER);
            ok = 0;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && out) {
        float s = 0.f;
        if (ok) {
            const volatile float* mine = reinterpret_cast<const volatile float*>(vals.p[rank]) + par * 8;
            for (int r = 0; r < world; ++r) s += mine[r];
        }
        out[0] = s;
    }
}
KB_API int kb_scalar_allreduce(void* const* peer_vals, void* const* peer_flags, int world, int rank, int slot,
                               int epoch, const float* in, float* out, double limit_s, int* status,
                               cudaStream_t st) {
    if (world < 1 || world > 8) return 5;
    PeerPtrs pv, pf;
    for (int i = 0; i < 8; ++i) {
        pv.p[i] = i < world ? peer_vals[i] : nullptr;
        pf.p[i] = i < world ? peer_flags[i] : nullptr;
    }
    scalar_allreduce_kernel<<<1, 32, 0, st>>>(pv, pf, world, rank, slot, epoch, in, out,
                                              (unsigned long long)(limit_s * 1e9), status);
    return kb_launch_status();
}

// Packed small all-reduce: up to 8 floats per rank summed in one launch (loss terms, squared gradient
// norms: the reductions a tensor-parallel step needs besides its activation collectives).  Every rank
// stores its `count` values into slot [parity][rank] of every peer, raises its flag there, waits for
// all flags and sums in rank order - bitwise identical on every rank.  vals layout on every rank:
// float vals[2][8][8]; flags as above.
__global__ void packed_allreduce_kernel(PeerPtrs vals, PeerPtrs flags, int world, int rank, int slot, int epoch,
                                        const float* __restrict__ in, float* __restrict__ out, int count,
                                        unsigned long long limit_ns, int* status) {
    __shared__ int ok;
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    const int par = epoch & 1;
    if (threadIdx.x < world) {
        float* dst = reinterpret_cast<float*>(vals.p[threadIdx.x]) + (par * 8 + rank) * 8;
        for (int j = 0; j < count; ++j) dst[j] = in[j];
        __threadfence_system();
        st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + slot * 8 + rank, epoch);
        if (!wait_flag(reinterpret_cast<const int*>(flags.p[rank]) + slot * 8 + threadIdx.x, epoch, limit_ns)) {
            atomicMax(status, (int)KB_TIMEOUT_PEER);
            ok = 0;
        }
    }
    __syncthreads();
    if (threadIdx.x < count) {
        float s = 0.f;
        if (ok) {
            const volatile float* mine = reinterpret_cast<const volatile float*>(vals.p[rank]) + par * 64;
            for (int r = 0; r < world; ++r) s += mine[r * 8 + threadIdx.x];
        }
        out[threadIdx.x] = s;
    }
}
KB_API int kb_packed_allreduce(void* const* peer_vals, void* const* peer_flags, int world, int rank, int slot,
                               int epoch, const float* in, float* out, int count, double limit_s, int* status,
                               cudaStream_t st) {
    if (world < 1 || world > 8 || count < 1 || count > 8 || !in || !out) return 5;
    PeerPtrs pv, pf;
    for (int i = 0; i < 8; ++i) {
        pv.p[i] = i < world ? peer_vals[i] : nullptr;
        pf.p[i] = i < world ? peer_flags[i] : nullptr;
    }
    packed_allreduce_kernel<<<1, 32, 0, st>>>(pv, pf, world, rank, slot, epoch, in, out, count,
                                              (unsigned long long)(limit_s * 1e9), status);
    return kb_launch_status();
}

// Owner's Muon parameter write, broadcast: every rank's arena gets p*decay - alpha*orth.
// params.p[r] is rank r's arena base; the matrix sits at `offset`, shape [R,C]; orth is fp16
// [R,C], or [C,R] when `transposed`.
// 64x64 tiles, block (8, 32): thread (x, y) owns 8 consecutive columns of rows y and y+32.
__global__ void __launch_bounds__(256)
muon_apply_bcast_kernel(PeerPtrs params, int world, int rank, long long offset, const __half* __restrict__ o,
                        int R, int C, float decay, float alpha, int transposed) {
    __shared__ float tile[64][65];
    const int bx = blockIdx.x * 64, by = blockIdx.y * 64;
    const bf16* mine = reinterpret_cast<const bf16*>(params.p[rank]) + offset;
    if (transposed) {
        // o is [C,R]: tile[j][i] = o[bx + j][by + i]
        for (int j = threadIdx.y; j < 64; j += 32) {
            const int oc = bx + j;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int orow = by + threadIdx.x * 8 + e;
                tile[j][threadIdx.x * 8 + e] = (oc < C && orow < R) ? __half2float(o[(size_t)oc * R + orow]) : 0.f;
            }
        }
        __syncthreads();
    }
    const bool vec = (C & 7) == 0 && (offset & 7) == 0;
    for (int j = threadIdx.y; j < 64; j += 32) {
        const int r = by + j, c0 = bx + threadIdx.x * 8;
        if (r >= R || c0 >= C) continue;
        const size_t idx = (size_t)r * C + c0;
        if (vec && c0 + 8 <= C) {
            float p[8], ov[8];
            unpack8(ld8(mine + idx), p);
            if (transposed) {
#pragma unroll
                for (int e = 0; e < 8; ++e) ov[e] = tile[threadIdx.x * 8 + e][j];
            } else {
                const uint4 raw = *reinterpret_cast<const uint4*>(o + idx);
                const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
                for (int e = 0; e < 8; ++e) ov[e] = __half2float(h[e]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) p[e] = p[e] * decay - alpha * ov[e];
            const bf16x8 v = pack8(p);
            for (int q = 0; q < world; ++q) st8(reinterpret_cast<bf16*>(params.p[q]) + offset + idx, v);
        } else {
            for (int e = 0; e < 8 && c0 + e < C; ++e) {
                const float ov = transposed ? tile[threadIdx.x * 8 + e][j] : __half2float(o[idx + e]);
                const bf16 v = __float2bfloat16(__bfloat162float(mine[idx + e]) * decay - alpha * ov);
                for (int q = 0; q < world; ++q) (reinterpret_cast<bf16*>(params.p[q]) + offset)[idx + e] = v;
            }
        }
    }
}
KB_API int kb_muon_apply_bcast(void* const* peer_params, int world, int rank, long long offset, const void* orth,
                               int R, int C, float lr, float wd, float scale, int transposed, cudaStream_t st) {
    if (world < 1 || world > 8) return 5;
    PeerPtrs pp;
    for (int i = 0; i < 8; ++i) pp.p[i] = i < world ? peer_params[i] : nullptr;
    dim3 grid((C + 63) / 64, (R + 63) / 64), block(8, 32);
    muon_apply_bcast_kernel<<<grid, block, 0, st>>>(pp, world, rank, offset, (const __half*)orth, R, C,
                                                    wd > 0 ? 1.f - lr * wd : 1.f, lr * scale, transposed);
    return kb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// Tensor-parallel collectives fused with the GEMMs (sequence parallelism).

// Last-block election: returns true in every thread of the block that finishes last.
__device__ __forceinline__ bool last_block_done(unsigned* counter) {
    __shared__ int s_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(counter, 1u);
        s_last = prev == gridDim.x - 1;
        if (s_last) *counter = 0;
    }
    __syncthreads();
    return s_last != 0;
}

// Shard push.  stage.p[q] = peer q's staging slot for this source rank; ready.p[q] = address of
// this rank's ready flag on peer q.  `done[q]` (local) is the last call whose staging buffer peer q
// has finished reading; the slot may be overwritten once done[q] >= need.  Targets are the
// `count` ranks starting at `first` (cyclically): the caller pushes to itself first (a local
// copy, so its GEMM can start at once) and to the peers from a side stream.
__global__ void __launch_bounds__(256)
ag_push_kernel(const uint4* __restrict__ src, long long nvec, PeerPtrs stage, PeerPtrs ready, int world, int first,
               int count, int epoch, const int* done, int need, unsigned* counter, unsigned long long limit_ns,
               int* status) {
    __shared__ int ok;
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    if (need > 0 && threadIdx.x < count) {
        if (!wait_flag(done + (first + threadIdx.x) % world, need, limit_ns)) {
            atomicMax(status, (int)KB_TIMEOUT_PEER);
            ok = 0;
        }
    }
    __syncthreads();
    const bool good = ok != 0;
    if (good) {
        const long long stride = (long long)gridDim.x * blockDim.x;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
            const uint4 v = __ldg(src + i);
            for (int t = 0; t < count; ++t) {
                int q = first + t;
                if (q >= world) q -= world;
                reinterpret_cast<uint4*>(stage.p[q])[i] = v;
            }
        }
    }
    if (last_block_done(counter) && good && threadIdx.x < count) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<int*>(ready.p[(first + threadIdx.x) % world]), epoch);
    }
}
KB_API int kb_ag_push(const void* src, long long n_elems, void* const* peer_stage, void* const* peer_ready, int world,
                      int first, int count, int epoch, const int* done, int need, unsigned* counter, double limit_s,
                      int* status, int max_ctas, cudaStream_t st) {
    if (world < 1 || world > 8 || (n_elems & 7) || ((uintptr_t)src & 15)) return 5;
    if (first < 0 || first >= world || count < 1 || count > world) return 5;
    PeerPtrs ps, pr;
    for (int i = 0; i < 8; ++i) {
        ps.p[i] = i < world ? peer_stage[i] : nullptr;
        pr.p[i] = i < world ? peer_ready[i] : nullptr;
    }
    const long long nvec = n_elems >> 3;
    long long blocks = (nvec + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > max_ctas) blocks = max_ctas;
    ag_push_kernel<<<(int)blocks, 256, 0, st>>>((const uint4*)src, nvec, ps, pr, world, first, count, epoch, done,
                                                need, counter, (unsigned long long)(limit_s * 1e9), status);
    return kb_launch_status();
}

// out[i] = sum_s slab[s][i] (+ residual[i]) once cnt[s] >= expected (arrivals of this call) for
// every source s; then the counters are zeroed and
// `done_epoch` is written to this rank's slot on every peer: the slabs may be reused.
__global__ void __launch_bounds__(256)
rs_reduce_kernel(const bf16* __restrict__ slabs, long long slab_elems, int* cnt, int expected, int world,
                 const bf16* __restrict__ residual, bf16* __restrict__ out, PeerPtrs done, int done_epoch,
                 unsigned* counter, unsigned long long limit_ns, int* status) {
    __shared__ int ok;
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    if (threadIdx.x < world) {
        if (!wait_flag(cnt + threadIdx.x, expected, limit_ns)) {
            atomicMax(status, (int)KB_TIMEOUT_PEER);
            ok = 0;
        }
    }
    __syncthreads();
    const bool good = ok != 0;
    if (good) {
        const long long nvec = slab_elems >> 3;
        const long long stride = (long long)gridDim.x * blockDim.x;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
            float acc[8];
            if (residual) unpack8(ld8(residual + i * 8), acc);
            else {
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            }
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                if (s < world) {
                    float t[8];
                    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(slabs + s * slab_elems) + i);
                    unpack8(*reinterpret_cast<const bf16x8*>(&raw), t);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] += t[j];
                }
            }
            st8(out + i * 8, pack8(acc));
        }
    }
    if (last_block_done(counter) && good && threadIdx.x < world) {
        // every block has read the slabs: zero the arrival counters for the call after next (its
        // producers start only after they have seen the done flag below), then release the slabs
        cnt[threadIdx.x] = 0;
        __threadfence_system();
        __syncwarp(__activemask());
        st_release_sys(reinterpret_cast<int*>(done.p[threadIdx.x]), done_epoch);
    }
}
KB_API int kb_rs_reduce(const void* slabs, long long slab_elems, int* cnt, int expected, int world,
                        const void* residual, void* out, void* const* peer_done, int done_epoch, unsigned* counter,
                        double limit_s, int* status, int max_ctas, cudaStream_t st) {
    if (world < 1 || world > 8 || (slab_elems & 7)) return 5;
    PeerPtrs pd;
    for (int i = 0; i < 8; ++i) pd.p[i] = i < world ? peer_done[i] : nullptr;
    long long blocks = ((slab_elems >> 3) + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > max_ctas) blocks = max_ctas;
    rs_reduce_kernel<<<(int)blocks, 256, 0, st>>>((const bf16*)slabs, slab_elems, cnt, expected, world,
                                                  (const bf16*)residual, (bf16*)out, pd, done_epoch, counter,
                                                  (unsigned long long)(limit_s * 1e9), status);
    return kb_launch_status();
}

// One-shot all-reduce of a small bf16 vector (decode-time row-parallel outputs): every rank's
// partial already sits in its own symmetric buffer (the GEMM wrote it there); block 0 raises this
// rank's flag on every peer, every block waits for all flags, then each rank sums all partials for
// itself.  out = sum_r partial_r (+ residual).  Buffers alternate by call parity on the host side.
__global__ void __launch_bounds__(256)
allreduce_oneshot_kernel(PeerPtrs parts, PeerPtrs flags, int world, int rank, int slot, int epoch, long long n,
                         const bf16* __restrict__ residual, bf16* __restrict__ out, unsigned long long limit_ns,
                         int* status) {
    __shared__ int ok;
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    if (threadIdx.x < world) {
        if (blockIdx.x == 0) {
            __threadfence_system();
            st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + slot * 8 + rank, epoch);
        }
        if (!wait_flag(reinterpret_cast<const int*>(flags.p[rank]) + slot * 8 + threadIdx.x, epoch, limit_ns)) {
            atomicMax(status, (int)KB_TIMEOUT_PEER);
            ok = 0;
        }
    }
    __syncthreads();
    if (!ok) return;
    const long long nvec = n >> 3;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
        uint4 raw[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (r < world) raw[r] = __ldcg(reinterpret_cast<const uint4*>(parts.p[r]) + i);
        float acc[8];
        if (residual) unpack8(ld8(residual + i * 8), acc);
        else {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < world) {
                float t[8];
                unpack8(*reinterpret_cast<const bf16x8*>(&raw[r]), t);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += t[j];
            }
        }
        st8(out + i * 8, pack8(acc));
    }
}
KB_API int kb_allreduce_oneshot(void* const* peer_parts, void* const* peer_flags, int world, int rank, int slot,
                                int epoch, long long n, const void* residual, void* out, double limit_s, int* status,
                                int max_ctas, cudaStream_t st) {
    if (world < 1 || world > 8 || (n & 7)) return 5;
    PeerPtrs pp, pf;
    for (int i = 0; i < 8; ++i) {
        pp.p[i] = i < world ? peer_parts[i] : nullptr;
        pf.p[i] = i < world ? peer_flags[i] : nullptr;
    }
    long long blocks = ((n >> 3) + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > max_ctas) blocks = max_ctas;
    allreduce_oneshot_kernel<<<(int)blocks, 256, 0, st>>>(pp, pf, world, rank, slot, epoch, n, (const bf16*)residual,
                                                          (bf16*)out, (unsigned long long)(limit_s * 1e9), status);
    return kb_launch_status();
}

// Graph-replayable all-reduce for decode-sized activations (row-parallel projections under tensor
// parallelism: 2 per layer and step, latency-bound).  Nothing on the host changes between calls:
// the call number lives in device memory (`epoch_ptr`, advanced by the last block on the way
// out), so a captured launch can be replayed.  Push protocol: every rank stores its partial into
// slot [parity][rank] of every rank's receive buffer, the last block to finish its stores raises
// this rank's flag [parity][rank] everywhere, all blocks then wait (bounded) for the `world` flags
// and sum the local slots in rank order (bitwise identical on every rank) plus the residual.
// The grid must be co-resident (<= one block per SM): blocks wait for each other's stores.
__global__ void __launch_bounds__(256)
allreduce_push_kernel(const uint4* __restrict__ x, long long nvec, long long slot_vecs, PeerPtrs recv, PeerPtrs flags,
                      int world, int rank, const bf16* __restrict__ residual, bf16* __restrict__ out, int* epoch_ptr,
                      unsigned* counters, unsigned long long limit_ns, int* status) {
    __shared__ int ok;
    const int epoch = *reinterpret_cast<volatile int*>(epoch_ptr) + 1;
    const int par = epoch & 1;
    if (threadIdx.x == 0) ok = 1;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long my_slot = ((long long)par * world + rank) * slot_vecs;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const uint4 v = x[i];
#pragma unroll
        for (int q = 0; q < 8; ++q)
            if (q < world) (reinterpret_cast<uint4*>(recv.p[q]) + my_slot)[i] = v;
    }
    if (last_block_done(counters) && threadIdx.x < world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + par * 8 + rank, epoch);
    }
    if (threadIdx.x < world) {
        if (!wait_flag(reinterpret_cast<const int*>(flags.p[rank]) + par * 8 + threadIdx.x, epoch, limit_ns)) {
            atomicMax(status, (int)KB_TIMEOUT_PEER);
            ok = 0;
        }
    }
    __syncthreads();
    if (ok) {
        const uint4* mine = reinterpret_cast<const uint4*>(recv.p[rank]) + (long long)par * world * slot_vecs;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
            float acc[8];
            if (residual) unpack8(ld8(residual + i * 8), acc);
            else {
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (r < world) {
                    float t[8];
                    const uint4 raw = __ldcg(mine + r * slot_vecs + i);
                    unpack8(*reinterpret_cast<const bf16x8*>(&raw), t);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] += t[j];
                }
            }
            st8(out + i * 8, pack8(acc));
        }
    }
    if (last_block_done(counters + 1) && threadIdx.x == 0) *epoch_ptr = epoch;
}
// The same all-reduce with the reduction done inside NVSwitch (`multimem.ld_reduce`).  Every rank
// keeps its partial in its OWN symmetric buffer (slot [parity]); `mc_base` is the multicast address
// of that buffer: one 16-byte `multimem.ld_reduce.add` at offset i returns the sum over all ranks'
// buffers at offset i, accumulated in fp32 by the switch.  Per call a rank sends nothing and
// receives n elements, where the push form receives (world - 1) * n.  Flags and the device-side
// call number are as above.  The multicast object covers symmetric buffers of this job's own ranks only.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc_addr)
                 : "memory");
    return v;
}
__global__ void __launch_bounds__(256)
allreduce_multimem_kernel(const uint4* __restrict__ x, long long nvec, long long slot_vecs, uint4* sym_local,
                          const uint4* mc_base, PeerPtrs flags, int world, int rank,
                          const bf16* __restrict__ residual, bf16* __restrict__ out, int* epoch_ptr, unsigned* counters,
                          unsigned long long limit_ns, int* status) {
    __shared__ int ok;
    const int epoch = *reinterpret_cast<volatile int*>(epoch_ptr) + 1;
    const int par = epoch & 1;
    if (threadIdx.x == 0) ok = 1;
    const long long stride = (long long)gridDim.x * blockDim.x;
    uint4* mine = sym_local + (long long)par * slot_vecs;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) mine[i] = x[i];
    if (last_block_done(counters) && threadIdx.x < world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + par * 8 + rank, epoch);
    }
    if (threadIdx.x < world) {
        if (!wait_flag(reinterpret_cast<const int*>(flags.p[rank]) + par * 8 + threadIdx.x, epoch, limit_ns)) {
            atomicMax(status, (int)KB_TIMEOUT_PEER);
            ok = 0;
        }
    }
    __syncthreads();
    if (ok) {
        const uint4* mc = mc_base + (long long)par * slot_vecs;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
            const uint4 raw = multimem_ld_reduce_bf16x8(mc + i);
            if (residual) {
                float acc[8], t[8];
                unpack8(ld8(residual + i * 8), acc);
                unpack8(*reinterpret_cast<const bf16x8*>(&raw), t);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += t[j];
                st8(out + i * 8, pack8(acc));
            } else {
                *reinterpret_cast<uint4*>(out + i * 8) = raw;
            }
        }
    }
    if (last_block_done(counters + 1) && threadIdx.x == 0) *epoch_ptr = epoch;
}
// sym_local: this rank's symmetric buffer of 2 * slot_elems bf16; mc_base: the multicast address of the
// same buffer; the rest as kb_allreduce_push.
KB_API int kb_allreduce_multimem(const void* x, long long n, long long slot_elems, void* sym_local, const void* mc_base,
                                 void* const* peer_flags, int world, int rank, const void* residual, void* out,
                                 int* epoch_ptr, unsigned* counters, double limit_s, int* status, int max_ctas,
                                 cudaStream_t st) {
    if (world < 1 || world > 8 || (n & 7) || (slot_elems & 7) || n > slot_elems || ((uintptr_t)x & 15)) return 5;
    if (!sym_local || !mc_base || ((uintptr_t)sym_local & 15) || ((uintptr_t)mc_base & 15)) return 6;
    PeerPtrs pf;
    for (int i = 0; i < 8; ++i) pf.p[i] = i < world ? peer_flags[i] : nullptr;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (max_ctas < 1 || max_ctas > sms) max_ctas = sms;
    long long blocks = ((n >> 3) + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > max_ctas) blocks = max_ctas;
    allreduce_multimem_kernel<<<(int)blocks, 256, 0, st>>>((const uint4*)x, n >> 3, slot_elems >> 3, (uint4*)sym_local,
                                                           (const uint4*)mc_base, pf, world, rank, (const bf16*)residual,
                                                           (bf16*)out, epoch_ptr, counters,
                                                           (unsigned long long)(limit_s * 1e9), status);
    return kb_launch_status();
}

// x: this rank's partial (n bf16 elements, 16-byte aligned, n % 8 == 0); peer_recv[q]: rank q's
// receive buffer of 2 * world * slot_elems elements; peer_flags[q]: rank q's 16 flag ints;
// epoch_ptr / counters (2 unsigned, zero-initialised): local device memory.
KB_API int kb_allreduce_push(const void* x, long long n, long long slot_elems, void* const* peer_recv,
                             void* const* peer_flags, int world, int rank, const void* residual, void* out,
                             int* epoch_ptr, unsigned* counters, double limit_s, int* status, int max_ctas,
                             cudaStream_t st) {
    if (world < 1 || world > 8 || (n & 7) || (slot_elems & 7) || n > slot_elems || ((uintptr_t)x & 15)) return 5;
    PeerPtrs pr, pf;
    for (int i = 0; i < 8; ++i) {
        pr.p[i] = i < world ? peer_recv[i] : nullptr;
        pf.p[i] = i < world ? peer_flags[i] : nullptr;
    }
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (max_ctas < 1 || max_ctas > sms) max_ctas = sms;
    long long blocks = ((n >> 3) + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > max_ctas) blocks = max_ctas;
    allreduce_push_kernel<<<(int)blocks, 256, 0, st>>>((const uint4*)x, n >> 3, slot_elems >> 3, pr, pf, world, rank,
                                                       (const bf16*)residual, (bf16*)out, epoch_ptr, counters,
                                                       (unsigned long long)(limit_s * 1e9), status);
    return kb_launch_status();
}
