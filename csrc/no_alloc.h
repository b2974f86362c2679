// Allocation-free entry point (no counterpart in the reference project).
//
// Who needs it: code that drives the paged decode attention from a context where device
// allocation is not available to it -- a C/C++ host that links this library without PyTorch's
// caching allocator, a serving loop whose memory budget was fixed at start-up and must not grow,
// or a caller that is inside a region where cudaMalloc would serialise or fail.  The regular
// entry point (kb_paged_decode) needs two caller-allocated workspaces for its split-KV partial
// results; this variant keeps that workspace in a fixed array inside the library instead.
//
//   int kb_paged_decode_noalloc(q, q_stride, k_pages, v_pages, page_table, max_pages, ctx_lens,
//                               B, n_q, n_kv, hd, max_ctx, split_tokens, scale, out, out_stride, stream)
//
// Same arguments and result as kb_paged_decode minus the two workspace pointers.  The caller
// still owns every input and output buffer.  The call itself performs no cudaMalloc, cudaFree or
// any other allocating call.
//
// Limit: the partial results need  B * n_q * ceil(max_ctx / split_tokens) * (hd + 2)  floats and
// the built-in array holds KB_NOALLOC_SCRATCH_FLOATS of them (8 MiB; every GPU that loads the
// library keeps that much device memory until the process exits).  A larger request is refused:
// the function prints the required and available sizes to stderr and returns
// KB_NOALLOC_TOO_LARGE without launching anything.
//
// Set-up: the first call on each device (with that device current) looks up the array's device
// address once and caches it.  Make that first call outside of any stream capture.
//
// Sharing: all calls on a device use the one array, which keeps whatever the previous call left
// in it.  Nothing in it has to start at zero (every slot that is read is written earlier in the
// same call), but two calls that overlap on the GPU -- different streams, or concurrent host
// threads -- race on it; serialise them.
#pragma once
#include <cuda_runtime.h>

#define KB_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define KB_NOALLOC_TOO_LARGE 40
#define KB_NOALLOC_SETUP_FAILED 41

#ifdef __cplusplus
extern "C" {
#endif
int kb_paged_decode_noalloc(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                            const int* page_table, int max_pages, const int* ctx_lens, int B, int n_q, int n_kv,
                            int hd, int max_ctx, int split_tokens, float scale, void* out, long long out_stride,
                            cudaStream_t stream);
#ifdef __cplusplus
}
#endif
