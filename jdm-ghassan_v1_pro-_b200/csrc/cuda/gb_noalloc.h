// Entry points of _gb200_cuda.so that never allocate.  This header has no counterpart in the reference: the
// reference computes its gradient norm into buffers that its trainer allocates up front and offers no call for a
// host program that cannot allocate at all.
//
// Who needs this.  Every other entry point of the library takes its scratch buffers from the caller, and the
// Python layer gets them from PyTorch's caching allocator.  Some callers have no allocator to ask:
//   * a C or C++ host program (a monitoring or serving process) that links the kernel library alone, without
//     PyTorch, and wants the norm of a buffer that somebody else owns;
//   * a second host thread (a watchdog, a health check) that must stay out of the allocator the training thread is
//     using, because a cudaMalloc from that thread would serialise against all work on the device, and a call into
//     the caching allocator from a foreign thread and stream would hand out blocks whose reuse the training stream
//     knows nothing about;
//   * a diagnostics path that runs after an out-of-memory error, when asking for more memory is exactly what failed.
// For these the scratch lives in the library image itself: a file-scope device array of fixed size.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest input the static scratch covers: one double per 65536-element chunk, 4096 chunks (32 KiB of scratch plus a
// 256-byte control block), i.e. 268,435,456 floats (1 GiB of gradients).  Longer inputs are rejected, never truncated.
#define GB_NOALLOC_MAX_CHUNKS 4096
#define GB_NOALLOC_MAX_ELEMS (4096LL * 65536LL)

// out[0] = grad_scale * clip factor (0 when the norm is not finite), out[1] = ||g||_2 * grad_scale: the same two numbers
// gb_sqnorm_partial + gb_finish_norm produce, computed by ONE kernel whose per-chunk partial sums and arrival counter
// sit in the static scratch.  g: device, 16-byte aligned, n floats; out: device, 2 floats.
//
// Returns 0, or: -1 bad arguments (null pointer, n < 0), -2 misaligned g, -3 n larger than GB_NOALLOC_MAX_ELEMS,
// -4 the scratch symbol could not be resolved on the current device, -11 launch error (for -4 and -11 the CUDA error
// code is in gb_noalloc_last_cuda_error).  n == 0 writes {grad_scale, 0} and needs no scratch.
//
// Calls no cudaMalloc, cudaFree or any library routine that allocates.  The first call on each device resolves the
// scratch address with cudaGetSymbolAddress and caches it (the cache is atomic: host threads may make their first
// calls concurrently); make that first call during set-up, before any stream capture begins.  The arrival counter has to be zero when the kernel starts: every call clears it on `st` ahead of
// the kernel, and the last block clears it again on the way out.
//
// The scratch is one per device and is not locked: two calls that overlap in time on the same device (different
// streams or threads) race on it and both results are garbage.  Serialise such calls on one stream.
int gb_grad_norm_noalloc(const float* g, long long n, float grad_scale, float clip, float* out, cudaStream_t st);

// CUDA error code of the last failed set-up or launch of this entry point (0 = none).
int gb_noalloc_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
