// Gradient norm and clip factor without any allocation: see gb_noalloc.h for who calls this and why.
#include <stdint.h>

#include <atomic>

#include "gb_noalloc.h"

namespace {

constexpr int NA_THREADS = 256;
constexpr long long NA_CHUNK = 1 << 16;          // elements per block: the chunking of gb_sqnorm_partial
constexpr int NA_MAX_DEVICES = 64;

// The scratch: a 256-byte control block (arrival counter in its first word), then one double per chunk.
// 256 + 8 * 4096 = 33,024 bytes per device, part of the library image; nothing is ever allocated for it.
constexpr int NA_CTRL_BYTES = 256;
constexpr int NA_SCRATCH_BYTES = NA_CTRL_BYTES + 8 * GB_NOALLOC_MAX_CHUNKS;
static __device__ __align__(256) unsigned char g_scratch[NA_SCRATCH_BYTES];

__global__ void __launch_bounds__(NA_THREADS) grad_norm_static_kernel(const float* __restrict__ g, long long n,
                                                                       unsigned char* __restrict__ scratch, int n_chunks,
                                                                       float grad_scale, float clip,
                                                                       float* __restrict__ out) {
  __shared__ double s[NA_THREADS];
  __shared__ bool last;
  unsigned int* arrived = reinterpret_cast<unsigned int*>(scratch);
  double* partial = reinterpret_cast<double*>(scratch + NA_CTRL_BYTES);
  const long long lo = blockIdx.x * NA_CHUNK, hi = min(n, lo + NA_CHUNK);
  double acc = 0.0;
  for (long long i = lo + threadIdx.x * 4; i < hi; i += NA_THREADS * 4) {
    if (i + 4 <= hi) {
      const float4 a = *reinterpret_cast<const float4*>(g + i);
      acc += (double)a.x * a.x + (double)a.y * a.y + (double)a.z * a.z + (double)a.w * a.w;
    } else {
      for (long long k = i; k < hi; ++k) acc += (double)g[k] * g[k];
    }
  }
  s[threadIdx.x] = acc;
  __syncthreads();
  for (int o = NA_THREADS / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) s[threadIdx.x] += s[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    partial[blockIdx.x] = s[0];
    __threadfence();                                         // partial visible before the ticket
    last = atomicAdd(arrived, 1u) == (unsigned)(n_chunks - 1);
  }
  __syncthreads();
  if (!last) return;
  // The block that arrives last folds all partials in a fixed order (independent of which block that is).
  __threadfence();
  acc = 0.0;
  for (int i = threadIdx.x; i < n_chunks; i += NA_THREADS) acc += *((volatile double*)&partial[i]);
  s[threadIdx.x] = acc;
  __syncthreads();
  for (int o = NA_THREADS / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) s[threadIdx.x] += s[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const double gnorm = sqrt(s[0]) * (double)grad_scale;
    float clip_scale = 1.0f;
    if (clip > 0.0f && gnorm > (double)clip) clip_scale = (float)((double)clip / (gnorm + 1e-6));
    out[0] = isfinite(gnorm) ? grad_scale * clip_scale : 0.f;
    out[1] = (float)gnorm;
    *arrived = 0;                                         // ready for the next call
  }
}

__global__ void grad_norm_empty_kernel(float grad_scale, float* __restrict__ out) {
  out[0] = grad_scale;
  out[1] = 0.f;
}

// Address of each device's copy of the scratch, published with release/acquire ordering: a second host thread that
// makes its first call while another thread is inside the set-up either sees the finished pointer or resolves the
// (identical) address itself; it never sees a half-written cache.
std::atomic<unsigned char*> g_ptr[NA_MAX_DEVICES];
std::atomic<int> g_last_err{0};

// Resolve (once per device) where this device's copy of the scratch lives.
unsigned char* scratch_for_current_device() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= NA_MAX_DEVICES) {
    g_last_err.store(e != cudaSuccess ? (int)e : (int)cudaErrorInvalidDevice, std::memory_order_relaxed);
    return nullptr;
  }
  unsigned char* p = g_ptr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    e = cudaGetSymbolAddress((void**)&p, g_scratch);
    if (e != cudaSuccess || p == nullptr) {
      g_last_err.store((int)e, std::memory_order_relaxed);
      return nullptr;
    }
    g_ptr[dev].store(p, std::memory_order_release);
  }
  return p;
}

// Result of the launch just issued.  cudaPeekAtLastError leaves an earlier, unrelated sticky error for its owner
// to find; a failure is recorded so that gb_noalloc_last_cuda_error() names it.
int launch_result() {
  const cudaError_t e = cudaPeekAtLastError();
  if (e == cudaSuccess) return 0;
  g_last_err.store((int)e, std::memory_order_relaxed);
  return -11;
}

}  // namespace

extern "C" int gb_noalloc_last_cuda_error(void) { return g_last_err.load(std::memory_order_relaxed); }

extern "C" int gb_grad_norm_noalloc(const float* g, long long n, float grad_scale, float clip, float* out,
                                    cudaStream_t st) {
  if (out == nullptr || n < 0 || (g == nullptr && n > 0)) return -1;
  if (reinterpret_cast<uintptr_t>(g) & 15) return -2;
  if (n > GB_NOALLOC_MAX_ELEMS) return -3;       // beyond the static scratch: refuse rather than truncate
  if (n == 0) {                                  // needs no scratch at all
    grad_norm_empty_kernel<<<1, 1, 0, st>>>(grad_scale, out);
    return launch_result();
  }
  unsigned char* sc = scratch_for_current_device();
  if (sc == nullptr) return -4;
  const int n_chunks = (int)((n + NA_CHUNK - 1) / NA_CHUNK);
  // The arrival counter must be zero when the first block takes its ticket.  A kernel that was interrupted could have
  // left it non-zero, so it is cleared here on the same stream, ahead of the kernel.
  const cudaError_t me = cudaMemsetAsync(sc, 0, sizeof(unsigned int), st);
  if (me != cudaSuccess) {
    g_last_err.store((int)me, std::memory_order_relaxed);
    return -11;
  }
  grad_norm_static_kernel<<<n_chunks, NA_THREADS, 0, st>>>(g, n, sc, n_chunks, grad_scale, clip, out);
  return launch_result();
}
