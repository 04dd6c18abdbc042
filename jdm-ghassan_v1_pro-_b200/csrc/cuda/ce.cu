// Softmax cross-entropy with z-loss on a chunk of 16-bit logits, gradient written in place.
//   loss_row = logZ - logit[target] + z * logZ^2          (rows with target < 0 are ignored)
//   dlogit   = (softmax * (1 + 2 z logZ) - onehot) * grad_scale      (sum-of-losses gradient, then loss scale)
// Same quantities as the reference's k_ce / k_sce_fold (cuda/kernels.cu:731-874), but the logits stay in
// 16 bits, the gradient replaces them (no second [rows, V] buffer) and the loss/count sums are folded on the
// device in a fixed order (no atomics, no host round trip per chunk).
#include "sm100_common.cuh"
#include "gb_api.h"

namespace gb {

template <typename T>
__global__ void __launch_bounds__(256) ce_row_kernel(T* __restrict__ logits, long long ld, const int* __restrict__ targets,
                                                     int V, float z, float grad_scale_val,
                                                     const float* __restrict__ grad_scale_dev, int write_grad,
                                                     float* __restrict__ row_loss) {
  __shared__ float red[8];
  __shared__ float bcast;
  const int row = blockIdx.x;
  T* lr = logits + (long long)row * ld;
  const int tgt = targets[row];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vec = V / 8;
  if (tgt < 0 || tgt >= V) {
    if (threadIdx.x == 0) row_loss[row] = -1.f;   // marker: not supervised
    if (write_grad) {
      for (int i = threadIdx.x; i < vec; i += 256) reinterpret_cast<uint4*>(lr)[i] = make_uint4(0, 0, 0, 0);
      for (int i = vec * 8 + threadIdx.x; i < V; i += 256) lr[i] = Cvt<T>::from_f(0.f);
    }
    return;
  }
  // pass 1: max
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vec; i += 256) {
    const uint4 q = reinterpret_cast<const uint4*>(lr)[i];
    const float2 a = Cvt<T>::unpack2(q.x), b = Cvt<T>::unpack2(q.y), c = Cvt<T>::unpack2(q.z), d = Cvt<T>::unpack2(q.w);
    mx = fmaxf(mx, fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y)), fmaxf(fmaxf(c.x, c.y), fmaxf(d.x, d.y))));
  }
  for (int i = vec * 8 + threadIdx.x; i < V; i += 256) mx = fmaxf(mx, Cvt<T>::to_f(lr[i]));
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    bcast = m;
  }
  __syncthreads();
  mx = bcast;
  // pass 2: sum of exp
  float sum = 0.f;
  for (int i = threadIdx.x; i < vec; i += 256) {
    const uint4 q = reinterpret_cast<const uint4*>(lr)[i];
    const float2 a = Cvt<T>::unpack2(q.x), b = Cvt<T>::unpack2(q.y), c = Cvt<T>::unpack2(q.z), d = Cvt<T>::unpack2(q.w);
    sum += __expf(a.x - mx) + __expf(a.y - mx) + __expf(b.x - mx) + __expf(b.y - mx) + __expf(c.x - mx) +
           __expf(c.y - mx) + __expf(d.x - mx) + __expf(d.y - mx);
  }
  for (int i = vec * 8 + threadIdx.x; i < V; i += 256) sum += __expf(Cvt<T>::to_f(lr[i]) - mx);
  sum = warp_sum(sum);
  __syncthreads();
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += red[i];
    bcast = s;
  }
  __syncthreads();
  sum = bcast;
  const float logz = mx + logf(sum);
  const float tl = Cvt<T>::to_f(lr[tgt]);
  __syncthreads();   // everyone has read the target logit before it is overwritten
  if (threadIdx.x == 0) row_loss[row] = logz - tl + z * logz * logz;
  if (!write_grad) return;
  const float grad_scale = grad_scale_dev ? grad_scale_dev[0] : grad_scale_val;
  const float coef = (1.f + 2.f * z * logz) / sum * grad_scale;
  for (int i = threadIdx.x; i < vec; i += 256) {
    const uint4 q = reinterpret_cast<const uint4*>(lr)[i];
    const float2 a = Cvt<T>::unpack2(q.x), b = Cvt<T>::unpack2(q.y), c = Cvt<T>::unpack2(q.z), d = Cvt<T>::unpack2(q.w);
    float g[8] = {__expf(a.x - mx) * coef, __expf(a.y - mx) * coef, __expf(b.x - mx) * coef, __expf(b.y - mx) * coef,
                  __expf(c.x - mx) * coef, __expf(c.y - mx) * coef, __expf(d.x - mx) * coef, __expf(d.y - mx) * coef};
    const int base = i * 8;
    if (tgt >= base && tgt < base + 8) g[tgt - base] -= grad_scale;
    uint4 o;
    o.x = Cvt<T>::pack2(g[0], g[1]); o.y = Cvt<T>::pack2(g[2], g[3]);
    o.z = Cvt<T>::pack2(g[4], g[5]); o.w = Cvt<T>::pack2(g[6], g[7]);
    reinterpret_cast<uint4*>(lr)[i] = o;
  }
  for (int i = vec * 8 + threadIdx.x; i < V; i += 256) {
    float g = __expf(Cvt<T>::to_f(lr[i]) - mx) * coef;
    if (i == tgt) g -= grad_scale;
    lr[i] = Cvt<T>::from_f(g);
  }
}

// acc[0] += sum of row losses, acc[1] += supervised rows; single block, fixed-order tree
__global__ void ce_fold_kernel(const float* __restrict__ row_loss, int rows, double* __restrict__ acc) {
  __shared__ double s_l[256];
  __shared__ double s_n[256];
  double l = 0.0, n = 0.0;
  for (int i = threadIdx.x; i < rows; i += 256) {
    const float v = row_loss[i];
    if (v >= 0.f || isnan(v)) { l += (double)v; n += 1.0; }
  }
  s_l[threadIdx.x] = l;
  s_n[threadIdx.x] = n;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) { s_l[threadIdx.x] += s_l[threadIdx.x + o]; s_n[threadIdx.x] += s_n[threadIdx.x + o]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { acc[0] += s_l[0]; acc[1] += s_n[0]; }
}

}  // namespace gb

using namespace gb;

// row_loss: scratch of `rows` floats.  The logits base and ld must keep rows 16-byte aligned.
extern "C" int gb_softmax_ce(void* logits, long long ld, const int* targets, int rows, int V, float z_loss,
                             float grad_scale, const float* grad_scale_dev, int write_grad, float* row_loss, double* acc,
                             int is_bf16,
                             cudaStream_t st) {
  if (rows <= 0 || V <= 0 || (ld * 2) % 16 || (reinterpret_cast<uintptr_t>(logits) & 15)) return -1;
  if (is_bf16)
    ce_row_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>((__nv_bfloat16*)logits, ld, targets, V, z_loss, grad_scale,
                                                       grad_scale_dev, write_grad, row_loss);
  else
    ce_row_kernel<__half><<<rows, 256, 0, st>>>((__half*)logits, ld, targets, V, z_loss, grad_scale, grad_scale_dev,
                                                write_grad, row_loss);
  ce_fold_kernel<<<1, 256, 0, st>>>(row_loss, rows, acc);
  return gb_launch_rc();
}
