// Flat-buffer optimizer kernels: one launch per (decay / no-decay) region instead of one per tensor, the
// gradient scale (unscale x clip, or 0 = "skip this step") read from device memory so that the inf/NaN
// decision never round-trips through the host, and the 16-bit shadow weights written in the same pass.
// Arithmetic per element is the reference's k_adamw / k_lion (cuda/kernels.cu:1021-1066, see also
// core/ops_cpu_dense.cpp:997-1030); the squared-norm reduction replaces one launch + D2H per tensor
// (cuda/kernels.cu:1068-1128) by a two-stage deterministic reduction over the flat gradient.
#include "sm100_common.cuh"
#include "gb_api.h"

namespace gb {

template <typename T, int KIND>
__global__ void __launch_bounds__(256) opt_step_kernel(float* __restrict__ w, const float* __restrict__ g,
                                                       float* __restrict__ m, float* __restrict__ v, T* __restrict__ w16,
                                                       long long n, const float* __restrict__ hyper,
                                                       const float* __restrict__ scale_dev, float beta1, float beta2,
                                                       float eps, float wd) {
  const float scale = scale_dev[0];
  if (scale == 0.f) return;   // rejected step: weights, moments and shadows stay as they are
  const float lr = hyper[0], bc1 = hyper[1], bc2 = hyper[2];
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (; i < n; i += stride) {
    float wv[4], gv[4], mv[4], vv[4];
    const int cnt = (int)min((long long)4, n - i);
    if (cnt == 4) {
      const float4 a = *reinterpret_cast<const float4*>(w + i), b = *reinterpret_cast<const float4*>(g + i),
                   c = *reinterpret_cast<const float4*>(m + i);
      wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w;
      gv[0] = b.x; gv[1] = b.y; gv[2] = b.z; gv[3] = b.w;
      mv[0] = c.x; mv[1] = c.y; mv[2] = c.z; mv[3] = c.w;
      if (KIND == 0) {
        const float4 d = *reinterpret_cast<const float4*>(v + i);
        vv[0] = d.x; vv[1] = d.y; vv[2] = d.z; vv[3] = d.w;
      }
    } else {
      for (int k = 0; k < cnt; ++k) { wv[k] = w[i + k]; gv[k] = g[i + k]; mv[k] = m[i + k]; if (KIND == 0) vv[k] = v[i + k]; }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (k >= cnt) break;
      const float gi = gv[k] * scale;
      if (KIND == 0) {
        const float mi = beta1 * mv[k] + (1.0f - beta1) * gi;
        const float vi = beta2 * vv[k] + (1.0f - beta2) * gi * gi;
        mv[k] = mi;
        vv[k] = vi;
        float upd = (mi / bc1) / (sqrtf(vi / bc2) + eps);
        if (wd != 0.0f) upd += wd * wv[k];
        wv[k] -= lr * upd;
      } else {
        const float c = beta1 * mv[k] + (1.0f - beta1) * gi;
        float upd = (c > 0.0f) ? 1.0f : ((c < 0.0f) ? -1.0f : 0.0f);
        if (wd != 0.0f) upd += wd * wv[k];
        wv[k] -= lr * upd;
        mv[k] = beta2 * mv[k] + (1.0f - beta2) * gi;
      }
    }
    if (cnt == 4) {
      *reinterpret_cast<float4*>(w + i) = make_float4(wv[0], wv[1], wv[2], wv[3]);
      *reinterpret_cast<float4*>(m + i) = make_float4(mv[0], mv[1], mv[2], mv[3]);
      if (KIND == 0) *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      if (w16) {
        uint2 q;
        q.x = Cvt<T>::pack2(wv[0], wv[1]);
        q.y = Cvt<T>::pack2(wv[2], wv[3]);
        *reinterpret_cast<uint2*>(w16 + i) = q;
      }
    } else {
      for (int k = 0; k < cnt; ++k) {
        w[i + k] = wv[k]; m[i + k] = mv[k];
        if (KIND == 0) v[i + k] = vv[k];
        if (w16) w16[i + k] = Cvt<T>::from_f(wv[k]);
      }
    }
  }
}

constexpr int SQ_THREADS = 256;
constexpr long long SQ_CHUNK = 1 << 16;   // elements per block

__global__ void __launch_bounds__(SQ_THREADS) sqnorm_partial_kernel(const float* __restrict__ g, long long n,
                                                                    double* __restrict__ partial) {
  __shared__ double s[SQ_THREADS];
  const long long lo = blockIdx.x * SQ_CHUNK, hi = min(n, lo + SQ_CHUNK);
  double acc = 0.0;
  for (long long i = lo + threadIdx.x * 4; i < hi; i += SQ_THREADS * 4) {
    if (i + 4 <= hi) {
      const float4 a = *reinterpret_cast<const float4*>(g + i);
      acc += (double)a.x * a.x + (double)a.y * a.y + (double)a.z * a.z + (double)a.w * a.w;
    } else {
      for (long long k = i; k < hi; ++k) acc += (double)g[k] * g[k];
    }
  }
  s[threadIdx.x] = acc;
  __syncthreads();
  for (int o = SQ_THREADS / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) s[threadIdx.x] += s[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[blockIdx.x] = s[0];
}

// out[0] = grad_scale * clip_factor, or 0 when the norm is not finite; out[1] = gnorm.
// extra_sq (optional): further squared-norm terms already reduced elsewhere (e.g. other ranks' shards).
__global__ void finish_norm_kernel(const double* __restrict__ partial, int n_partial, const float* __restrict__ gs_dev,
                                   float grad_scale, float clip, float* __restrict__ out) {
  __shared__ double s[256];
  double acc = 0.0;
  for (int i = threadIdx.x; i < n_partial; i += 256) acc += partial[i];
  s[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) s[threadIdx.x] += s[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float gs = gs_dev ? gs_dev[0] : grad_scale;
    const double gnorm = sqrt(s[0]) * (double)gs;
    float clip_scale = 1.0f;
    if (clip > 0.0f && gnorm > (double)clip) clip_scale = (float)((double)clip / (gnorm + 1e-6));
    const bool finite = isfinite(gnorm);
    out[0] = finite ? gs * clip_scale : 0.f;
    out[1] = (float)gnorm;
  }
}

__global__ void fill_f32_kernel(float* __restrict__ p, float v, long long n) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) p[i] = v;
}

}  // namespace gb

using namespace gb;

extern "C" int gb_optimizer_step(const gb_opt_args* a, cudaStream_t st) {
  if (!a || a->n < 0 || !a->w || !a->g || !a->m || !a->scale_dev || !a->hyper) return -1;
  if (a->kind == 0 && !a->v) return -1;
  if (a->n == 0) return 0;
  if ((reinterpret_cast<uintptr_t>(a->w) | reinterpret_cast<uintptr_t>(a->g) | reinterpret_cast<uintptr_t>(a->m)) & 15) return -2;
  long long blocks = (a->n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
#define GB_OPT(T, KIND)                                                                                              \
  opt_step_kernel<T, KIND><<<(int)blocks, 256, 0, st>>>(a->w, a->g, a->m, a->v, (T*)a->w16, a->n, a->hyper, a->scale_dev, \
                                                        a->beta1, a->beta2, a->eps, a->wd)
  if (a->is_bf16) { if (a->kind == 0) GB_OPT(__nv_bfloat16, 0); else GB_OPT(__nv_bfloat16, 1); }
  else { if (a->kind == 0) GB_OPT(__half, 0); else GB_OPT(__half, 1); }
#undef GB_OPT
  return gb_launch_rc();
}

extern "C" int gb_sqnorm_blocks(long long n) { return (int)((n + SQ_CHUNK - 1) / SQ_CHUNK); }

extern "C" int gb_sqnorm_partial(const float* g, long long n, double* partial, cudaStream_t st) {
  if (n <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(g) & 15) return -2;
  sqnorm_partial_kernel<<<gb_sqnorm_blocks(n), SQ_THREADS, 0, st>>>(g, n, partial);
  return gb_launch_rc();
}

extern "C" int gb_finish_norm(const double* partial, int n_partial, const float* grad_scale_dev, float grad_scale,
                              float clip, float* out, cudaStream_t st) {
  finish_norm_kernel<<<1, 256, 0, st>>>(partial, n_partial, grad_scale_dev, grad_scale, clip, out);
  return gb_launch_rc();
}

extern "C" int gb_fill_f32(float* p, float v, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  fill_f32_kernel<<<(int)blocks, 256, 0, st>>>(p, v, n);
  return gb_launch_rc();
}
