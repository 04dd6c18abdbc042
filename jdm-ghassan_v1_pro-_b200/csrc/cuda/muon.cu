// Elementwise halves of the Muon optimizer; the matrix products of its Newton-Schulz iteration run on the tcgen05
// GEMM (gemm_pair_sm100.cu / gemm_sm100.cu), driven from training/muon_cuda.py.
//
// The reference updates every 2-D decayed matrix W (R x C) by  m <- b1 m + (1 - b1) g,  O <- m / |m|_F,
// ns_steps x { A = O^T O ; O <- 1.5 O - 0.5 O A },  W <- (W - lr O) (1 - lr wd)   (training/optimizer.cpp:385-455).
// Here all matrices of one shape are stacked into one "class" buffer [n * Rp, C] (Rp = R rounded up to 256 rows, pad
// rows zero) so that one grouped GEMM serves all layers at once:
//     gram   A[g]  = Y16[g]^T Y16[g]                       grouped over the reduction dim, fp32 out
//     cast   B16   = bf16(-0.5 A)
//     step   Y     = T + Y16 B16[g]   with T = 1.5 Y       grouped over rows, fp32 out with addend
//     cast   Y16   = bf16(Y),  T = 1.5 Y
// The iterate Y, its 1.5-multiple T and the accumulation stay fp32; only the GEMM operands are bf16.
// Rows of a class live at arbitrary places of the flat parameter / gradient buffers (fused QKV rows, gate and up rows
// interleaved in blocks of 64): `row_src[r]` is the flat offset of class row r, or -1 for a pad row.
//
// Every kernel reads the step's scale (grad_scale * clip factor, 0 = rejected step) from device memory and returns at
// once when it is 0, so a rejected step leaves momentum and weights untouched without a host decision.
#include "sm100_common.cuh"
#include "gb_api.h"

namespace gb {

constexpr int MU_THREADS = 256;
constexpr int MU_ROWS = 8;          // class rows per block (one warp per row at a time)

// m <- b1 m + (1 - b1) scale g ; partial[block] = sum of m^2 over the block's rows (double)
__global__ void __launch_bounds__(MU_THREADS) muon_momentum_kernel(float* __restrict__ m, const float* __restrict__ g,
                                                                   const long long* __restrict__ row_src, long long rows,
                                                                   int C, float beta1, const float* __restrict__ scale_dev,
                                                                   double* __restrict__ partial) {
  __shared__ double red[MU_THREADS / 32];
  const float scale = scale_dev[0];
  if (scale == 0.f) return;
  const float c = (1.f - beta1) * scale;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * MU_ROWS + warp;
  double acc = 0.0;
  if (r < rows) {
    const long long src = row_src[r];
    if (src >= 0) {
      float* mr = m + r * C;
      const float* gr = g + src;
      for (int j = lane * 4; j < C; j += 128) {
        if (j + 4 <= C) {
          float4 mv = *reinterpret_cast<float4*>(mr + j);
          const float4 gv = *reinterpret_cast<const float4*>(gr + j);
          mv.x = beta1 * mv.x + c * gv.x; mv.y = beta1 * mv.y + c * gv.y;
          mv.z = beta1 * mv.z + c * gv.z; mv.w = beta1 * mv.w + c * gv.w;
          *reinterpret_cast<float4*>(mr + j) = mv;
          acc += (double)mv.x * mv.x + (double)mv.y * mv.y + (double)mv.z * mv.z + (double)mv.w * mv.w;
        } else {
          for (int k = j; k < C; ++k) {
            const float v = beta1 * mr[k] + c * gr[k];
            mr[k] = v;
            acc += (double)v * v;
          }
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int w = 0; w < MU_THREADS / 32; ++w) s += red[w];   // fixed order
    partial[blockIdx.x] = s;
  }
}

// Y = m / |m|_F of its matrix (|m|_F from the block partials, summed in block order), Y16 = bf16(Y), T = 1.5 Y.
// A matrix whose norm is not finite or below 1e-12 keeps Y = m and is flagged: its iteration is skipped (the reference
// returns the momentum itself in that case).
__global__ void __launch_bounds__(MU_THREADS) muon_normalize_kernel(const float* __restrict__ m, float* __restrict__ Y,
                                                                    float* __restrict__ T, __nv_bfloat16* __restrict__ Y16,
                                                                    const double* __restrict__ partial, int rows_per_mat,
                                                                    int C, const float* __restrict__ scale_dev,
                                                                    int* __restrict__ skip_flag) {
  __shared__ float s_inv;
  if (scale_dev[0] == 0.f) return;
  const int blocks_per_mat = rows_per_mat / MU_ROWS;
  const int mat = blockIdx.x / blocks_per_mat;
  if (threadIdx.x == 0) {
    double s = 0.0;
    const double* p = partial + (long long)mat * blocks_per_mat;
    for (int i = 0; i < blocks_per_mat; ++i) s += p[i];
    const double frob = sqrt(s);
    const bool bad = !isfinite(frob) || frob < 1e-12;
    s_inv = bad ? 1.f : (float)(1.0 / frob);
    if (blockIdx.x % blocks_per_mat == 0) skip_flag[mat] = bad ? 1 : 0;
  }
  __syncthreads();
  const float inv = s_inv;
  const long long base = (long long)blockIdx.x * MU_ROWS * C;
  const int n = MU_ROWS * C;
  for (int i = threadIdx.x * 4; i < n; i += MU_THREADS * 4) {
    if (i + 4 <= n) {
      const float4 v = *reinterpret_cast<const float4*>(m + base + i);
      const float4 y = make_float4(v.x * inv, v.y * inv, v.z * inv, v.w * inv);
      *reinterpret_cast<float4*>(Y + base + i) = y;
      *reinterpret_cast<float4*>(T + base + i) = make_float4(1.5f * y.x, 1.5f * y.y, 1.5f * y.z, 1.5f * y.w);
      __nv_bfloat162 a = __floats2bfloat162_rn(y.x, y.y), b = __floats2bfloat162_rn(y.z, y.w);
      uint2 q;
      q.x = *reinterpret_cast<uint32_t*>(&a);
      q.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(Y16 + base + i) = q;
    } else {
      for (int k = i; k < n; ++k) {
        const float y = m[base + k] * inv;
        Y[base + k] = y;
        T[base + k] = 1.5f * y;
        Y16[base + k] = __float2bfloat16_rn(y);
      }
    }
  }
}

// B16 = bf16(-0.5 A), n elements (all Gram matrices of a class)
__global__ void __launch_bounds__(MU_THREADS) muon_gram_cast_kernel(const float* __restrict__ A, __nv_bfloat16* __restrict__ B16,
                                                                    long long n, const float* __restrict__ scale_dev) {
  if (scale_dev[0] == 0.f) return;
  const long long stride = (long long)gridDim.x * MU_THREADS * 4;
  for (long long i = ((long long)blockIdx.x * MU_THREADS + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      const float4 v = *reinterpret_cast<const float4*>(A + i);
      __nv_bfloat162 a = __floats2bfloat162_rn(-0.5f * v.x, -0.5f * v.y), b = __floats2bfloat162_rn(-0.5f * v.z, -0.5f * v.w);
      uint2 q;
      q.x = *reinterpret_cast<uint32_t*>(&a);
      q.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(B16 + i) = q;
    } else {
      for (long long k = i; k < n; ++k) B16[k] = __float2bfloat16_rn(-0.5f * A[k]);
    }
  }
}

// After a step GEMM wrote Y = T + Y16 B16: refresh the operand copy and the addend of the next step.  A flagged matrix
// gets its pre-iteration Y back (Y = T / 1.5), i.e. stays at the momentum.
__global__ void __launch_bounds__(MU_THREADS) muon_refresh_kernel(float* __restrict__ Y, float* __restrict__ T,
                                                                  __nv_bfloat16* __restrict__ Y16, int rows_per_mat, int C,
                                                                  const float* __restrict__ scale_dev,
                                                                  const int* __restrict__ skip_flag) {
  if (scale_dev[0] == 0.f) return;
  const int blocks_per_mat = rows_per_mat / MU_ROWS;
  const bool skip = skip_flag[blockIdx.x / blocks_per_mat] != 0;
  const long long base = (long long)blockIdx.x * MU_ROWS * C;
  const int n = MU_ROWS * C;
  for (int i = threadIdx.x; i < n; i += MU_THREADS) {
    const float y = skip ? T[base + i] * (1.f / 1.5f) : Y[base + i];
    if (skip) Y[base + i] = y;
    T[base + i] = 1.5f * y;
    Y16[base + i] = __float2bfloat16_rn(y);
  }
}

// W <- (W - lr Y) (1 - lr wd) on the flat master weights, and the 16-bit shadow
template <typename T16>
__global__ void __launch_bounds__(MU_THREADS) muon_apply_kernel(float* __restrict__ w, T16* __restrict__ w16,
                                                                const float* __restrict__ Y,
                                                                const long long* __restrict__ row_src, long long rows, int C,
                                                                const float* __restrict__ lr_dev, float wd,
                                                                const float* __restrict__ scale_dev) {
  if (scale_dev[0] == 0.f) return;
  const float lr = lr_dev[0];
  const float keep = 1.f - lr * wd;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * MU_ROWS + warp;
  if (r >= rows) return;
  const long long src = row_src[r];
  if (src < 0) return;
  const float* yr = Y + r * C;
  float* wr = w + src;
  T16* hr = w16 ? w16 + src : nullptr;
  for (int j = lane; j < C; j += 32) {
    float v = wr[j] - lr * yr[j];
    if (wd != 0.f) v *= keep;
    wr[j] = v;
    if (hr) hr[j] = Cvt<T16>::from_f(v);
  }
}

}  // namespace gb

using namespace gb;

extern "C" int gb_muon_blocks(long long rows) { return (int)((rows + MU_ROWS - 1) / MU_ROWS); }

extern "C" int gb_muon_momentum(float* m, const float* g, const long long* row_src, long long rows, int C, float beta1,
                                const float* scale_dev, double* partial, cudaStream_t st) {
  if (!m || !g || !row_src || !scale_dev || !partial || rows <= 0 || C <= 0 || rows % MU_ROWS || C % 4) return -1;
  muon_momentum_kernel<<<(unsigned)(rows / MU_ROWS), MU_THREADS, 0, st>>>(m, g, row_src, rows, C, beta1, scale_dev, partial);
  return gb_launch_rc();
}

extern "C" int gb_muon_normalize(const float* m, float* Y, float* T, void* Y16, const double* partial, long long rows,
                                 int rows_per_mat, int C, const float* scale_dev, int* skip_flag, cudaStream_t st) {
  if (!m || !Y || !T || !Y16 || !partial || !scale_dev || !skip_flag || rows <= 0 || rows_per_mat <= 0 ||
      rows % rows_per_mat || rows_per_mat % MU_ROWS || C % 4)
    return -1;
  muon_normalize_kernel<<<(unsigned)(rows / MU_ROWS), MU_THREADS, 0, st>>>(m, Y, T, (__nv_bfloat16*)Y16, partial, rows_per_mat,
                                                                           C, scale_dev, skip_flag);
  return gb_launch_rc();
}

extern "C" int gb_muon_gram_cast(const float* A, void* B16, long long n, const float* scale_dev, cudaStream_t st) {
  if (!A || !B16 || !scale_dev || n <= 0) return -1;
  long long blocks = (n + MU_THREADS * 4 - 1) / (MU_THREADS * 4);
  if (blocks > 148 * 16) blocks = 148 * 16;
  muon_gram_cast_kernel<<<(unsigned)blocks, MU_THREADS, 0, st>>>(A, (__nv_bfloat16*)B16, n, scale_dev);
  return gb_launch_rc();
}

extern "C" int gb_muon_refresh(float* Y, float* T, void* Y16, long long rows, int rows_per_mat, int C, const float* scale_dev,
                               const int* skip_flag, cudaStream_t st) {
  if (!Y || !T || !Y16 || !scale_dev || !skip_flag || rows <= 0 || rows_per_mat <= 0 || rows % rows_per_mat ||
      rows_per_mat % MU_ROWS)
    return -1;
  muon_refresh_kernel<<<(unsigned)(rows / MU_ROWS), MU_THREADS, 0, st>>>(Y, T, (__nv_bfloat16*)Y16, rows_per_mat, C, scale_dev,
                                                                         skip_flag);
  return gb_launch_rc();
}

extern "C" int gb_muon_apply(float* w, void* w16, int is_bf16, const float* Y, const long long* row_src, long long rows, int C,
                             const float* lr_dev, float wd, const float* scale_dev, cudaStream_t st) {
  if (!w || !Y || !row_src || !lr_dev || !scale_dev || rows <= 0 || rows % MU_ROWS) return -1;
  const unsigned blocks = (unsigned)(rows / MU_ROWS);
  if (is_bf16) muon_apply_kernel<__nv_bfloat16><<<blocks, MU_THREADS, 0, st>>>(w, (__nv_bfloat16*)w16, Y, row_src, rows, C, lr_dev, wd, scale_dev);
  else muon_apply_kernel<__half><<<blocks, MU_THREADS, 0, st>>>(w, (__half*)w16, Y, row_src, rows, C, lr_dev, wd, scale_dev);
  return gb_launch_rc();
}
