// Memory-bound model kernels: embedding gather/scatter, RMSNorm forward/backward (with the residual
// stream kept in fp32 and 16-bit GEMM operands produced in the same pass), QK-norm + RoPE forward/backward.
// They replace k_embed_*, k_rmsnorm_*, k_rope_freq, k_split_qkv and the add/copy kernels of the reference
// (cuda/kernels.cu:327-692): the split of the fused QKV output, the per-head norm and the rotation are one
// pass, residual adds live in GEMM epilogues, and weight-gradient column sums are two-stage and deterministic.
#include "sm100_common.cuh"
#include "gb_api.h"

namespace gb {

template <typename T> struct Vec8 { uint4 v; };

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  float2 a = Cvt<T>::unpack2(q.x), b = Cvt<T>::unpack2(q.y), c = Cvt<T>::unpack2(q.z), d = Cvt<T>::unpack2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  uint4 q;
  q.x = Cvt<T>::pack2(f[0], f[1]); q.y = Cvt<T>::pack2(f[2], f[3]);
  q.z = Cvt<T>::pack2(f[4], f[5]); q.w = Cvt<T>::pack2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = q;
}

// ------------------------------------------------------------------------------------------ embedding
__global__ void embed_fwd_kernel(const int* __restrict__ ids, const float* __restrict__ table, float* __restrict__ out,
                                 int n_tok, int d, int vocab) {
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_tok) return;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const float4* src = reinterpret_cast<const float4*>(table + (size_t)id * d);
  float4* dst = reinterpret_cast<float4*>(out + (size_t)t * d);
  for (int i = threadIdx.x; i < d / 4; i += blockDim.x) dst[i] = src[i];
}

// dtable[id] += sum over the tokens t with ids[t] == id of dx[t], added in increasing t: no atomics on the sums, so
// the embedding gradient is the same bits on every run (the reference scatters with atomicAdd,
// cuda/kernels.cu:420-442, and is not).  A first pass records the first token of every id (atomicMin on an index:
// order-independent).  Then one block per token: the block of the FIRST occurrence owns that id's row and walks the
// later tokens, 1024 ids per trip (four per thread, ballots into shared memory), adding the matches in index order;
// every other block leaves at once.
constexpr int EMB_THREADS = 256;
constexpr int EMB_MAX_COLS = 32;           // columns per thread: d <= 8192
constexpr int EMB_MAX_VOCAB = 1 << 19;     // ids covered by the first-occurrence table (2 MB of device memory)
__device__ int g_emb_first[EMB_MAX_VOCAB];

__global__ void embed_first_kernel(const int* __restrict__ ids, int n_tok, int vocab) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tok) return;
  const int id = ids[t];
  if (id >= 0 && id < vocab) atomicMin(&g_emb_first[id], t);
}

__global__ void __launch_bounds__(EMB_THREADS) embed_bwd_kernel(const int* __restrict__ ids, const float* __restrict__ dx,
                                                               float* __restrict__ dtable, int n_tok, int d, int vocab) {
  __shared__ unsigned int mask[4][EMB_THREADS / 32];
  const int t = blockIdx.x;
  if (t >= n_tok) return;
  const int id = ids[t];
  if (id < 0 || id >= vocab) return;
  if (g_emb_first[id] != t) return;              // an earlier token owns this id
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float acc[EMB_MAX_COLS];
  const int ncol = (d + EMB_THREADS - 1) / EMB_THREADS;
#pragma unroll
  for (int c = 0; c < EMB_MAX_COLS; ++c) acc[c] = 0.f;
  constexpr int TRIP = 4 * EMB_THREADS;
  for (int base = t - (t % TRIP); base < n_tok; base += TRIP) {
    // thread i looks at ids base + k*256 + i for k = 0..3, so that mask[k] is in index order
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int j = base + k * EMB_THREADS + threadIdx.x;
      const bool hit = j >= t && j < n_tok && ids[j] == id;
      const unsigned int b = __ballot_sync(0xffffffffu, hit);
      if (lane == 0) mask[k][warp] = b;
    }
    __syncthreads();
#pragma unroll 1
    for (int k = 0; k < 4; ++k)
      for (int w = 0; w < EMB_THREADS / 32; ++w) {
        unsigned int m = mask[k][w];
        while (m) {
          const int bit = __ffs(m) - 1;
          m &= m - 1;
          const float* src = dx + (size_t)(base + k * EMB_THREADS + w * 32 + bit) * d;
#pragma unroll
          for (int c = 0; c < EMB_MAX_COLS; ++c)
            if (c < ncol) {
              const int col = c * EMB_THREADS + threadIdx.x;
              if (col < d) acc[c] += src[col];
            }
        }
      }
    __syncthreads();
  }
  float* dst = dtable + (size_t)id * d;
#pragma unroll
  for (int c = 0; c < EMB_MAX_COLS; ++c)
    if (c < ncol) {
      const int col = c * EMB_THREADS + threadIdx.x;
      if (col < d) dst[col] += acc[c];
    }
}

__global__ void __launch_bounds__(EMB_THREADS) embed_bwd_sorted_kernel(const int* __restrict__ sid,
                                                                      const long long* __restrict__ order,
                                                                      const float* __restrict__ dx, float* __restrict__ dtable,
                                                                      int n_tok, int d, int vocab) {
  const int p = blockIdx.x;
  if (p >= n_tok) return;
  const int id = sid[p];
  if (id < 0 || id >= vocab) return;
  if (p > 0 && sid[p - 1] == id) return;          // not the first position of this id's run
  float acc[EMB_MAX_COLS];
  const int ncol = (d + EMB_THREADS - 1) / EMB_THREADS;
#pragma unroll
  for (int c = 0; c < EMB_MAX_COLS; ++c) acc[c] = 0.f;
  long long tok = order[p];
  for (int q = p; q < n_tok; ++q) {
    const bool more = q + 1 < n_tok && sid[q + 1] == id;
    const long long next_tok = more ? order[q + 1] : 0;   // fetched while this row is added
    if (tok >= 0 && tok < n_tok) {
      const float* src = dx + (size_t)tok * d;
#pragma unroll
      for (int c = 0; c < EMB_MAX_COLS; ++c)
        if (c < ncol) {
          const int col = c * EMB_THREADS + threadIdx.x;
          if (col < d) acc[c] += src[col];
        }
    }
    if (!more) break;
    tok = next_tok;
  }
  float* dst = dtable + (size_t)id * d;
#pragma unroll
  for (int c = 0; c < EMB_MAX_COLS; ++c)
    if (c < ncol) {
      const int col = c * EMB_THREADS + threadIdx.x;
      if (col < d) dst[col] += acc[c];
    }
}

// ------------------------------------------------------------------------------------------ RMSNorm
// One warp per row.  y16 = x * inv * w (16-bit), rrms[row] = inv;  inv = 0 when it is not finite.
template <typename T>
__global__ void rmsnorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                                   float* __restrict__ rrms, int rows, int d, float eps) {
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * d);
  float ss = 0.f;
  for (int i = lane; i < d / 4; i += 32) {
    float4 v = xr[i];
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = warp_sum(ss);
  float inv = rsqrtf(ss / (float)d + eps);
  if (!isfinite(inv)) inv = 0.f;
  if (lane == 0 && rrms) rrms[row] = inv;
  const float4* wr = reinterpret_cast<const float4*>(w);
  T* yr = y + (size_t)row * d;
  for (int i = lane; i < d / 4; i += 32) {
    float4 v = xr[i], g = wr[i];
    uint2 o;
    o.x = Cvt<T>::pack2(v.x * inv * g.x, v.y * inv * g.y);
    o.y = Cvt<T>::pack2(v.z * inv * g.z, v.w * inv * g.w);
    *reinterpret_cast<uint2*>(yr + 4 * i) = o;
  }
}

// dx_out = dres + g*w*inv - x*inv^3/d * sum(g*w*x);  optional 16-bit copy of dx_out.
// Also writes this block's column partials of dw (sum over its rows of g*x*inv) to part[blockIdx.x, :].
template <typename T>
__global__ void rmsnorm_bwd_kernel(const T* __restrict__ g, const float* __restrict__ x, const float* __restrict__ w,
                                   const float* __restrict__ rrms, const float* __restrict__ dres,
                                   float* __restrict__ dx_out, T* __restrict__ dx16, float* __restrict__ part,
                                   int rows, int d, int rows_per_block) {
  extern __shared__ float sm_dw_all[];  // [nwarps][d]: every warp sums its own rows, lanes own distinct columns
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < d * nwarps; i += blockDim.x) sm_dw_all[i] = 0.f;
  __syncthreads();
  float* sm_dw = sm_dw_all + (size_t)warp * d;
  const int row0 = blockIdx.x * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  for (int row = row0 + warp; row < row1; row += nwarps) {
    const float inv = rrms[row];
    const float* xr = x + (size_t)row * d;
    const T* gr = g + (size_t)row * d;
    float dot = 0.f;
    for (int i = lane * 4; i < d; i += 128) {
      float4 xv = *reinterpret_cast<const float4*>(xr + i);
      float4 wv = *reinterpret_cast<const float4*>(w + i);
      uint2 gq = *reinterpret_cast<const uint2*>(gr + i);
      float2 g01 = Cvt<T>::unpack2(gq.x), g23 = Cvt<T>::unpack2(gq.y);
      dot += g01.x * wv.x * xv.x + g01.y * wv.y * xv.y + g23.x * wv.z * xv.z + g23.y * wv.w * xv.w;
    }
    dot = warp_sum(dot);
    const float coef = inv * inv * inv * dot / (float)d;
    for (int i = lane * 4; i < d; i += 128) {
      float4 xv = *reinterpret_cast<const float4*>(xr + i);
      float4 wv = *reinterpret_cast<const float4*>(w + i);
      uint2 gq = *reinterpret_cast<const uint2*>(gr + i);
      float2 g01 = Cvt<T>::unpack2(gq.x), g23 = Cvt<T>::unpack2(gq.y);
      float4 r = dres ? *reinterpret_cast<const float4*>(dres + (size_t)row * d + i) : make_float4(0, 0, 0, 0);
      float4 o;
      o.x = r.x + g01.x * wv.x * inv - xv.x * coef;
      o.y = r.y + g01.y * wv.y * inv - xv.y * coef;
      o.z = r.z + g23.x * wv.z * inv - xv.z * coef;
      o.w = r.w + g23.y * wv.w * inv - xv.w * coef;
      *reinterpret_cast<float4*>(dx_out + (size_t)row * d + i) = o;
      if (dx16) {
        uint2 q;
        q.x = Cvt<T>::pack2(o.x, o.y);
        q.y = Cvt<T>::pack2(o.z, o.w);
        *reinterpret_cast<uint2*>(dx16 + (size_t)row * d + i) = q;
      }
      sm_dw[i + 0] += g01.x * xv.x * inv;
      sm_dw[i + 1] += g01.y * xv.y * inv;
      sm_dw[i + 2] += g23.x * xv.z * inv;
      sm_dw[i + 3] += g23.y * xv.w * inv;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float s = 0.f;
    for (int wv = 0; wv < nwarps; ++wv) s += sm_dw_all[(size_t)wv * d + i];
    part[(size_t)blockIdx.x * d + i] = s;
  }
}

// The same for d = 128 * NV with a whole row in registers: every load of a row (x, g, dres) is issued before the
// first use and the row is read once.  The rolled loop above waits for DRAM twelve times per row and ran at about
// half of the copy bandwidth.  The column sums of dw live in the warp's own slice of shared memory (lanes own
// distinct columns), not in registers: that keeps the kernel at 64 registers and four blocks of 8 warps per SM,
// and the number of rows in flight is what this kernel's speed depends on.
template <typename T, int NV>
__global__ void __launch_bounds__(256, 4) rmsnorm_bwd_vec_kernel(const T* __restrict__ g, const float* __restrict__ x,
                                                              const float* __restrict__ w, const float* __restrict__ rrms,
                                                              const float* __restrict__ dres, float* __restrict__ dx_out,
                                                              T* __restrict__ dx16, float* __restrict__ part, int rows,
                                                              int rows_per_block) {
  constexpr int D = NV * 128;
  extern __shared__ float sm_dw_all[];  // [8][D] column sums of the warps, then [D] weights
  float* s_w = sm_dw_all + 8 * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < D; i += blockDim.x) s_w[i] = w[i];
  float* s_acc = sm_dw_all + (size_t)warp * D + lane * 4;
#pragma unroll
  for (int k = 0; k < NV; ++k) *reinterpret_cast<float4*>(s_acc + k * 128) = make_float4(0.f, 0.f, 0.f, 0.f);
  __syncthreads();
  const int row0 = blockIdx.x * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  for (int row = row0 + warp; row < row1; row += 8) {
    const float inv = rrms[row];
    const float* xr = x + (size_t)row * D;
    const T* gr = g + (size_t)row * D;
    float4 xv[NV];
    uint2 gq[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = k * 128 + lane * 4;
      xv[k] = *reinterpret_cast<const float4*>(xr + i);
      gq[k] = *reinterpret_cast<const uint2*>(gr + i);
    }
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const float4 wv = *reinterpret_cast<const float4*>(s_w + k * 128 + lane * 4);
      const float2 g01 = Cvt<T>::unpack2(gq[k].x), g23 = Cvt<T>::unpack2(gq[k].y);
      dot += g01.x * wv.x * xv[k].x + g01.y * wv.y * xv[k].y + g23.x * wv.z * xv[k].z + g23.y * wv.w * xv[k].w;
    }
    dot = warp_sum(dot);
    const float coef = inv * inv * inv * dot / (float)D;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = k * 128 + lane * 4;
      const float4 wv = *reinterpret_cast<const float4*>(s_w + i);
      const float2 g01 = Cvt<T>::unpack2(gq[k].x), g23 = Cvt<T>::unpack2(gq[k].y);
      const float4 rv = dres ? __ldcs(reinterpret_cast<const float4*>(dres + (size_t)row * D + i)) : make_float4(0, 0, 0, 0);
      float4 o;
      o.x = rv.x + g01.x * wv.x * inv - xv[k].x * coef;
      o.y = rv.y + g01.y * wv.y * inv - xv[k].y * coef;
      o.z = rv.z + g23.x * wv.z * inv - xv[k].z * coef;
      o.w = rv.w + g23.y * wv.w * inv - xv[k].w * coef;
      *reinterpret_cast<float4*>(dx_out + (size_t)row * D + i) = o;
      if (dx16) {
        uint2 q;
        q.x = Cvt<T>::pack2(o.x, o.y);
        q.y = Cvt<T>::pack2(o.z, o.w);
        *reinterpret_cast<uint2*>(dx16 + (size_t)row * D + i) = q;
      }
      float4 a = *reinterpret_cast<float4*>(s_acc + k * 128);
      a.x += g01.x * xv[k].x * inv;
      a.y += g01.y * xv[k].y * inv;
      a.z += g23.x * xv[k].z * inv;
      a.w += g23.y * xv[k].w * inv;
      *reinterpret_cast<float4*>(s_acc + k * 128) = a;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < 8; ++wv) s += sm_dw_all[(size_t)wv * D + i];
    part[(size_t)blockIdx.x * D + i] = s;
  }
}

// dw[c] += sum_b part[b, c]
// 256 threads = 32 columns x 8 row lanes; fixed summation order (row lane, then lanes 0..7)
__global__ void colsum_finalize_kernel(const float* __restrict__ part, float* __restrict__ dw, int nblocks, int d) {
  __shared__ float s_part[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < d)
    for (int b = ty; b < nblocks; b += 8) s += part[(size_t)b * d + c];
  s_part[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < d) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += s_part[k][tx];
    dw[c] += t;
  }
}

// ------------------------------------------------------------------------------------------ QK-norm + RoPE
// qkv: [N, ld_in] fused GEMM output (q heads, then k heads, then v heads).  One warp per (token, head) for the
// q and k heads: optional RMSNorm over head_dim with a shared [hd] weight, then rotation by the cached
// cos/sin of the row position.  rope_type 0 rotates (2i, 2i+1), 1 rotates (i, i + hd/2).
template <typename T, int HD>
__global__ void qk_norm_rope_fwd_kernel(const T* __restrict__ qkv, int ld_in, T* __restrict__ out, int ld_out,
                                        const float* __restrict__ qw, const float* __restrict__ kw,
                                        const float* __restrict__ cs, const int* __restrict__ pos, int n_tok, int H,
                                        int KV, float eps, int rope_type) {
  pdl_wait();
  constexpr int PAIRS = HD / 2;
  constexpr int PPL = (PAIRS + 31) / 32;  // pairs per lane
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = H + KV;
  if (gw >= n_tok * heads) return;
  const int t = gw / heads, h = gw - t * heads;
  const T* src = qkv + (size_t)t * ld_in + (size_t)h * HD;
  T* dst = out + (size_t)t * ld_out + (size_t)h * HD;
  const float* w = (h < H) ? qw : kw;
  float a[PPL], b[PPL];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PPL; ++k) {
    const int p = lane + 32 * k;
    if (p < PAIRS) {
      const int i0 = rope_type == 0 ? 2 * p : p, i1 = rope_type == 0 ? 2 * p + 1 : p + PAIRS;
      a[k] = Cvt<T>::to_f(src[i0]);
      b[k] = Cvt<T>::to_f(src[i1]);
      ss += a[k] * a[k] + b[k] * b[k];
    }
  }
  float inv = 1.f;
  if (w) {
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)HD + eps);
    if (!isfinite(inv)) inv = 0.f;
  }
  const float* csr = cs + (size_t)pos[t] * HD;  // [pos][PAIRS cos | PAIRS sin]
#pragma unroll
  for (int k = 0; k < PPL; ++k) {
    const int p = lane + 32 * k;
    if (p < PAIRS) {
      const int i0 = rope_type == 0 ? 2 * p : p, i1 = rope_type == 0 ? 2 * p + 1 : p + PAIRS;
      float x0 = a[k], x1 = b[k];
      if (w) { x0 *= inv * w[i0]; x1 *= inv * w[i1]; }
      const float c = csr[p], s = csr[PAIRS + p];
      dst[i0] = Cvt<T>::from_f(x0 * c - x1 * s);
      dst[i1] = Cvt<T>::from_f(x0 * s + x1 * c);
    }
  }
}

// Backward: dq_r/dk_r (grads after rotation) -> grads of the raw projections, written into dqkv (q and k parts).
// Per-block partials of the norm-weight grads go to part_q / part_k ([gridDim.x, HD]).
template <typename T, int HD>
__global__ void qk_norm_rope_bwd_kernel(const T* __restrict__ dout, int ld_dout, const T* __restrict__ qkv, int ld_in,
                                        T* __restrict__ dqkv, int ld_dqkv, const float* __restrict__ qw,
                                        const float* __restrict__ kw, const float* __restrict__ cs,
                                        const int* __restrict__ pos, float* __restrict__ part_q,
                                        float* __restrict__ part_k, int n_tok, int H, int KV, float eps, int rope_type,
                                        int items_per_block) {
  constexpr int PAIRS = HD / 2;
  constexpr int PPL = (PAIRS + 31) / 32;
  __shared__ float s_dwq_all[8][HD], s_dwk_all[8][HD];  // launched with 8 warps; each warp sums its own items
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < 8 * HD; i += blockDim.x) { (&s_dwq_all[0][0])[i] = 0.f; (&s_dwk_all[0][0])[i] = 0.f; }
  __syncthreads();
  float* s_dwq = s_dwq_all[warp];
  float* s_dwk = s_dwk_all[warp];
  const int heads = H + KV;
  const int total = n_tok * heads;
  const int it0 = blockIdx.x * items_per_block, it1 = min(total, it0 + items_per_block);
  for (int item = it0 + warp; item < it1; item += nwarps) {
    const int t = item / heads, h = item - t * heads;
    const T* gsrc = dout + (size_t)t * ld_dout + (size_t)h * HD;
    const T* raw = qkv + (size_t)t * ld_in + (size_t)h * HD;
    T* dst = dqkv + (size_t)t * ld_dqkv + (size_t)h * HD;
    const float* w = (h < H) ? qw : kw;
    float* sdw = (h < H) ? s_dwq : s_dwk;
    const float* csr = cs + (size_t)pos[t] * HD;
    float g0[PPL], g1[PPL], x0[PPL], x1[PPL];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int k = 0; k < PPL; ++k) {
      const int p = lane + 32 * k;
      if (p < PAIRS) {
        const int i0 = rope_type == 0 ? 2 * p : p, i1 = rope_type == 0 ? 2 * p + 1 : p + PAIRS;
        const float c = csr[p], s = csr[PAIRS + p];
        const float d0 = Cvt<T>::to_f(gsrc[i0]), d1 = Cvt<T>::to_f(gsrc[i1]);
        g0[k] = d0 * c + d1 * s;    // inverse rotation
        g1[k] = -d0 * s + d1 * c;
        if (w) {
          x0[k] = Cvt<T>::to_f(raw[i0]);
          x1[k] = Cvt<T>::to_f(raw[i1]);
          ss += x0[k] * x0[k] + x1[k] * x1[k];
          dot += g0[k] * w[i0] * x0[k] + g1[k] * w[i1] * x1[k];
        }
      }
    }
    if (!w) {
#pragma unroll
      for (int k = 0; k < PPL; ++k) {
        const int p = lane + 32 * k;
        if (p < PAIRS) {
          const int i0 = rope_type == 0 ? 2 * p : p, i1 = rope_type == 0 ? 2 * p + 1 : p + PAIRS;
          dst[i0] = Cvt<T>::from_f(g0[k]);
          dst[i1] = Cvt<T>::from_f(g1[k]);
        }
      }
      continue;
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    float inv = rsqrtf(ss / (float)HD + eps);
    if (!isfinite(inv)) inv = 0.f;
    const float coef = inv * inv * inv * dot / (float)HD;
#pragma unroll
    for (int k = 0; k < PPL; ++k) {
      const int p = lane + 32 * k;
      if (p < PAIRS) {
        const int i0 = rope_type == 0 ? 2 * p : p, i1 = rope_type == 0 ? 2 * p + 1 : p + PAIRS;
        dst[i0] = Cvt<T>::from_f(g0[k] * w[i0] * inv - x0[k] * coef);
        dst[i1] = Cvt<T>::from_f(g1[k] * w[i1] * inv - x1[k] * coef);
        sdw[i0] += g0[k] * x0[k] * inv;
        sdw[i1] += g1[k] * x1[k] * inv;
      }
    }
  }
  __syncthreads();
  if (part_q)
    for (int i = threadIdx.x; i < HD; i += blockDim.x) {
      float sq = 0.f, sk = 0.f;
      for (int wv = 0; wv < nwarps; ++wv) { sq += s_dwq_all[wv][i]; sk += s_dwk_all[wv][i]; }
      part_q[(size_t)blockIdx.x * HD + i] = sq;
      part_k[(size_t)blockIdx.x * HD + i] = sk;
    }
}

// The same backward with HD/8 lanes per (token, head) item: a lane owns four rotation pairs and moves them with
// 16-byte (interleaved pairs) or 8-byte (half-split pairs) accesses, a warp works on 256/HD items at once and on
// two such groups per trip, so that enough bytes are in flight to cover the DRAM latency (with one item per warp
// the kernel ran at a fifth of the copy bandwidth).  Needs 16-byte aligned rows; HD in {32, 64, 128, 256}.
template <typename T>
__device__ __forceinline__ void qk_load8(const T* p, int j, int pairs, int rope_type, float (&a)[4], float (&b)[4]) {
  if (rope_type == 0) {
    const uint4 v = *reinterpret_cast<const uint4*>(p + 8 * j);
    const float2 e0 = Cvt<T>::unpack2(v.x), e1 = Cvt<T>::unpack2(v.y), e2 = Cvt<T>::unpack2(v.z), e3 = Cvt<T>::unpack2(v.w);
    a[0] = e0.x; b[0] = e0.y; a[1] = e1.x; b[1] = e1.y; a[2] = e2.x; b[2] = e2.y; a[3] = e3.x; b[3] = e3.y;
  } else {
    const uint2 lo = *reinterpret_cast<const uint2*>(p + 4 * j);
    const uint2 hi = *reinterpret_cast<const uint2*>(p + pairs + 4 * j);
    const float2 l0 = Cvt<T>::unpack2(lo.x), l1 = Cvt<T>::unpack2(lo.y), h0 = Cvt<T>::unpack2(hi.x), h1 = Cvt<T>::unpack2(hi.y);
    a[0] = l0.x; a[1] = l0.y; a[2] = l1.x; a[3] = l1.y; b[0] = h0.x; b[1] = h0.y; b[2] = h1.x; b[3] = h1.y;
  }
}
template <typename T>
__device__ __forceinline__ void qk_store8(T* p, int j, int pairs, int rope_type, const float (&a)[4], const float (&b)[4]) {
  if (rope_type == 0) {
    uint4 v;
    v.x = Cvt<T>::pack2(a[0], b[0]); v.y = Cvt<T>::pack2(a[1], b[1]);
    v.z = Cvt<T>::pack2(a[2], b[2]); v.w = Cvt<T>::pack2(a[3], b[3]);
    *reinterpret_cast<uint4*>(p + 8 * j) = v;
  } else {
    uint2 lo, hi;
    lo.x = Cvt<T>::pack2(a[0], a[1]); lo.y = Cvt<T>::pack2(a[2], a[3]);
    hi.x = Cvt<T>::pack2(b[0], b[1]); hi.y = Cvt<T>::pack2(b[2], b[3]);
    *reinterpret_cast<uint2*>(p + 4 * j) = lo;
    *reinterpret_cast<uint2*>(p + pairs + 4 * j) = hi;
  }
}
// fp32 vector of the four first / second pair members a lane owns (weights)
__device__ __forceinline__ void qk_loadw(const float* w, int j, int pairs, int rope_type, float (&a)[4], float (&b)[4]) {
  if (rope_type == 0) {
    const float4 u = *reinterpret_cast<const float4*>(w + 8 * j), v = *reinterpret_cast<const float4*>(w + 8 * j + 4);
    a[0] = u.x; b[0] = u.y; a[1] = u.z; b[1] = u.w; a[2] = v.x; b[2] = v.y; a[3] = v.z; b[3] = v.w;
  } else {
    const float4 u = *reinterpret_cast<const float4*>(w + 4 * j), v = *reinterpret_cast<const float4*>(w + pairs + 4 * j);
    a[0] = u.x; a[1] = u.y; a[2] = u.z; a[3] = u.w; b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w;
  }
}

// Forward with the same lane layout: HD/8 lanes per (token, head) item, 256/HD items per warp.
template <typename T, int HD>
__global__ void __launch_bounds__(256) qk_norm_rope_fwd_vec_kernel(
    const T* __restrict__ qkv, int ld_in, T* __restrict__ out, int ld_out, const float* __restrict__ qw,
    const float* __restrict__ kw, const float* __restrict__ cs, const int* __restrict__ pos, int n_tok, int H, int KV,
    float eps, int rope_type) {
  pdl_wait();
  constexpr int PAIRS = HD / 2, LPI = HD / 8, IPW = 32 / LPI;
  const int lane = threadIdx.x & 31, sub = lane / LPI, j = lane % LPI;
  const int heads = H + KV;
  const int item = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * IPW + sub;
  const bool live = item < n_tok * heads;
  const int t = live ? item / heads : 0, h = live ? item - t * heads : 0;
  float a[4] = {0, 0, 0, 0}, b[4] = {0, 0, 0, 0};
  float4 c = make_float4(1, 1, 1, 1), s = make_float4(0, 0, 0, 0);
  if (live) {
    const float* csr = cs + (size_t)pos[t] * HD;
    qk_load8<T>(qkv + (size_t)t * ld_in + (size_t)h * HD, j, PAIRS, rope_type, a, b);
    c = *reinterpret_cast<const float4*>(csr + 4 * j);
    s = *reinterpret_cast<const float4*>(csr + PAIRS + 4 * j);
  }
  const float* w = (h < H) ? qw : kw;
  if (w) {
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) ss += a[k] * a[k] + b[k] * b[k];
#pragma unroll
    for (int o = LPI / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    float inv = rsqrtf(ss / (float)HD + eps);
    if (!isfinite(inv)) inv = 0.f;
    float w0[4], w1[4];
    qk_loadw(w, j, PAIRS, rope_type, w0, w1);
#pragma unroll
    for (int k = 0; k < 4; ++k) { a[k] *= inv * w0[k]; b[k] *= inv * w1[k]; }
  }
  const float cc[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
  float o0[4], o1[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    o0[k] = a[k] * cc[k] - b[k] * sn[k];
    o1[k] = a[k] * sn[k] + b[k] * cc[k];
  }
  if (live) qk_store8<T>(out + (size_t)t * ld_out + (size_t)h * HD, j, PAIRS, rope_type, o0, o1);
}

template <typename T, int HD>
__global__ void __launch_bounds__(256) qk_norm_rope_bwd_vec_kernel(
    const T* __restrict__ dout, int ld_dout, const T* __restrict__ qkv, int ld_in, T* __restrict__ dqkv, int ld_dqkv,
    const float* __restrict__ qw, const float* __restrict__ kw, const float* __restrict__ cs, const int* __restrict__ pos,
    float* __restrict__ part_q, float* __restrict__ part_k, int n_tok, int H, int KV, float eps, int rope_type,
    int items_per_block) {
  constexpr int PAIRS = HD / 2, LPI = HD / 8, IPW = 32 / LPI, U = 2;
  __shared__ __align__(16) float s_w[2][HD];        // q and k norm weights
  __shared__ float s_dw[2][8][HD];                  // [q|k][warp][column], summed over the warp's items
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPI, j = lane % LPI;
  const bool norm = qw != nullptr;
  if (norm)
    for (int i = threadIdx.x; i < HD; i += blockDim.x) { s_w[0][i] = qw[i]; s_w[1][i] = kw[i]; }
  __syncthreads();
  float accq0[4] = {0, 0, 0, 0}, accq1[4] = {0, 0, 0, 0}, acck0[4] = {0, 0, 0, 0}, acck1[4] = {0, 0, 0, 0};
  const int heads = H + KV;
  const int total = n_tok * heads;
  const int it0 = blockIdx.x * items_per_block, it1 = min(total, it0 + items_per_block);
  for (int base = it0 + warp * (IPW * U); base < it1; base += 8 * IPW * U) {
    float g0[U][4], g1[U][4], x0[U][4], x1[U][4];
    bool live[U], isq[U];
    int tt[U], hh[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int item = base + u * IPW + sub;
      live[u] = item < it1;
      const int t = live[u] ? item / heads : 0;
      tt[u] = t;
      hh[u] = live[u] ? item - t * heads : 0;
      isq[u] = hh[u] < H;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float d0[4] = {0, 0, 0, 0}, d1[4] = {0, 0, 0, 0};
      float4 c = make_float4(1, 1, 1, 1), s = make_float4(0, 0, 0, 0);
#pragma unroll
      for (int k = 0; k < 4; ++k) { x0[u][k] = 0.f; x1[u][k] = 0.f; }
      if (live[u]) {
        const float* csr = cs + (size_t)pos[tt[u]] * HD;
        qk_load8<T>(dout + (size_t)tt[u] * ld_dout + (size_t)hh[u] * HD, j, PAIRS, rope_type, d0, d1);
        if (norm) qk_load8<T>(qkv + (size_t)tt[u] * ld_in + (size_t)hh[u] * HD, j, PAIRS, rope_type, x0[u], x1[u]);
        c = *reinterpret_cast<const float4*>(csr + 4 * j);
        s = *reinterpret_cast<const float4*>(csr + PAIRS + 4 * j);
      }
      const float cc[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        g0[u][k] = d0[k] * cc[k] + d1[k] * sn[k];   // inverse rotation
        g1[u][k] = -d0[k] * sn[k] + d1[k] * cc[k];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      T* dst = dqkv + (size_t)tt[u] * ld_dqkv + (size_t)hh[u] * HD;
      if (!norm) {
        if (live[u]) qk_store8<T>(dst, j, PAIRS, rope_type, g0[u], g1[u]);
        continue;
      }
      float w0[4], w1[4];
      qk_loadw(s_w[isq[u] ? 0 : 1], j, PAIRS, rope_type, w0, w1);
      float ss = 0.f, dot = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        ss += x0[u][k] * x0[u][k] + x1[u][k] * x1[u][k];
        dot += g0[u][k] * w0[k] * x0[u][k] + g1[u][k] * w1[k] * x1[u][k];
      }
#pragma unroll
      for (int o = LPI / 2; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        dot += __shfl_xor_sync(0xffffffffu, dot, o);
      }
      float inv = rsqrtf(ss / (float)HD + eps);
      if (!isfinite(inv)) inv = 0.f;
      const float coef = inv * inv * inv * dot / (float)HD;
      float o0[4], o1[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        o0[k] = g0[u][k] * w0[k] * inv - x0[u][k] * coef;
        o1[k] = g1[u][k] * w1[k] * inv - x1[u][k] * coef;
        const float a0 = live[u] ? g0[u][k] * x0[u][k] * inv : 0.f;
        const float a1 = live[u] ? g1[u][k] * x1[u][k] * inv : 0.f;
        accq0[k] += isq[u] ? a0 : 0.f;
        accq1[k] += isq[u] ? a1 : 0.f;
        acck0[k] += isq[u] ? 0.f : a0;
        acck1[k] += isq[u] ? 0.f : a1;
      }
      if (live[u]) qk_store8<T>(dst, j, PAIRS, rope_type, o0, o1);
    }
  }
  if (!part_q) return;
  // lanes with the same j hold the same columns: fold the item groups of the warp, then the warps, in a fixed order
#pragma unroll
  for (int k = 0; k < 4; ++k) {
#pragma unroll
    for (int o = LPI; o < 32; o <<= 1) {
      accq0[k] += __shfl_xor_sync(0xffffffffu, accq0[k], o);
      accq1[k] += __shfl_xor_sync(0xffffffffu, accq1[k], o);
      acck0[k] += __shfl_xor_sync(0xffffffffu, acck0[k], o);
      acck1[k] += __shfl_xor_sync(0xffffffffu, acck1[k], o);
    }
  }
  if (sub == 0) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i0 = rope_type == 0 ? 8 * j + 2 * k : 4 * j + k;
      const int i1 = rope_type == 0 ? 8 * j + 2 * k + 1 : PAIRS + 4 * j + k;
      s_dw[0][warp][i0] = accq0[k]; s_dw[0][warp][i1] = accq1[k];
      s_dw[1][warp][i0] = acck0[k]; s_dw[1][warp][i1] = acck1[k];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < HD; i += blockDim.x) {
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int wv = 0; wv < 8; ++wv) { sq += s_dw[0][wv][i]; sk += s_dw[1][wv][i]; }
    part_q[(size_t)blockIdx.x * HD + i] = sq;
    part_k[(size_t)blockIdx.x * HD + i] = sk;
  }
}

// ------------------------------------------------------------------------------------------ casts / fills
template <typename T>
__global__ void cast_f32_to_16_kernel(const float* __restrict__ src, T* __restrict__ dst, long long n) {
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8;
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (; i + 8 <= n; i += stride) {
    float4 a = *reinterpret_cast<const float4*>(src + i), b = *reinterpret_cast<const float4*>(src + i + 4);
    float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    store8<T>(dst + i, f);
  }
  if (i < n && i + 8 > n)
    for (long long j = i; j < n; ++j) dst[j] = Cvt<T>::from_f(src[j]);
}

}  // namespace gb

using namespace gb;

#define GB_LAUNCH_OK() gb_launch_rc()

extern "C" int gb_embed_fwd(const int* ids, const float* table, float* out, int n_tok, int d, int vocab, cudaStream_t st) {
  if (d % 4) return -1;
  GB_PDL_LAUNCH(embed_fwd_kernel, dim3(n_tok), dim3(128), st, ids, table, out, n_tok, d, vocab);
  return GB_LAUNCH_OK();
}
extern "C" int gb_embed_bwd(const int* ids, const float* dx, float* dtable, int n_tok, int d, int vocab, cudaStream_t st) {
  if (d > EMB_THREADS * EMB_MAX_COLS || vocab > EMB_MAX_VOCAB || vocab <= 0) return -1;
  void* first = nullptr;
  if (cudaGetSymbolAddress(&first, g_emb_first) != cudaSuccess) return -12;
  if (cudaMemsetAsync(first, 0x7f, (size_t)vocab * sizeof(int), st) != cudaSuccess) return -12;   // 0x7f7f7f7f > any token index
  embed_first_kernel<<<(n_tok + 255) / 256, 256, 0, st>>>(ids, n_tok, vocab);
  embed_bwd_kernel<<<n_tok, EMB_THREADS, 0, st>>>(ids, dx, dtable, n_tok, d, vocab);
  return GB_LAUNCH_OK();
}

// The same sums from ids that were sorted with a STABLE sort (sorted_ids ascending, order[p] = the token that
// landed at p): the tokens of one id are neighbours and already in increasing token order, so the block at the
// first position of a run adds that run's rows and every other block leaves.  Linear in the number of tokens,
// where the unsorted form above walks the whole id list once per distinct id.
extern "C" int gb_embed_bwd_sorted(const int* sorted_ids, const long long* order, const float* dx, float* dtable,
                                   int n_tok, int d, int vocab, cudaStream_t st) {
  if (d > EMB_THREADS * EMB_MAX_COLS || vocab <= 0 || n_tok <= 0) return -1;
  embed_bwd_sorted_kernel<<<n_tok, EMB_THREADS, 0, st>>>(sorted_ids, order, dx, dtable, n_tok, d, vocab);
  return GB_LAUNCH_OK();
}

extern "C" int gb_rmsnorm_fwd(const float* x, const float* w, void* y, float* rrms, int rows, int d, float eps, int is_bf16,
                              cudaStream_t st) {
  if (d % 4) return -1;
  const int wpb = 8;
  dim3 grid((rows + wpb - 1) / wpb);
  if (is_bf16) GB_PDL_LAUNCH(rmsnorm_fwd_kernel<__nv_bfloat16>, dim3(grid), dim3(wpb * 32), st, x, w, (__nv_bfloat16*)y, rrms, rows, d, eps);
  else GB_PDL_LAUNCH(rmsnorm_fwd_kernel<__half>, dim3(grid), dim3(wpb * 32), st, x, w, (__half*)y, rrms, rows, d, eps);
  return GB_LAUNCH_OK();
}

// Number of row blocks (and rows of the partial buffer) gb_rmsnorm_bwd uses for `rows`.
extern "C" int gb_rmsnorm_bwd_blocks(int rows) {
  int b = (rows + 7) / 8;   // one row per warp while that still fits a modest partial buffer
  return b > 592 ? 592 : (b < 1 ? 1 : b);   // four blocks of 8 warps per SM
}

// dw (fp32 [d]) is accumulated (+=).  `part` must hold gb_rmsnorm_bwd_blocks(rows) * d floats.
// Column sums are formed per warp, then per block, then block by block in index order: the result is
// bit-reproducible from run to run.
extern "C" int gb_rmsnorm_bwd(const void* g, const float* x, const float* w, const float* rrms, const float* dres,
                              float* dx_out, void* dx16, float* part, float* dw, int rows, int d, int is_bf16,
                              cudaStream_t st) {
  if (d % 4) return -1;
  const int nb = gb_rmsnorm_bwd_blocks(rows);
  const int rpb = (rows + nb - 1) / nb;
  int wpb = 12288 / d;
  wpb = wpb > 8 ? 8 : wpb;
  if (wpb < 1) return -1;
  const size_t smem = (size_t)d * wpb * sizeof(float);
  const int threads = wpb * 32;
  const bool vec = d % 256 == 0 && d <= 1024 &&
                   (((uintptr_t)g | (uintptr_t)x | (uintptr_t)dres | (uintptr_t)dx_out | (uintptr_t)dx16) & 15) == 0;
  if (vec) {
    const size_t vsmem = (size_t)d * 9 * sizeof(float);
#define GB_RMS_BWD_VEC(T, NV)                                                                                      \
  rmsnorm_bwd_vec_kernel<T, NV><<<nb, 256, vsmem, st>>>((const T*)g, x, w, rrms, dres, dx_out, (T*)dx16, part, rows, rpb)
#define GB_RMS_BWD_VEC_T(T)          \
  switch (d / 128) {                 \
    case 2: GB_RMS_BWD_VEC(T, 2); break; \
    case 4: GB_RMS_BWD_VEC(T, 4); break; \
    case 6: GB_RMS_BWD_VEC(T, 6); break; \
    default: GB_RMS_BWD_VEC(T, 8); break; \
  }
    if (is_bf16) { GB_RMS_BWD_VEC_T(__nv_bfloat16) } else { GB_RMS_BWD_VEC_T(__half) }
#undef GB_RMS_BWD_VEC_T
#undef GB_RMS_BWD_VEC
  } else if (is_bf16)
    rmsnorm_bwd_kernel<__nv_bfloat16><<<nb, threads, smem, st>>>((const __nv_bfloat16*)g, x, w, rrms, dres, dx_out,
                                                             (__nv_bfloat16*)dx16, part, rows, d, rpb);
  else
    rmsnorm_bwd_kernel<__half><<<nb, threads, smem, st>>>((const __half*)g, x, w, rrms, dres, dx_out, (__half*)dx16, part,
                                                      rows, d, rpb);
  if (dw) colsum_finalize_kernel<<<(d + 31) / 32, 256, 0, st>>>(part, dw, nb, d);
  return GB_LAUNCH_OK();
}

extern "C" int gb_qk_rope_blocks(int n_items) {
  int b = (n_items + 31) / 32;
  return b > 444 ? 444 : (b < 1 ? 1 : b);   // three 256-thread blocks of the backward kernel per SM
}

template <typename T>
static int qk_fwd_t(const void* qkv, int ld_in, void* out, int ld_out, const float* qw, const float* kw, const float* cs,
                    const int* pos, int n_tok, int H, int KV, int hd, float eps, int rope_type, cudaStream_t st) {
  const int items = n_tok * (H + KV);
  const int wpb = 8;
  const bool aligned = ld_in % 8 == 0 && ld_out % 8 == 0 && (qw == nullptr) == (kw == nullptr) &&
                       (((uintptr_t)qkv | (uintptr_t)out | (uintptr_t)cs | (uintptr_t)qw | (uintptr_t)kw) & 15) == 0;
  // Up to 64 tokens (a decode step) keep the one-item-per-warp kernel: its sums are grouped exactly as in the
  // token step's fused QK-norm + RoPE + cache-append kernel, so the two decode paths stay bit-identical.
  if (aligned && n_tok > 64 && (hd == 32 || hd == 64 || hd == 128 || hd == 256)) {
    const int ipb = wpb * (256 / hd);   // items per block
    dim3 vgrid((items + ipb - 1) / ipb);
#define GB_QK_FWD_VEC(HD) \
  GB_PDL_LAUNCH((qk_norm_rope_fwd_vec_kernel<T, HD>), dim3(vgrid), dim3(wpb * 32), st, (const T*)qkv, ld_in, (T*)out, ld_out, qw, kw, cs, pos, n_tok, H, KV, eps, rope_type)
    switch (hd) {
      case 32: GB_QK_FWD_VEC(32); break;
      case 64: GB_QK_FWD_VEC(64); break;
      case 128: GB_QK_FWD_VEC(128); break;
      default: GB_QK_FWD_VEC(256); break;
    }
#undef GB_QK_FWD_VEC
    return GB_LAUNCH_OK();
  }
  dim3 grid((items + wpb - 1) / wpb);
#define GB_QK_FWD(HD) \
  GB_PDL_LAUNCH((qk_norm_rope_fwd_kernel<T, HD>), dim3(grid), dim3(wpb * 32), st, (const T*)qkv, ld_in, (T*)out, ld_out, qw, kw, cs, pos, n_tok, H, KV, eps, rope_type)
  switch (hd) {
    case 32: GB_QK_FWD(32); break;
    case 64: GB_QK_FWD(64); break;
    case 96: GB_QK_FWD(96); break;
    case 128: GB_QK_FWD(128); break;
    case 256: GB_QK_FWD(256); break;
    default: return -1;
  }
#undef GB_QK_FWD
  return GB_LAUNCH_OK();
}

extern "C" int gb_qk_norm_rope_fwd(const void* qkv, int ld_in, void* out, int ld_out, const float* qw, const float* kw,
                                   const float* cos_sin, const int* pos, int n_tok, int H, int KV, int hd, float eps,
                                   int rope_type, int is_bf16, cudaStream_t st) {
  return is_bf16 ? qk_fwd_t<__nv_bfloat16>(qkv, ld_in, out, ld_out, qw, kw, cos_sin, pos, n_tok, H, KV, hd, eps, rope_type, st)
                 : qk_fwd_t<__half>(qkv, ld_in, out, ld_out, qw, kw, cos_sin, pos, n_tok, H, KV, hd, eps, rope_type, st);
}

template <typename T>
static int qk_bwd_t(const void* dout, int ld_dout, const void* qkv, int ld_in, void* dqkv, int ld_dqkv, const float* qw,
                    const float* kw, const float* cs, const int* pos, float* part, float* dqw, float* dkw, int n_tok,
                    int H, int KV, int hd, float eps, int rope_type, cudaStream_t st) {
  const int items = n_tok * (H + KV);
  const int nb = gb_qk_rope_blocks(items);
  const int ipb = (items + nb - 1) / nb;
  float* pq = part;
  float* pk = part ? part + (size_t)nb * hd : nullptr;
  const bool aligned = ld_dout % 8 == 0 && ld_in % 8 == 0 && ld_dqkv % 8 == 0 && (qw == nullptr) == (kw == nullptr) &&
                       (((uintptr_t)dout | (uintptr_t)qkv | (uintptr_t)dqkv | (uintptr_t)cs) & 15) == 0;
#define GB_QK_BWD_VEC(HD)                                                                                        \
  qk_norm_rope_bwd_vec_kernel<T, HD><<<nb, 256, 0, st>>>((const T*)dout, ld_dout, (const T*)qkv, ld_in, (T*)dqkv, \
                                                         ld_dqkv, qw, kw, cs, pos, pq, pk, n_tok, H, KV, eps,   \
                                                         rope_type, ipb)
#define GB_QK_BWD(HD)                                                                                                 \
  qk_norm_rope_bwd_kernel<T, HD><<<nb, 256, 0, st>>>((const T*)dout, ld_dout, (const T*)qkv, ld_in, (T*)dqkv, ld_dqkv, \
                                                     qw, kw, cs, pos, pq, pk, n_tok, H, KV, eps, rope_type, ipb)
  if (aligned && (hd == 32 || hd == 64 || hd == 128 || hd == 256)) {
    switch (hd) {
      case 32: GB_QK_BWD_VEC(32); break;
      case 64: GB_QK_BWD_VEC(64); break;
      case 128: GB_QK_BWD_VEC(128); break;
      default: GB_QK_BWD_VEC(256); break;
    }
  } else
  switch (hd) {
    case 32: GB_QK_BWD(32); break;
    case 64: GB_QK_BWD(64); break;
    case 96: GB_QK_BWD(96); break;
    case 128: GB_QK_BWD(128); break;
    case 256: GB_QK_BWD(256); break;
    default: return -1;
  }
#undef GB_QK_BWD
  if (qw && part && dqw) {
    colsum_finalize_kernel<<<(hd + 31) / 32, 256, 0, st>>>(pq, dqw, nb, hd);
    colsum_finalize_kernel<<<(hd + 31) / 32, 256, 0, st>>>(pk, dkw, nb, hd);
  }
  return GB_LAUNCH_OK();
}

// part: 2 * gb_qk_rope_blocks(n_tok*(H+KV)) * hd floats; dqw/dkw ([hd], fp32) are accumulated.
extern "C" int gb_qk_norm_rope_bwd(const void* dout, int ld_dout, const void* qkv, int ld_in, void* dqkv, int ld_dqkv,
                                   const float* qw, const float* kw, const float* cos_sin, const int* pos, float* part,
                                   float* dqw, float* dkw, int n_tok, int H, int KV, int hd, float eps, int rope_type,
                                   int is_bf16, cudaStream_t st) {
  return is_bf16 ? qk_bwd_t<__nv_bfloat16>(dout, ld_dout, qkv, ld_in, dqkv, ld_dqkv, qw, kw, cos_sin, pos, part, dqw, dkw,
                                           n_tok, H, KV, hd, eps, rope_type, st)
                 : qk_bwd_t<__half>(dout, ld_dout, qkv, ld_in, dqkv, ld_dqkv, qw, kw, cos_sin, pos, part, dqw, dkw, n_tok,
                                    H, KV, hd, eps, rope_type, st);
}

// out16[i] = sum_s part[s * n + i] (fixed order), the second stage of a split-K GEMM
template <typename T>
__global__ void splitk_reduce_kernel(const float* __restrict__ part, int splits, long long n, T* __restrict__ out) {
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (; i < n; i += stride) {
    float4 acc = *reinterpret_cast<const float4*>(part + i);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(part + (long long)s * n + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    uint2 q;
    q.x = gb::Cvt<T>::pack2(acc.x, acc.y);
    q.y = gb::Cvt<T>::pack2(acc.z, acc.w);
    *reinterpret_cast<uint2*>(out + i) = q;
  }
}

extern "C" int gb_splitk_reduce(const float* part, int splits, long long n, void* out16, int is_bf16, cudaStream_t st) {
  if (n <= 0 || n % 4 || splits < 1) return -1;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (is_bf16) splitk_reduce_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, st>>>(part, splits, n, (__nv_bfloat16*)out16);
  else splitk_reduce_kernel<__half><<<(int)blocks, 256, 0, st>>>(part, splits, n, (__half*)out16);
  return GB_LAUNCH_OK();
}

// out[i] += sum_s part[s * n + i] (fixed order): second stage of a split-K weight gradient
__global__ void splitk_accumulate_kernel(const float* __restrict__ part, int splits, long long n, float* __restrict__ out) {
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (; i < n; i += stride) {
    float4 acc = *reinterpret_cast<const float4*>(out + i);
    for (int s = 0; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(part + (long long)s * n + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(out + i) = acc;
  }
}

extern "C" int gb_splitk_accumulate(const float* part, int splits, long long n, float* out, cudaStream_t st) {
  if (!part || !out || n <= 0 || n % 4 || splits < 1) return -1;
  if ((reinterpret_cast<uintptr_t>(part) | reinterpret_cast<uintptr_t>(out)) & 15) return -2;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  splitk_accumulate_kernel<<<(int)blocks, 256, 0, st>>>(part, splits, n, out);
  return GB_LAUNCH_OK();
}

extern "C" int gb_cast_f32_to_16(const float* src, void* dst, long long n, int is_bf16, cudaStream_t st) {
  if (n <= 0) return 0;
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  if (is_bf16) cast_f32_to_16_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, st>>>(src, (__nv_bfloat16*)dst, n);
  else cast_f32_to_16_kernel<__half><<<(int)blocks, 256, 0, st>>>(src, (__half*)dst, n);
  return GB_LAUNCH_OK();
}
