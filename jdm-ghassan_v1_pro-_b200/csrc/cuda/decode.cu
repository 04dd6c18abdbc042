// Decode-time kernels (contract in gb_decode.h).  Batch-1 decoding reads every active weight once per token and
// does two flops per weight: it is bound by HBM bandwidth and launch count, not by the tensor cores.  So weights
// stay in their storage format (fp16 / bf16 / 8-bit / 4-bit blocks) and are expanded in registers inside the dot
// product; one warp owns one output row, lanes stride over 8-value units of the row, partial sums are fp32.
#include <type_traits>

#include "sm100_common.cuh"
#include "gb_decode.h"
#include "decode_fmt.cuh"

namespace gb {

constexpr int GV_WARPS = 8;            // output rows per CTA
constexpr int GV_THREADS = GV_WARPS * 32;

template <typename XT>
__device__ __forceinline__ float dot8(const float (&w)[8], const XT* __restrict__ x) {
  const uint4 q = *reinterpret_cast<const uint4*>(x);
  float s = 0.f;
  if constexpr (std::is_same<XT, __half>::value) {
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); s += w[2 * i] * f.x + w[2 * i + 1] * f.y; }
  } else {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); s += w[2 * i] * f.x + w[2 * i + 1] * f.y; }
  }
  return s;
}

// KS warps share one stored row: warp slice ks takes units ks*32 + lane, stepping by 32*KS.  Decoding one token is
// bound by load latency, not bandwidth (a row is a few hundred bytes), so the short rows are spread over more warps
// and every lane keeps several independent loads in flight; the slices meet in shared memory.
template <int FMT, int NB, int KS, typename XT>
__device__ __forceinline__ void row_partial(const uint8_t* __restrict__ wrow, int K, const XT* __restrict__ x, long long ldx,
                                            int nb, int ks, float (&acc)[NB]) {
  const int lane = threadIdx.x & 31;
#pragma unroll 2
  for (int u = lane + 32 * ks; u < (K >> 3); u += 32 * KS) {
    float w[8];
    load8<FMT>(wrow, u, w);
#pragma unroll
    for (int j = 0; j < NB; ++j)
      if (j < nb) acc[j] += dot8<XT>(w, x + j * ldx + 8 * u);
  }
}

// sum over lanes, then over the KS warps of the row; the result is valid in lane 0 of slice 0
template <int KS>
__device__ __forceinline__ float row_finish(float v, float* __restrict__ sm, int row_in_cta, int ks) {
  v = warp_sum(v);
  if constexpr (KS == 1) return v;
  if ((threadIdx.x & 31) == 0) sm[row_in_cta * KS + ks] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < KS; ++i) t += sm[row_in_cta * KS + i];
  __syncthreads();
  return t;
}

template <int FMT, int NB, int KS, typename XT>
__global__ void __launch_bounds__(GV_THREADS) gemv_kernel(const uint8_t* __restrict__ W, long long row_bytes, int N, int K,
                                                         const XT* __restrict__ x, long long ldx, int B,
                                                         void* __restrict__ out, long long ldo, int out_f32,
                                                         const float* __restrict__ addend, long long ld_add) {
  pdl_wait();
  __shared__ float sm[GV_WARPS];
  const int warp = threadIdx.x >> 5, ric = warp / KS, ks = warp % KS;
  const int row = blockIdx.x * (GV_WARPS / KS) + ric;
  const bool live = row < N;                              // dead rows still take part in the block barriers
  const uint8_t* wrow = W + (size_t)(live ? row : 0) * row_bytes;
  for (int b0 = 0; b0 < B; b0 += NB) {
    float acc[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) acc[j] = 0.f;
    const int nb = min(NB, B - b0);
    if (live) row_partial<FMT, NB, KS, XT>(wrow, K, x + (long long)b0 * ldx, ldx, nb, ks, acc);
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const float v0 = row_finish<KS>(acc[j], sm, ric, ks);
      if (live && j < nb && ks == 0 && (threadIdx.x & 31) == 0) {
        float v = v0;
        if (addend) v += addend[(long long)(b0 + j) * ld_add + row];
        if (out_f32) reinterpret_cast<float*>(out)[(long long)(b0 + j) * ldo + row] = v;
        else reinterpret_cast<XT*>(out)[(long long)(b0 + j) * ldo + row] = Cvt<XT>::from_f(v);
      }
    }
  }
}

template <int FMT, int KS, typename XT>
__global__ void __launch_bounds__(GV_THREADS) expert_swiglu_kernel(const uint8_t* __restrict__ Wg, const uint8_t* __restrict__ Wu,
                                                                  long long row_bytes, int ne, int E, int d,
                                                                  const XT* __restrict__ x, const int* __restrict__ idx,
                                                                  int top_k, int slots, XT* __restrict__ act) {
  pdl_wait();
  __shared__ float sm[2 * GV_WARPS];
  const int warp = threadIdx.x >> 5, ric = warp / KS, ks = warp % KS;
  const int j = blockIdx.x * (GV_WARPS / KS) + ric;
  const int b = blockIdx.y / slots, slot = blockIdx.y % slots;
  const int e = slot < top_k ? idx[b * top_k + slot] : ne;
  const bool live = j < E && e >= 0 && e <= ne;
  float g[1] = {0.f}, u[1] = {0.f};
  if (live) {
    const size_t r = (size_t)e * E + j;
    row_partial<FMT, 1, KS, XT>(Wg + r * row_bytes, d, x + (long long)b * d, d, 1, ks, g);
    row_partial<FMT, 1, KS, XT>(Wu + r * row_bytes, d, x + (long long)b * d, d, 1, ks, u);
  }
  const float gs = row_finish<KS>(g[0], sm, ric, ks);
  const float us = row_finish<KS>(u[0], sm + GV_WARPS, ric, ks);
  if (live && ks == 0 && (threadIdx.x & 31) == 0)
    act[((long long)b * slots + slot) * E + j] = Cvt<XT>::from_f(gs / (1.f + __expf(-gs)) * us);
}

template <int FMT, int KS, typename XT>
__global__ void __launch_bounds__(GV_THREADS) expert_down_kernel(const uint8_t* __restrict__ Wd, long long row_bytes, int ne, int d,
                                                                int E, const XT* __restrict__ act, const int* __restrict__ idx,
                                                                const float* __restrict__ w, int top_k, int slots,
                                                                const float* __restrict__ resid, float* __restrict__ out) {
  pdl_wait();
  __shared__ float sm[GV_WARPS];
  const int warp = threadIdx.x >> 5, ric = warp / KS, ks = warp % KS;
  const int r = blockIdx.x * (GV_WARPS / KS) + ric;
  const int b = blockIdx.y;
  const bool live = r < d;
  // weighted sum over the slots taken per lane before any reduction: one reduction per output value, and the
  // loads of different slots do not wait for one another.  Slot order and lane order are fixed: reproducible.
  float total = 0.f;
  if (live) {
    for (int slot = 0; slot < slots; ++slot) {
      const int e = slot < top_k ? idx[b * top_k + slot] : ne;
      if (e < 0 || e > ne) continue;
      const float wgt = slot < top_k ? w[b * top_k + slot] : 1.f;
      float y[1] = {0.f};
      row_partial<FMT, 1, KS, XT>(Wd + ((size_t)e * d + r) * row_bytes, E, act + ((long long)b * slots + slot) * E, E, 1, ks, y);
      total += wgt * y[0];
    }
  }
  const float t = row_finish<KS>(total, sm, ric, ks);
  if (live && ks == 0 && (threadIdx.x & 31) == 0) out[(long long)b * d + r] = resid[(long long)b * d + r] + t;
}

// Router for decode: one block per token, one warp per expert (round robin), then a serial soft-max / top-k over at
// most 64 experts.  Same rules as the training router: bias steers the selection only, ties go to the lowest index,
// weights are the selected probabilities renormalised.
template <typename XT>
__global__ void __launch_bounds__(256) decode_route_kernel(const XT* __restrict__ x, const float* __restrict__ rw,
                                                          const float* __restrict__ bias, int d, int ne, int top_k,
                                                          int* __restrict__ idx, float* __restrict__ wout) {
  pdl_wait();
  __shared__ float lg[64];
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const XT* xr = x + (long long)b * d;
  for (int e = warp; e < ne; e += 8) {
    const float* wr = rw + (size_t)e * d;
    float s = 0.f;
    for (int i = lane * 2; i < d; i += 64) {
      const float2 xv = Cvt<XT>::unpack2(*reinterpret_cast<const uint32_t*>(xr + i));
      const float2 wv = *reinterpret_cast<const float2*>(wr + i);
      s += xv.x * wv.x + xv.y * wv.y;
    }
    s = warp_sum(s);
    if (lane == 0) lg[e] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mx = -INFINITY;
    for (int e = 0; e < ne; ++e) mx = fmaxf(mx, lg[e]);
    float sum = 0.f;
    for (int e = 0; e < ne; ++e) { lg[e] = __expf(lg[e] - mx); sum += lg[e]; }
    const float inv = 1.f / sum;
    unsigned long long taken = 0ull;
    float psel[8], psum = 0.f;
    int esel[8];
    for (int k = 0; k < top_k; ++k) {
      float bv = -INFINITY;
      int bi = 0;
      for (int e = 0; e < ne; ++e) {
        if (taken >> e & 1ull) continue;
        const float sc = lg[e] * inv + (bias ? bias[e] : 0.f);
        if (sc > bv) { bv = sc; bi = e; }
      }
      taken |= 1ull << bi;
      esel[k] = bi;
      psel[k] = lg[bi] * inv;
      psum += psel[k];
    }
    const float invs = psum > 1e-8f ? 1.f / psum : 0.f;
    for (int k = 0; k < top_k; ++k) {
      idx[b * top_k + k] = esel[k];
      wout[b * top_k + k] = psel[k] * invs;
    }
  }
}

// ---------------------------------------------------------------------------------------------- KV cache
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k, long long ld_k, const T* __restrict__ v, long long ld_v,
                                 T* __restrict__ cK, T* __restrict__ cV, int* __restrict__ slot_pos,
                                 const gb_seq_state* __restrict__ st, int cap, int pinned, int kv_dim) {
  pdl_wait();
  const int b = blockIdx.x;
  const gb_seq_state s = st[b];
  const int slot = s.cache_len < cap ? s.cache_len : pinned + s.ring_start;
  T* dk = cK + ((long long)b * cap + slot) * kv_dim;
  T* dv = cV + ((long long)b * cap + slot) * kv_dim;
  for (int i = threadIdx.x * 8; i < kv_dim; i += blockDim.x * 8) {
    *reinterpret_cast<uint4*>(dk + i) = *reinterpret_cast<const uint4*>(k + b * ld_k + i);
    *reinterpret_cast<uint4*>(dv + i) = *reinterpret_cast<const uint4*>(v + b * ld_v + i);
  }
  if (threadIdx.x == 0) slot_pos[(long long)b * cap + slot] = s.abs_pos;
}

__global__ void decode_advance_kernel(gb_seq_state* __restrict__ st, int* __restrict__ pos_out, int B, int cap, int pinned) {
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  gb_seq_state s = st[b];
  if (s.cache_len < cap) s.cache_len += 1;
  else s.ring_start = (s.ring_start + 1) % max(1, cap - pinned);
  s.abs_pos += 1;
  st[b] = s;
  pos_out[b] = s.abs_pos;
}

// ---------------------------------------------------------------------------------------------- decode attention
// grid (B*KV, splits), 4 warps.  A block serves the G = H/KV query heads that share one K/V head, so each cached
// row is read once per group.  Each warp walks its share of the slots with an online softmax per query head; the
// four warps and then the splits are merged with the usual (max, sum, weighted output) rule.
template <typename T, int HD, int G>
__global__ void __launch_bounds__(128) decode_attn_kernel(const T* __restrict__ q, long long ld_q, const T* __restrict__ cK,
                                                         const T* __restrict__ cV, const int* __restrict__ slot_pos,
                                                         const gb_seq_state* __restrict__ st, float* __restrict__ scratch,
                                                         int splits, int H, int KV, int cap, int window, float scale,
                                                         int* __restrict__ ticket, T* __restrict__ out, long long ld_o) {
  pdl_wait();
  constexpr int EPL = HD / 32;   // elements per lane
  const int b = blockIdx.x / KV, kvh = blockIdx.x % KV, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const gb_seq_state s = st[b];
  // the step's own token was appended before this kernel and is not counted in cache_len yet
  const int n_slots = min(cap, s.cache_len + 1);
  const int own_slot = s.cache_len < cap ? s.cache_len : -1;   // when the ring is full the new token replaced a slot
  (void)own_slot;
  float qv[G][EPL], m[G], l[G], o[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const T* qp = q + b * ld_q + (long long)(kvh * G + g) * HD + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) { qv[g][e] = Cvt<T>::to_f(qp[e]) * scale; o[g][e] = 0.f; }
    m[g] = -INFINITY;
    l[g] = 0.f;
  }
  const int per = (n_slots + splits - 1) / splits;
  const int lo = split * per, hi = min(n_slots, lo + per);
  const long long kvd = (long long)KV * HD;
  for (int j = lo + warp; j < hi; j += 4) {
    if (window > 0 && s.abs_pos - slot_pos[(long long)b * cap + j] >= window) continue;
    const T* kp = cK + ((long long)b * cap + j) * kvd + kvh * HD + lane * EPL;
    const T* vp = cV + ((long long)b * cap + j) * kvd + kvh * HD + lane * EPL;
    float kf[EPL], vf[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) { kf[e] = Cvt<T>::to_f(kp[e]); vf[e] = Cvt<T>::to_f(vp[e]); }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) d += qv[g][e] * kf[e];
      d = warp_sum(d);
      const float mn = fmaxf(m[g], d);
      const float c = __expf(m[g] - mn), p = __expf(d - mn);
      l[g] = l[g] * c + p;
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[g][e] = o[g][e] * c + p * vf[e];
      m[g] = mn;
    }
  }
  // merge the four warps through shared memory
  __shared__ float sm_m[4][G], sm_l[4][G], sm_o[4][G][HD];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
#pragma unroll
    for (int e = 0; e < EPL; ++e) sm_o[warp][g][lane * EPL + e] = o[g][e];
  }
  __syncthreads();
  for (int t = threadIdx.x; t < G * HD; t += 128) {
    const int g = t / HD, c = t % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = sm_m[w][g] == -INFINITY ? 0.f : __expf(sm_m[w][g] - mm);
      ll += sm_l[w][g] * f;
      oo += sm_o[w][g][c] * f;
    }
    float* dst = scratch + (((long long)b * H + kvh * G + g) * splits + split) * (HD + 2);
    dst[2 + c] = oo;
    if (c == 0) { dst[0] = mm; dst[1] = ll; }
  }
  if (ticket == nullptr) return;            // the splits are merged by decode_attn_merge_kernel
  // The last split of this (sequence, kv head) to get here merges all of them, in split order: same result whoever
  // it is.  The ticket returns to zero for the next launch.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(&ticket[blockIdx.x], 1);
    s_last = (t == splits - 1);
    if (s_last) ticket[blockIdx.x] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int t = threadIdx.x; t < G * HD; t += 128) {
    const int g = t / HD, c = t % HD;
    const float* base = scratch + ((long long)b * H + kvh * G + g) * splits * (HD + 2);
    float mm = -INFINITY;
    for (int sp = 0; sp < splits; ++sp) mm = fmaxf(mm, __ldcg(base + sp * (HD + 2)));
    float ll = 0.f, oo = 0.f;
    for (int sp = 0; sp < splits; ++sp) {
      const float ms = __ldcg(base + sp * (HD + 2));
      const float f = ms == -INFINITY ? 0.f : __expf(ms - mm);
      ll += __ldcg(base + sp * (HD + 2) + 1) * f;
      oo += __ldcg(base + sp * (HD + 2) + 2 + c) * f;
    }
    out[b * ld_o + (long long)(kvh * G + g) * HD + c] = Cvt<T>::from_f(ll > 0.f ? oo / ll : 0.f);
  }
}

// One block of HD threads per (sequence, head).  The split maxima and sums are read by one thread per split and the
// per-split factors go through shared memory, so that the long loop over the splits carries no dependent load: the
// earlier form (every thread walking all splits twice, each step waiting for its load) took 12 us per launch, a
// fifth of a token step, for a few kilobytes.
template <typename T, int HD>
__global__ void decode_attn_merge_kernel(const float* __restrict__ scratch, int splits, T* __restrict__ out, long long ld_o, int H) {
  __shared__ float s_f[128];
  __shared__ float s_red[4];
  pdl_wait();
  const int b = blockIdx.x / H, h = blockIdx.x % H, c = threadIdx.x;
  const float* base = scratch + ((long long)b * H + h) * splits * (HD + 2);
  // maximum over the splits (splits <= 128: up to two per thread)
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  if (c < splits) { m0 = base[c * (HD + 2)]; l0 = base[c * (HD + 2) + 1]; }
  if (c + HD < splits) { m1 = base[(c + HD) * (HD + 2)]; l1 = base[(c + HD) * (HD + 2) + 1]; }
  float mm = warp_max(fmaxf(m0, m1));
  if ((c & 31) == 0) s_red[c >> 5] = mm;
  __syncthreads();
  mm = s_red[0];
  for (int w = 1; w < HD / 32; ++w) mm = fmaxf(mm, s_red[w]);
  const float f0 = m0 == -INFINITY ? 0.f : __expf(m0 - mm), f1 = m1 == -INFINITY ? 0.f : __expf(m1 - mm);
  if (c < splits) s_f[c] = f0;
  if (c + HD < splits) s_f[c + HD] = f1;
  __syncthreads();                       // also orders the reads of s_red above against the writes below
  float ll = warp_sum(l0 * f0 + l1 * f1);
  if ((c & 31) == 0) s_red[c >> 5] = ll;
  __syncthreads();
  ll = 0.f;
  for (int w = 0; w < HD / 32; ++w) ll += s_red[w];
  float oo = 0.f;
#pragma unroll 8
  for (int s = 0; s < splits; ++s) oo += base[s * (HD + 2) + 2 + c] * s_f[s];
  out[b * ld_o + (long long)h * HD + c] = Cvt<T>::from_f(ll > 0.f ? oo / ll : 0.f);
}

// ---------------------------------------------------------------------------------------------- fused decode step
// Fewer, fatter kernels for the token step: at batch 1 every kernel costs a few microseconds however little it does.
//   gemv_norm:            RMSNorm of the fp32 residual inside the GEMV (every block normalises the row it needs)
//   route_norm:           RMSNorm + router (soft-max, bias-steered top-k), one block per token
//   swiglu_norm:          RMSNorm + gate/up rows of the selected experts
//   qk_rope_append:       QK-norm + RoPE; k heads land in the cache slot, v heads are copied beside them
//   decode_attn (ticket): the last split to finish merges the partial results; measured slower than the separate
//                         merge launch (the merge is a serial tail of the longest block), so the engine does not use it
// Rounding points are those of the separate kernels (normalised activations pass through 16 bits), so both routes
// give the same numbers.

// Row b of x (fp32, d values) normalised into xs (16-bit) by one warp, as rmsnorm_fwd_kernel does it.
template <typename XT>
__device__ __forceinline__ void norm_row_to_smem(const float* __restrict__ x, const float* __restrict__ w, XT* __restrict__ xs,
                                                 int d, float eps) {
  const int lane = threadIdx.x & 31;
  const float4* xr = reinterpret_cast<const float4*>(x);
  float ss = 0.f;
  for (int i = lane; i < d / 4; i += 32) {
    const float4 v = xr[i];
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = warp_sum(ss);
  float inv = rsqrtf(ss / (float)d + eps);
  if (!isfinite(inv)) inv = 0.f;
  const float4* wr = reinterpret_cast<const float4*>(w);
  for (int i = lane; i < d / 4; i += 32) {
    const float4 v = xr[i], g = wr[i];
    uint2 o;
    o.x = Cvt<XT>::pack2(v.x * inv * g.x, v.y * inv * g.y);
    o.y = Cvt<XT>::pack2(v.z * inv * g.z, v.w * inv * g.w);
    *reinterpret_cast<uint2*>(xs + 4 * i) = o;
  }
}

template <int FMT, int NB, int KS, typename XT>
__global__ void __launch_bounds__(GV_THREADS) gemv_norm_kernel(const uint8_t* __restrict__ W, long long row_bytes, int N, int K,
                                                              const float* __restrict__ x32, long long ldx32,
                                                              const float* __restrict__ norm_w, float eps, int B,
                                                              void* __restrict__ out, long long ldo, int out_f32) {
  pdl_wait();
  extern __shared__ __align__(16) uint8_t gv_dyn[];
  XT* xs = reinterpret_cast<XT*>(gv_dyn);                 // [B][K]
  __shared__ float sm[GV_WARPS];
  const int warp = threadIdx.x >> 5, ric = warp / KS, ks = warp % KS;
  for (int b = warp; b < B; b += GV_WARPS) norm_row_to_smem<XT>(x32 + b * ldx32, norm_w, xs + (long long)b * K, K, eps);
  __syncthreads();
  const int row = blockIdx.x * (GV_WARPS / KS) + ric;
  const bool live = row < N;
  const uint8_t* wrow = W + (size_t)(live ? row : 0) * row_bytes;
  for (int b0 = 0; b0 < B; b0 += NB) {
    float acc[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) acc[j] = 0.f;
    const int nb = min(NB, B - b0);
    if (live) row_partial<FMT, NB, KS, XT>(wrow, K, xs + (long long)b0 * K, K, nb, ks, acc);
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const float v0 = row_finish<KS>(acc[j], sm, ric, ks);
      if (live && j < nb && ks == 0 && (threadIdx.x & 31) == 0) {
        if (out_f32) reinterpret_cast<float*>(out)[(long long)(b0 + j) * ldo + row] = v0;
        else reinterpret_cast<XT*>(out)[(long long)(b0 + j) * ldo + row] = Cvt<XT>::from_f(v0);
      }
    }
  }
}

// Router of one token from its normalised activations in shared memory (rules of decode_route_kernel).  All threads
// of the block call it; the selection is left in esel / wsel (shared).
template <typename XT>
__device__ __forceinline__ void route_in_block(const XT* __restrict__ xs, const float* __restrict__ rw, const float* __restrict__ bias,
                                               int d, int ne, int top_k, float* __restrict__ lg, int* __restrict__ esel,
                                               float* __restrict__ wsel) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = warp; e < ne; e += GV_WARPS) {
    const float* wr = rw + (size_t)e * d;
    float s = 0.f;
    for (int i = lane * 2; i < d; i += 64) {
      const float2 xv = Cvt<XT>::unpack2(*reinterpret_cast<const uint32_t*>(xs + i));
      const float2 wv = *reinterpret_cast<const float2*>(wr + i);
      s += xv.x * wv.x + xv.y * wv.y;
    }
    s = warp_sum(s);
    if (lane == 0) lg[e] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mx = -INFINITY;
    for (int e = 0; e < ne; ++e) mx = fmaxf(mx, lg[e]);
    float sum = 0.f;
    for (int e = 0; e < ne; ++e) { lg[e] = __expf(lg[e] - mx); sum += lg[e]; }
    const float inv = 1.f / sum;
    unsigned long long taken = 0ull;
    float psel[8], psum = 0.f;
    for (int k = 0; k < top_k; ++k) {
      float bv = -INFINITY;
      int bi = 0;
      for (int e = 0; e < ne; ++e) {
        if (taken >> e & 1ull) continue;
        const float sc = lg[e] * inv + (bias ? bias[e] : 0.f);
        if (sc > bv) { bv = sc; bi = e; }
      }
      taken |= 1ull << bi;
      esel[k] = bi;
      psel[k] = lg[bi] * inv;
      psum += psel[k];
    }
    const float invs = psum > 1e-8f ? 1.f / psum : 0.f;
    for (int k = 0; k < top_k; ++k) wsel[k] = psel[k] * invs;
  }
  __syncthreads();
}

// Router of a token on its own: RMSNorm of the fp32 row + soft-max + bias-steered top-k; one block per token.  (Doing
// this inside every gate/up block was measured: thousands of blocks re-reading the router weights cost more than
// the launch it saved.)
template <typename XT>
__global__ void __launch_bounds__(GV_THREADS) route_norm_kernel(const float* __restrict__ x32, const float* __restrict__ norm_w,
                                                               float eps, const float* __restrict__ rw,
                                                               const float* __restrict__ bias, int d, int ne, int top_k,
                                                               int* __restrict__ idx_out, float* __restrict__ w_out) {
  pdl_wait();
  extern __shared__ __align__(16) uint8_t gv_dyn[];
  XT* xs = reinterpret_cast<XT*>(gv_dyn);
  __shared__ float lg[64];
  __shared__ int esel[8];
  __shared__ float wsel[8];
  const int b = blockIdx.x;
  if ((threadIdx.x >> 5) == 0) norm_row_to_smem<XT>(x32 + (long long)b * d, norm_w, xs, d, eps);
  __syncthreads();
  route_in_block<XT>(xs, rw, bias, d, ne, top_k, lg, esel, wsel);
  if (threadIdx.x < top_k) {
    idx_out[b * top_k + threadIdx.x] = esel[threadIdx.x];
    w_out[b * top_k + threadIdx.x] = wsel[threadIdx.x];
  }
}

// grid (ceil(E / rows per block), B * slots).  idx == nullptr: dense feed-forward (one "expert" 0).
template <int FMT, int KS, typename XT>
__global__ void __launch_bounds__(GV_THREADS) swiglu_norm_kernel(
    const uint8_t* __restrict__ Wg, const uint8_t* __restrict__ Wu, long long row_bytes, int ne, int E, int d,
    const float* __restrict__ x32, const float* __restrict__ norm_w, float eps, const int* __restrict__ idx, int top_k,
    int slots, XT* __restrict__ act) {
  pdl_wait();
  extern __shared__ __align__(16) uint8_t gv_dyn[];
  XT* xs = reinterpret_cast<XT*>(gv_dyn);                 // [d]
  __shared__ float sm[2 * GV_WARPS];
  const int warp = threadIdx.x >> 5, ric = warp / KS, ks = warp % KS;
  const int b = blockIdx.y / slots, slot = blockIdx.y % slots;
  if (warp == 0) norm_row_to_smem<XT>(x32 + (long long)b * d, norm_w, xs, d, eps);
  __syncthreads();
  const int e = idx ? (slot < top_k ? idx[b * top_k + slot] : ne) : 0;
  const int j = blockIdx.x * (GV_WARPS / KS) + ric;
  const bool live = j < E && e >= 0 && e <= ne;
  float g[1] = {0.f}, u[1] = {0.f};
  if (live) {
    const size_t r = (size_t)e * E + j;
    row_partial<FMT, 1, KS, XT>(Wg + r * row_bytes, d, xs, d, 1, ks, g);
    row_partial<FMT, 1, KS, XT>(Wu + r * row_bytes, d, xs, d, 1, ks, u);
  }
  const float gs = row_finish<KS>(g[0], sm, ric, ks);
  const float us = row_finish<KS>(u[0], sm + GV_WARPS, ric, ks);
  if (live && ks == 0 && (threadIdx.x & 31) == 0)
    act[((long long)b * slots + slot) * E + j] = Cvt<XT>::from_f(gs / (1.f + __expf(-gs)) * us);
}

// One warp per (sequence, head) over the q, k and v heads of the fused projection.  q heads: norm + rotation into
// `q_out`.  k heads: norm + rotation straight into the cache slot of the step.  v heads: copied into the cache.
template <typename T, int HD>
__global__ void qk_rope_append_kernel(const T* __restrict__ qkv, long long ld_in, T* __restrict__ q_out, long long ld_q,
                                      const float* __restrict__ qw, const float* __restrict__ kw, const float* __restrict__ cs,
                                      const int* __restrict__ pos, T* __restrict__ cK, T* __restrict__ cV,
                                      int* __restrict__ slot_pos, const gb_seq_state* __restrict__ st, int B, int H, int KV,
                                      int cap, int pinned, float eps, int rope_type) {
  pdl_wait();
  constexpr int PAIRS = HD / 2;
  constexpr int PPL = (PAIRS + 31) / 32;
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = H + 2 * KV;
  if (gw >= B * heads) return;
  const int b = gw / heads, h = gw - b * heads;
  const gb_seq_state s = st[b];
  const int slot = s.cache_len < cap ? s.cache_len : pinned + s.ring_start;
  const long long kvd = (long long)KV * HD;
  const T* src = qkv + b * ld_in + (long long)h * HD;
  if (h >= H + KV) {                                         // v head: plain copy into the cache
    T* dv = cV + ((long long)b * cap + slot) * kvd + (long long)(h - H - KV) * HD;
    for (int i = lane * 2; i < HD; i += 64) *reinterpret_cast<uint32_t*>(dv + i) = *reinterpret_cast<const uint32_t*>(src + i);
    return;
  }
  T* dst = h < H ? q_out + b * ld_q + (long long)h * HD : cK + ((long long)b * cap + slot) * kvd + (long long)(h - H) * HD;
  if (h == H && lane == 0) slot_pos[(long long)b * cap + slot] = s.abs_pos;
  const float* w = (h < H) ? qw : kw;
  float a[PPL], c2[PPL];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PPL; ++k) {
    const int p = lane + 32 * k;
    if (p < PAIRS) {
      const int i0 = rope_type == 0 ? 2 * p : p, i1 = rope_type == 0 ? 2 * p + 1 : p + PAIRS;
      a[k] = Cvt<T>::to_f(src[i0]);
      c2[k] = Cvt<T>::to_f(src[i1]);
      ss += a[k] * a[k] + c2[k] * c2[k];
    }
  }
  float inv = 1.f;
  if (w) {
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)HD + eps);
    if (!isfinite(inv)) inv = 0.f;
  }
  const float* csr = cs + (size_t)pos[b] * HD;
#pragma unroll
  for (int k = 0; k < PPL; ++k) {
    const int p = lane + 32 * k;
    if (p < PAIRS) {
      const int i0 = rope_type == 0 ? 2 * p : p, i1 = rope_type == 0 ? 2 * p + 1 : p + PAIRS;
      float x0 = a[k], x1 = c2[k];
      if (w) { x0 *= inv * w[i0]; x1 *= inv * w[i1]; }
      const float c = csr[p], sn = csr[PAIRS + p];
      dst[i0] = Cvt<T>::from_f(x0 * c - x1 * sn);
      dst[i1] = Cvt<T>::from_f(x0 * sn + x1 * c);
    }
  }
}

}  // namespace gb

using namespace gb;

extern "C" long long gb_wfmt_row_bytes(int fmt, int K) {
  switch (fmt) {
    case GB_W_F16: case GB_W_BF16: return K % 8 ? -1 : 2LL * K;
    case GB_W_GGML_Q8_0: return K % 32 ? -1 : (K / 32) * 34LL;
    case GB_W_Q4_0: return K % 32 ? -1 : (K / 32) * 18LL;
    case GB_W_Q8_64: return K % 64 ? -1 : (K / 64) * 68LL;
    case GB_W_Q4_1: return K % 32 ? -1 : (K / 32) * 20LL;
  }
  return -1;
}

#define GB_FMT_SWITCH(fmt, CALL)                          \
  switch (fmt) {                                          \
    case GB_W_F16: { CALL(GB_W_F16); break; }             \
    case GB_W_BF16: { CALL(GB_W_BF16); break; }           \
    case GB_W_GGML_Q8_0: { CALL(GB_W_GGML_Q8_0); break; } \
    case GB_W_Q4_0: { CALL(GB_W_Q4_0); break; }           \
    case GB_W_Q8_64: { CALL(GB_W_Q8_64); break; }         \
    case GB_W_Q4_1: { CALL(GB_W_Q4_1); break; }           \
    default: return -1;                                   \
  }

extern "C" int gb_gemv(const void* W, int fmt, int N, int K, const void* x16, int ldx, int B, void* out, int ldo, int out_f32,
                       const float* addend, int ld_add, int is_bf16, cudaStream_t st) {
  const long long rb = gb_wfmt_row_bytes(fmt, K);
  if (!W || !x16 || !out || N <= 0 || B <= 0 || B > 32 || rb < 0 || (ldx % 8)) return -1;
  const bool split = N <= 8192;   // few rows: spread each over four warps (latency bound); many rows fill the GPU anyway
  const uint8_t* w = static_cast<const uint8_t*>(W);
#define GEMV_GO(F, NB, KS, XT)                                                                                     \
  GB_PDL_LAUNCH((gemv_kernel<F, NB, KS, XT>), dim3((N + GV_WARPS / KS - 1) / (GV_WARPS / KS)), dim3(GV_THREADS), st, \
                w, rb, N, K, (const XT*)x16, (long long)ldx, B, out, (long long)ldo, out_f32, addend, (long long)ld_add)
#define CALL(F)                                                                        \
  if (is_bf16) {                                                                       \
    if (B == 1 && split) GEMV_GO(F, 1, 4, __nv_bfloat16);                              \
    else if (B == 1) GEMV_GO(F, 1, 1, __nv_bfloat16);                                  \
    else GEMV_GO(F, 4, 1, __nv_bfloat16);                                              \
  } else {                                                                             \
    if (B == 1 && split) GEMV_GO(F, 1, 4, __half);                                     \
    else if (B == 1) GEMV_GO(F, 1, 1, __half);                                         \
    else GEMV_GO(F, 4, 1, __half);                                                     \
  }
  GB_FMT_SWITCH(fmt, CALL)
#undef CALL
#undef GEMV_GO
  return gb_launch_rc();
}

extern "C" int gb_gemv_expert_swiglu(const void* Wg, const void* Wu, int fmt, int ne, int E, int d, const void* x16, int B,
                                     const int* idx, int top_k, int shared, void* act16, int is_bf16, cudaStream_t st) {
  const long long rb = gb_wfmt_row_bytes(fmt, d);
  if (!Wg || !Wu || !x16 || !idx || !act16 || rb < 0 || B <= 0 || top_k <= 0) return -1;
  const int slots = top_k + (shared ? 1 : 0);
  const uint8_t *g = static_cast<const uint8_t*>(Wg), *u = static_cast<const uint8_t*>(Wu);
  const bool split = B * slots <= 64;
#define SW_GO(F, KS, XT)                                                                                              \
  GB_PDL_LAUNCH((expert_swiglu_kernel<F, KS, XT>), dim3((E + GV_WARPS / KS - 1) / (GV_WARPS / KS), B * slots),       \
                dim3(GV_THREADS), st, g, u, rb, ne, E, d, (const XT*)x16, idx, top_k, slots, (XT*)act16)
#define CALL(F)                                                                                   \
  if (is_bf16) { if (split) SW_GO(F, 4, __nv_bfloat16); else SW_GO(F, 1, __nv_bfloat16); }        \
  else { if (split) SW_GO(F, 4, __half); else SW_GO(F, 1, __half); }
  GB_FMT_SWITCH(fmt, CALL)
#undef CALL
  return gb_launch_rc();
}

extern "C" int gb_gemv_expert_down(const void* Wd, int fmt, int ne, int d, int E, const void* act16, int B, const int* idx,
                                   const float* w, int top_k, int shared, const float* resid, float* out, int is_bf16,
                                   cudaStream_t st) {
  const long long rb = gb_wfmt_row_bytes(fmt, E);
  if (!Wd || !act16 || !idx || !w || !resid || !out || rb < 0 || B <= 0 || top_k <= 0) return -1;
  const int slots = top_k + (shared ? 1 : 0);
  const uint8_t* wd = static_cast<const uint8_t*>(Wd);
  const bool split = B <= 16;
#define DN_GO(F, KS, XT)                                                                                    \
  GB_PDL_LAUNCH((expert_down_kernel<F, KS, XT>), dim3((d + GV_WARPS / KS - 1) / (GV_WARPS / KS), B), dim3(GV_THREADS), st, \
                wd, rb, ne, d, E, (const XT*)act16, idx, w, top_k, slots, resid, out)
#define CALL(F)                                                                                   \
  if (is_bf16) { if (split) DN_GO(F, 4, __nv_bfloat16); else DN_GO(F, 1, __nv_bfloat16); }        \
  else { if (split) DN_GO(F, 4, __half); else DN_GO(F, 1, __half); }
  GB_FMT_SWITCH(fmt, CALL)
#undef CALL
  return gb_launch_rc();
}

extern "C" int gb_decode_route(const void* x16, const float* router_w, const float* bias, int B, int d, int ne, int top_k,
                               int* idx, float* w, int is_bf16, cudaStream_t st) {
  if (!x16 || !router_w || !idx || !w || B <= 0 || ne <= 0 || ne > 64 || top_k <= 0 || top_k > 8 || top_k > ne || d % 2) return -1;
  if (is_bf16) GB_PDL_LAUNCH(decode_route_kernel<__nv_bfloat16>, dim3(B), dim3(256), st, (const __nv_bfloat16*)x16, router_w, bias, d, ne, top_k, idx, w);
  else GB_PDL_LAUNCH(decode_route_kernel<__half>, dim3(B), dim3(256), st, (const __half*)x16, router_w, bias, d, ne, top_k, idx, w);
  return gb_launch_rc();
}

extern "C" int gb_kv_append(const void* k16, long long ld_k, const void* v16, long long ld_v, void* cacheK, void* cacheV,
                            int* slot_pos, const gb_seq_state* state, int B, int cap, int pinned, int kv_dim, cudaStream_t st) {
  if (!k16 || !v16 || !cacheK || !cacheV || !slot_pos || !state || B <= 0 || cap <= pinned || kv_dim % 8 || ld_k % 8 || ld_v % 8)
    return -1;
  // 16-bit elements of either type are copied as raw bits
  GB_PDL_LAUNCH(kv_append_kernel<__half>, dim3(B), dim3(128), st, (const __half*)k16, ld_k, (const __half*)v16, ld_v, (__half*)cacheK,
                                              (__half*)cacheV, slot_pos, state, cap, pinned, kv_dim);
  return gb_launch_rc();
}

extern "C" int gb_decode_advance(gb_seq_state* state, int* pos_out, int B, int cap, int pinned, cudaStream_t st) {
  if (!state || !pos_out || B <= 0) return -1;
  GB_PDL_LAUNCH(decode_advance_kernel, dim3((B + 63) / 64), dim3(64), st, state, pos_out, B, cap, pinned);
  return gb_launch_rc();
}

template <typename T, int HD>
static int launch_decode_attn(const void* q, long long ld_q, const void* cK, const void* cV, const int* slot_pos,
                              const gb_seq_state* state, void* out, long long ld_o, float* scratch, int splits, int B, int H,
                              int KV, int cap, int window, float scale, int* ticket, cudaStream_t st) {
  const int G = H / KV;
  if (!ticket && splits > 2 * HD) return -4;      // the merge kernel reads at most two splits per thread
  const dim3 grid(B * KV, splits);
#define ATT(GG)                                                                                                   \
  GB_PDL_LAUNCH((decode_attn_kernel<T, HD, GG>), grid, dim3(128), st, (const T*)q, ld_q, (const T*)cK, (const T*)cV, slot_pos, \
                state, scratch, splits, H, KV, cap, window, scale, ticket, (T*)out, ld_o)
  switch (G) {
    case 1: ATT(1); break;
    case 2: ATT(2); break;
    case 3: ATT(3); break;
    case 4: ATT(4); break;
    case 6: ATT(6); break;
    case 8: ATT(8); break;
    default: return -3;
  }
#undef ATT
  if (!ticket) GB_PDL_LAUNCH((decode_attn_merge_kernel<T, HD>), dim3(B * H), dim3(HD), st, (const float*)scratch, splits, (T*)out, ld_o, H);
  return gb_launch_rc();
}

static int decode_attn_any(const void* q16, long long ld_q, const void* cacheK, const void* cacheV, const int* slot_pos,
                           const gb_seq_state* state, void* out16, long long ld_o, float* scratch, int splits, int B, int H,
                           int KV, int hd, int cap, int window, float scale, int is_bf16, int* ticket, cudaStream_t st) {
  if (!q16 || !cacheK || !cacheV || !slot_pos || !state || !out16 || !scratch || splits < 1 || B <= 0 || KV <= 0 || H % KV)
    return -1;
#define GO(T, HD) return launch_decode_attn<T, HD>(q16, ld_q, cacheK, cacheV, slot_pos, state, out16, ld_o, scratch, splits, B, H, KV, cap, window, scale, ticket, st)
  if (hd == 64) { if (is_bf16) GO(__nv_bfloat16, 64); else GO(__half, 64); }
  if (hd == 128) { if (is_bf16) GO(__nv_bfloat16, 128); else GO(__half, 128); }
  if (hd == 32) { if (is_bf16) GO(__nv_bfloat16, 32); else GO(__half, 32); }
#undef GO
  return -2;
}

extern "C" int gb_decode_attn(const void* q16, long long ld_q, const void* cacheK, const void* cacheV, const int* slot_pos,
                              const gb_seq_state* state, void* out16, long long ld_o, float* scratch, int splits, int B, int H,
                              int KV, int hd, int cap, int window, float scale, int is_bf16, cudaStream_t st) {
  return decode_attn_any(q16, ld_q, cacheK, cacheV, slot_pos, state, out16, ld_o, scratch, splits, B, H, KV, hd, cap, window,
                         scale, is_bf16, nullptr, st);
}

// The same with the merge of the splits done by the last block to finish; `ticket` is B*KV ints, zero before the first call.
extern "C" int gb_decode_attn_fused(const void* q16, long long ld_q, const void* cacheK, const void* cacheV, const int* slot_pos,
                                    const gb_seq_state* state, void* out16, long long ld_o, float* scratch, int splits, int B,
                                    int H, int KV, int hd, int cap, int window, float scale, int is_bf16, int* ticket,
                                    cudaStream_t st) {
  if (!ticket) return -1;
  return decode_attn_any(q16, ld_q, cacheK, cacheV, slot_pos, state, out16, ld_o, scratch, splits, B, H, KV, hd, cap, window,
                         scale, is_bf16, ticket, st);
}

// RMSNorm of x32 [B, K] (fp32) fused into out = W @ norm(x32).  Shared memory holds the normalised rows: B*K*2 bytes.
extern "C" int gb_gemv_norm(const void* W, int fmt, int N, int K, const float* x32, int ldx32, const float* norm_w, float eps,
                            int B, void* out, int ldo, int out_f32, int is_bf16, cudaStream_t st) {
  const long long rb = gb_wfmt_row_bytes(fmt, K);
  if (!W || !x32 || !norm_w || !out || N <= 0 || B <= 0 || B > 32 || rb < 0 || (K % 8) || (ldx32 % 4)) return -1;
  const size_t smem = (size_t)B * K * 2;
  if (smem > 40 * 1024) return -2;                          // the caller takes the two-kernel route
  const bool split = N <= 8192;
  const uint8_t* w = static_cast<const uint8_t*>(W);
#define GEMVN_GO(F, NB, KS, XT)                                                                                      \
  do {                                                                                                               \
    cudaLaunchAttribute gb_attr_;                                                                                    \
    cudaLaunchConfig_t gb_cfg_ = gb_pdl_config(dim3((N + GV_WARPS / KS - 1) / (GV_WARPS / KS)), dim3(GV_THREADS), smem, st, &gb_attr_); \
    (void)cudaLaunchKernelEx(&gb_cfg_, (gemv_norm_kernel<F, NB, KS, XT>), w, rb, N, K, x32, (long long)ldx32, norm_w, eps, B, \
                             out, (long long)ldo, out_f32);                                                          \
  } while (0)
#define CALL(F)                                                                         \
  if (is_bf16) {                                                                        \
    if (B == 1 && split) GEMVN_GO(F, 1, 4, __nv_bfloat16);                              \
    else if (B == 1) GEMVN_GO(F, 1, 1, __nv_bfloat16);                                  \
    else GEMVN_GO(F, 4, 1, __nv_bfloat16);                                              \
  } else {                                                                              \
    if (B == 1 && split) GEMVN_GO(F, 1, 4, __half);                                     \
    else if (B == 1) GEMVN_GO(F, 1, 1, __half);                                         \
    else GEMVN_GO(F, 4, 1, __half);                                                     \
  }
  GB_FMT_SWITCH(fmt, CALL)
#undef CALL
#undef GEMVN_GO
  return gb_launch_rc();
}

// RMSNorm + router of x32 [B, d]: idx_out / w_out [B, top_k].
extern "C" int gb_route_norm(const float* x32, const float* norm_w, float eps, const float* router_w, const float* bias, int B,
                             int d, int ne, int top_k, int* idx_out, float* w_out, int is_bf16, cudaStream_t st) {
  if (!x32 || !norm_w || !router_w || !idx_out || !w_out || B <= 0 || ne <= 0 || ne > 64 || top_k <= 0 || top_k > 8 ||
      top_k > ne || (d % 8))
    return -1;
  const size_t smem = (size_t)d * 2;
  if (smem > 40 * 1024) return -2;
  cudaLaunchAttribute attr;
  cudaLaunchConfig_t cfg = gb_pdl_config(dim3(B), dim3(GV_THREADS), smem, st, &attr);
  if (is_bf16) (void)cudaLaunchKernelEx(&cfg, route_norm_kernel<__nv_bfloat16>, x32, norm_w, eps, router_w, bias, d, ne, top_k, idx_out, w_out);
  else (void)cudaLaunchKernelEx(&cfg, route_norm_kernel<__half>, x32, norm_w, eps, router_w, bias, d, ne, top_k, idx_out, w_out);
  return gb_launch_rc();
}

// RMSNorm + gate/up of the experts named by idx [B, top_k] (+ the shared one).  idx == nullptr: dense feed-forward.
extern "C" int gb_swiglu_norm(const void* Wg, const void* Wu, int fmt, int ne, int E, int d, const float* x32, const float* norm_w,
                              float eps, const int* idx, int B, int top_k, int shared, void* act16, int is_bf16,
                              cudaStream_t st) {
  const long long rb = gb_wfmt_row_bytes(fmt, d);
  if (!Wg || !Wu || !x32 || !norm_w || !act16 || rb < 0 || B <= 0 || top_k <= 0 || top_k > 8 || (d % 8)) return -1;
  const size_t smem = (size_t)d * 2;
  if (smem > 40 * 1024) return -2;
  const int slots = top_k + (shared ? 1 : 0);
  const uint8_t *g = static_cast<const uint8_t*>(Wg), *u = static_cast<const uint8_t*>(Wu);
  const bool split = B * slots <= 64;
#define SWN_GO(F, KS, XT)                                                                                            \
  do {                                                                                                               \
    cudaLaunchAttribute gb_attr_;                                                                                    \
    cudaLaunchConfig_t gb_cfg_ = gb_pdl_config(dim3((E + GV_WARPS / KS - 1) / (GV_WARPS / KS), B * slots), dim3(GV_THREADS), smem, st, &gb_attr_); \
    (void)cudaLaunchKernelEx(&gb_cfg_, (swiglu_norm_kernel<F, KS, XT>), g, u, rb, ne, E, d, x32, norm_w, eps, idx, top_k, slots, \
                             (XT*)act16);                                                                            \
  } while (0)
#define CALL(F)                                                                                     \
  if (is_bf16) { if (split) SWN_GO(F, 4, __nv_bfloat16); else SWN_GO(F, 1, __nv_bfloat16); }        \
  else { if (split) SWN_GO(F, 4, __half); else SWN_GO(F, 1, __half); }
  GB_FMT_SWITCH(fmt, CALL)
#undef CALL
#undef SWN_GO
  return gb_launch_rc();
}

extern "C" int gb_qk_rope_append(const void* qkv, long long ld_in, void* q_out, long long ld_q, const float* qw, const float* kw,
                                 const float* cos_sin, const int* pos, void* cacheK, void* cacheV, int* slot_pos,
                                 const gb_seq_state* state, int B, int H, int KV, int hd, int cap, int pinned, float eps,
                                 int rope_type, int is_bf16, cudaStream_t st) {
  if (!qkv || !q_out || !cos_sin || !pos || !cacheK || !cacheV || !slot_pos || !state || B <= 0 || H <= 0 || KV <= 0 ||
      cap <= pinned || (hd % 2) || (ld_in % 2))
    return -1;
  const int items = B * (H + 2 * KV);
  const int wpb = 8;
  const dim3 grid((items + wpb - 1) / wpb);
#define QKA(T, HD)                                                                                                       \
  GB_PDL_LAUNCH((qk_rope_append_kernel<T, HD>), grid, dim3(wpb * 32), st, (const T*)qkv, ld_in, (T*)q_out, ld_q, qw, kw, cos_sin, \
                pos, (T*)cacheK, (T*)cacheV, slot_pos, state, B, H, KV, cap, pinned, eps, rope_type)
  if (is_bf16) {
    switch (hd) { case 32: QKA(__nv_bfloat16, 32); break; case 64: QKA(__nv_bfloat16, 64); break; case 128: QKA(__nv_bfloat16, 128); break; default: return -2; }
  } else {
    switch (hd) { case 32: QKA(__half, 32); break; case 64: QKA(__half, 64); break; case 128: QKA(__half, 128); break; default: return -2; }
  }
#undef QKA
  return gb_launch_rc();
}
