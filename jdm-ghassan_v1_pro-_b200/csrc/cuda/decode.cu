// Decode-time kernels (contract in gb_decode.h).  Batch-1 decoding reads every active weight once per token and
// does two flops per weight: it is bound by HBM bandwidth and launch count, not by the tensor cores.  So weights
// stay in their storage format (fp16 / bf16 / 8-bit / 4-bit blocks) and are expanded in registers inside the dot
// product; one warp owns one output row, lanes stride over 8-value units of the row, partial sums are fp32.
#include <type_traits>

#include "sm100_common.cuh"
#include "gb_decode.h"

namespace gb {

constexpr int GV_WARPS = 8;            // output rows per CTA
constexpr int GV_THREADS = GV_WARPS * 32;

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t ld_u16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }

// Expand unit u (values 8u .. 8u+7) of one stored row into floats.
template <int FMT>
__device__ __forceinline__ void load8(const uint8_t* __restrict__ row, int u, float (&w)[8]) {
  if constexpr (FMT == GB_W_F16) {
    const uint4 q = *reinterpret_cast<const uint4*>(row + 16 * (size_t)u);
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); w[2 * i] = f.x; w[2 * i + 1] = f.y; }
  } else if constexpr (FMT == GB_W_BF16) {
    const uint4 q = *reinterpret_cast<const uint4*>(row + 16 * (size_t)u);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); w[2 * i] = f.x; w[2 * i + 1] = f.y; }
  } else if constexpr (FMT == GB_W_GGML_Q8_0) {
    const uint8_t* p = row + (size_t)(u >> 2) * 34;
    const float d = h2f(ld_u16(p));
    const uint8_t* q = p + 2 + (u & 3) * 8;           // 2-byte aligned: blocks are 34 bytes
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint16_t v = ld_u16(q + 2 * i);
      w[2 * i] = d * (float)(int8_t)(v & 0xFF);
      w[2 * i + 1] = d * (float)(int8_t)(v >> 8);
    }
  } else if constexpr (FMT == GB_W_Q4_0) {
    const uint8_t* p = row + (size_t)(u >> 2) * 18;
    const float d = h2f(ld_u16(p));
    const uint8_t* q = p + 2 + (u & 3) * 4;
    const uint32_t v = (uint32_t)ld_u16(q) | ((uint32_t)ld_u16(q + 2) << 16);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = d * (float)((int)((v >> (4 * i)) & 0xF) - 8);   // byte i: low nibble = value 2i
  } else if constexpr (FMT == GB_W_Q8_64) {
    const uint8_t* p = row + (size_t)(u >> 3) * 68;
    const float d = *reinterpret_cast<const float*>(p);
    // blocks are 68 bytes: the quants are 4-byte aligned but not 8-byte aligned, so two 32-bit loads
    const uint32_t* qp = reinterpret_cast<const uint32_t*>(p + 4 + (u & 7) * 8);
    const uint32_t vx = qp[0], vy = qp[1];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[i] = d * (float)(int8_t)((vx >> (8 * i)) & 0xFF);
      w[4 + i] = d * (float)(int8_t)((vy >> (8 * i)) & 0xFF);
    }
  } else {   // GB_W_Q4_1
    const uint8_t* p = row + (size_t)(u >> 2) * 20;
    const float d = h2f(ld_u16(p)), m = h2f(ld_u16(p + 2));
    const uint32_t v = *reinterpret_cast<const uint32_t*>(p + 4 + (u & 3) * 4);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = d * (float)((v >> (4 * i)) & 0xF) + m;
  }
}

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
                                                         int splits, int H, int KV, int cap, int window, float scale) {
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
}

template <typename T, int HD>
__global__ void decode_attn_merge_kernel(const float* __restrict__ scratch, int splits, T* __restrict__ out, long long ld_o, int H) {
  const int b = blockIdx.x / H, h = blockIdx.x % H, c = threadIdx.x;
  const float* base = scratch + ((long long)b * H + h) * splits * (HD + 2);
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, base[s * (HD + 2)]);
  float ll = 0.f, oo = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = base[s * (HD + 2)];
    const float f = ms == -INFINITY ? 0.f : __expf(ms - mm);
    ll += base[s * (HD + 2) + 1] * f;
    oo += base[s * (HD + 2) + 2 + c] * f;
  }
  out[b * ld_o + (long long)h * HD + c] = Cvt<T>::from_f(ll > 0.f ? oo / ll : 0.f);
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
  gemv_kernel<F, NB, KS, XT><<<dim3((N + GV_WARPS / KS - 1) / (GV_WARPS / KS)), GV_THREADS, 0, st>>>(                 \
      w, rb, N, K, (const XT*)x16, ldx, B, out, ldo, out_f32, addend, ld_add)
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
  expert_swiglu_kernel<F, KS, XT><<<dim3((E + GV_WARPS / KS - 1) / (GV_WARPS / KS), B * slots), GV_THREADS, 0, st>>>( \
      g, u, rb, ne, E, d, (const XT*)x16, idx, top_k, slots, (XT*)act16)
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
  expert_down_kernel<F, KS, XT><<<dim3((d + GV_WARPS / KS - 1) / (GV_WARPS / KS), B), GV_THREADS, 0, st>>>( \
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
  if (is_bf16) decode_route_kernel<__nv_bfloat16><<<B, 256, 0, st>>>((const __nv_bfloat16*)x16, router_w, bias, d, ne, top_k, idx, w);
  else decode_route_kernel<__half><<<B, 256, 0, st>>>((const __half*)x16, router_w, bias, d, ne, top_k, idx, w);
  return gb_launch_rc();
}

extern "C" int gb_kv_append(const void* k16, long long ld_k, const void* v16, long long ld_v, void* cacheK, void* cacheV,
                            int* slot_pos, const gb_seq_state* state, int B, int cap, int pinned, int kv_dim, cudaStream_t st) {
  if (!k16 || !v16 || !cacheK || !cacheV || !slot_pos || !state || B <= 0 || cap <= pinned || kv_dim % 8 || ld_k % 8 || ld_v % 8)
    return -1;
  // 16-bit elements of either type are copied as raw bits
  kv_append_kernel<__half><<<B, 128, 0, st>>>((const __half*)k16, ld_k, (const __half*)v16, ld_v, (__half*)cacheK,
                                              (__half*)cacheV, slot_pos, state, cap, pinned, kv_dim);
  return gb_launch_rc();
}

extern "C" int gb_decode_advance(gb_seq_state* state, int* pos_out, int B, int cap, int pinned, cudaStream_t st) {
  if (!state || !pos_out || B <= 0) return -1;
  decode_advance_kernel<<<(B + 63) / 64, 64, 0, st>>>(state, pos_out, B, cap, pinned);
  return gb_launch_rc();
}

template <typename T, int HD>
static int launch_decode_attn(const void* q, long long ld_q, const void* cK, const void* cV, const int* slot_pos,
                              const gb_seq_state* state, void* out, long long ld_o, float* scratch, int splits, int B, int H,
                              int KV, int cap, int window, float scale, cudaStream_t st) {
  const int G = H / KV;
  const dim3 grid(B * KV, splits);
#define ATT(GG)                                                                                                   \
  decode_attn_kernel<T, HD, GG><<<grid, 128, 0, st>>>((const T*)q, ld_q, (const T*)cK, (const T*)cV, slot_pos, state, \
                                                      scratch, splits, H, KV, cap, window, scale)
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
  decode_attn_merge_kernel<T, HD><<<B * H, HD, 0, st>>>(scratch, splits, (T*)out, ld_o, H);
  return gb_launch_rc();
}

extern "C" int gb_decode_attn(const void* q16, long long ld_q, const void* cacheK, const void* cacheV, const int* slot_pos,
                              const gb_seq_state* state, void* out16, long long ld_o, float* scratch, int splits, int B, int H,
                              int KV, int hd, int cap, int window, float scale, int is_bf16, cudaStream_t st) {
  if (!q16 || !cacheK || !cacheV || !slot_pos || !state || !out16 || !scratch || splits < 1 || B <= 0 || KV <= 0 || H % KV)
    return -1;
#define GO(T, HD) return launch_decode_attn<T, HD>(q16, ld_q, cacheK, cacheV, slot_pos, state, out16, ld_o, scratch, splits, B, H, KV, cap, window, scale, st)
  if (hd == 64) { if (is_bf16) GO(__nv_bfloat16, 64); else GO(__half, 64); }
  if (hd == 128) { if (is_bf16) GO(__nv_bfloat16, 128); else GO(__half, 128); }
  if (hd == 32) { if (is_bf16) GO(__nv_bfloat16, 32); else GO(__half, 32); }
#undef GO
  return -2;
}
