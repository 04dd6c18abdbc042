// Causal flash attention (forward + backward) on CUDA cores: online softmax, no T x T buffer, GQA,
// sliding window, packed-sequence segment mask, fully-masked rows -> 0.  This is the portable path used
// for every head size; it never materialises scores and its backward recomputes them from the saved
// log-sum-exp, unlike the reference's grouped-GEMM + softmax + grouped-GEMM pipeline that stores
// B*H*T^2 floats and runs the forward twice (cuda/attention.cu:297-550, 805-898 in the reference).
//
// Work split: TPR threads own one query (or key) row and HD/TPR of its head dims each; K/V (or Q/dO)
// tiles of KT rows are staged in shared memory as fp32 and broadcast to all rows of the block.
// Masks: key j is visible to query i iff j <= i, (window == 0 or j > i - window) and
// (no segments, or seg[i] < 0, or seg[j] == seg[i]).
#include "sm100_common.cuh"
#include "gb_api.h"

namespace gb {

template <int TPR>
__device__ __forceinline__ float row_sum(float v) {
#pragma unroll
  for (int o = TPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
__device__ __forceinline__ void stage_tile(const T* __restrict__ base, long long ld, int row0, int nrows, int T_len,
                                           int hd, float* __restrict__ dst) {
  // dst[r*hd + c] = base[(row0+r)*ld + c] (zero beyond T_len); 8 elements per step
  const int per_row = hd / 8;
  for (int idx = threadIdx.x; idx < nrows * per_row; idx += blockDim.x) {
    const int r = idx / per_row, c = (idx - r * per_row) * 8;
    float f[8];
    if (row0 + r < T_len) {
      uint4 q = *reinterpret_cast<const uint4*>(base + (long long)(row0 + r) * ld + c);
      float2 a = Cvt<T>::unpack2(q.x), b = Cvt<T>::unpack2(q.y), cc = Cvt<T>::unpack2(q.z), d = Cvt<T>::unpack2(q.w);
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = cc.x; f[5] = cc.y; f[6] = d.x; f[7] = d.y;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = 0.f;
    }
    float4* o = reinterpret_cast<float4*>(dst + r * hd + c);
    o[0] = make_float4(f[0], f[1], f[2], f[3]);
    o[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
}

struct AttnArgs {
  const void* q; long long ld_q;
  const void* k; long long ld_k;
  const void* v; long long ld_v;
  void* o; long long ld_o;
  float* lse;            // [B*T, H]
  const int* seg;        // [B*T] or null
  int B, T, H, KV, window;
  float scale;
  // backward
  const void* d_o; long long ld_do;
  float* delta;          // [B*T, H]
  void* dq; long long ld_dq;
  void* dk; long long ld_dk;
  void* dv; long long ld_dv;
};

__device__ __forceinline__ bool visible(int i, int j, int window, int seg_i, int seg_j, bool has_seg) {
  if (j > i) return false;
  if (window > 0 && j <= i - window) return false;
  if (has_seg && seg_i >= 0 && seg_j != seg_i) return false;
  return true;
}

// ----------------------------------------------------------------------------------------- forward
template <typename T, int HD, int TPR, int KT>
__global__ void __launch_bounds__(128) attn_fwd_kernel(const AttnArgs a) {
  constexpr int HDT = HD / TPR;
  constexpr int ROWS = 128 / TPR;
  extern __shared__ float smem[];
  float* sK = smem;
  float* sV = smem + KT * HD;
  int* sSeg = reinterpret_cast<int*>(sV + KT * HD);
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * ROWS;
  const int kvh = h / (a.H / a.KV);
  const int r = threadIdx.x / TPR, sub = threadIdx.x % TPR;
  const int i = q0 + r;
  const bool row_ok = i < a.T;
  const long long tok = (long long)b * a.T + i;
  const bool has_seg = a.seg != nullptr;
  const int seg_i = (has_seg && row_ok) ? a.seg[tok] : 0;

  float q[HDT], o[HDT];
#pragma unroll
  for (int d = 0; d < HDT; ++d) { q[d] = 0.f; o[d] = 0.f; }
  if (row_ok) {
    const T* qp = reinterpret_cast<const T*>(a.q) + tok * a.ld_q + (long long)h * HD + sub * HDT;
#pragma unroll
    for (int d = 0; d < HDT; ++d) q[d] = Cvt<T>::to_f(qp[d]) * a.scale;
  }
  float m = -INFINITY, l = 0.f;

  const int i_last = min(a.T, q0 + ROWS) - 1;
  const int j_hi = i_last + 1;
  int j_lo = 0;
  if (a.window > 0) j_lo = max(0, q0 - a.window + 1);
  j_lo = (j_lo / KT) * KT;
  const T* kb = reinterpret_cast<const T*>(a.k) + (long long)b * a.T * a.ld_k + (long long)kvh * HD;
  const T* vb = reinterpret_cast<const T*>(a.v) + (long long)b * a.T * a.ld_v + (long long)kvh * HD;

  for (int j0 = j_lo; j0 < j_hi; j0 += KT) {
    __syncthreads();
    stage_tile<T>(kb, a.ld_k, j0, KT, a.T, HD, sK);
    stage_tile<T>(vb, a.ld_v, j0, KT, a.T, HD, sV);
    if (has_seg)
      for (int t = threadIdx.x; t < KT; t += blockDim.x) sSeg[t] = (j0 + t < a.T) ? a.seg[(long long)b * a.T + j0 + t] : -2;
    __syncthreads();
    const int jn = min(KT, j_hi - j0);  // uniform over the block: every lane takes part in the row reductions
    for (int jj = 0; jj < jn; ++jj) {
      const int j = j0 + jj;
      const float* kr = sK + jj * HD + sub * HDT;
      float s = 0.f;
#pragma unroll
      for (int d = 0; d < HDT; ++d) s += q[d] * kr[d];
      s = row_sum<TPR>(s);
      if (!row_ok || !visible(i, j, a.window, seg_i, has_seg ? sSeg[jj] : 0, has_seg)) continue;
      const float m_new = fmaxf(m, s);
      const float corr = __expf(m - m_new);
      const float p = __expf(s - m_new);
      l = l * corr + p;
      const float* vr = sV + jj * HD + sub * HDT;
#pragma unroll
      for (int d = 0; d < HDT; ++d) o[d] = o[d] * corr + p * vr[d];
      m = m_new;
    }
  }
  if (!row_ok) return;
  const float inv_l = l > 0.f ? 1.f / l : 0.f;
  T* op = reinterpret_cast<T*>(a.o) + tok * a.ld_o + (long long)h * HD + sub * HDT;
#pragma unroll
  for (int d = 0; d < HDT; ++d) op[d] = Cvt<T>::from_f(o[d] * inv_l);
  // a fully masked row stores +inf so that exp(s - lse) is 0 in the backward pass
  if (sub == 0 && a.lse) a.lse[tok * a.H + h] = l > 0.f ? m + __logf(l) : INFINITY;
}

// ----------------------------------------------------------------------------------------- backward
// delta[i,h] = sum_d dO[i,h,d] * O[i,h,d]; one warp per (token, head)
template <typename T>
__global__ void attn_delta_kernel(const T* __restrict__ d_o, long long ld_do, const T* __restrict__ o, long long ld_o,
                                  float* __restrict__ delta, long long n_tok, int H, int hd) {
  const long long gw = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (gw >= n_tok * H) return;
  const long long t = gw / H;
  const int h = (int)(gw - t * H);
  const T* a = d_o + t * ld_do + (long long)h * hd;
  const T* b = o + t * ld_o + (long long)h * hd;
  float s = 0.f;
  for (int d = lane; d < hd; d += 32) s += Cvt<T>::to_f(a[d]) * Cvt<T>::to_f(b[d]);
  s = warp_sum(s);
  if (lane == 0) delta[gw] = s;
}

template <typename T, int HD, int TPR, int KT>
__global__ void __launch_bounds__(128) attn_bwd_dq_kernel(const AttnArgs a) {
  constexpr int HDT = HD / TPR;
  constexpr int ROWS = 128 / TPR;
  extern __shared__ float smem[];
  float* sK = smem;
  float* sV = smem + KT * HD;
  int* sSeg = reinterpret_cast<int*>(sV + KT * HD);
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * ROWS;
  const int kvh = h / (a.H / a.KV);
  const int r = threadIdx.x / TPR, sub = threadIdx.x % TPR;
  const int i = q0 + r;
  const bool row_ok = i < a.T;
  const long long tok = (long long)b * a.T + i;
  const bool has_seg = a.seg != nullptr;
  const int seg_i = (has_seg && row_ok) ? a.seg[tok] : 0;
  float q[HDT], g[HDT], dq[HDT];
  float lse = INFINITY, dl = 0.f;
#pragma unroll
  for (int d = 0; d < HDT; ++d) { q[d] = 0.f; g[d] = 0.f; dq[d] = 0.f; }
  if (row_ok) {
    const T* qp = reinterpret_cast<const T*>(a.q) + tok * a.ld_q + (long long)h * HD + sub * HDT;
    const T* gp = reinterpret_cast<const T*>(a.d_o) + tok * a.ld_do + (long long)h * HD + sub * HDT;
#pragma unroll
    for (int d = 0; d < HDT; ++d) { q[d] = Cvt<T>::to_f(qp[d]) * a.scale; g[d] = Cvt<T>::to_f(gp[d]); }
    lse = a.lse[tok * a.H + h];
    dl = a.delta[tok * a.H + h];
  }
  const int j_hi = min(a.T, q0 + ROWS);
  int j_lo = 0;
  if (a.window > 0) j_lo = max(0, q0 - a.window + 1);
  j_lo = (j_lo / KT) * KT;
  const T* kb = reinterpret_cast<const T*>(a.k) + (long long)b * a.T * a.ld_k + (long long)kvh * HD;
  const T* vb = reinterpret_cast<const T*>(a.v) + (long long)b * a.T * a.ld_v + (long long)kvh * HD;
  for (int j0 = j_lo; j0 < j_hi; j0 += KT) {
    __syncthreads();
    stage_tile<T>(kb, a.ld_k, j0, KT, a.T, HD, sK);
    stage_tile<T>(vb, a.ld_v, j0, KT, a.T, HD, sV);
    if (has_seg)
      for (int t = threadIdx.x; t < KT; t += blockDim.x) sSeg[t] = (j0 + t < a.T) ? a.seg[(long long)b * a.T + j0 + t] : -2;
    __syncthreads();
    const int jn = min(KT, j_hi - j0);
    for (int jj = 0; jj < jn; ++jj) {
      const int j = j0 + jj;
      const float* kr = sK + jj * HD + sub * HDT;
      const float* vr = sV + jj * HD + sub * HDT;
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int d = 0; d < HDT; ++d) { s += q[d] * kr[d]; dp += g[d] * vr[d]; }
      s = row_sum<TPR>(s);
      dp = row_sum<TPR>(dp);
      if (!row_ok || !visible(i, j, a.window, seg_i, has_seg ? sSeg[jj] : 0, has_seg)) continue;
      const float p = __expf(s - lse);
      const float ds = p * (dp - dl) * a.scale;
#pragma unroll
      for (int d = 0; d < HDT; ++d) dq[d] += ds * kr[d];
    }
  }
  if (!row_ok) return;
  T* dqp = reinterpret_cast<T*>(a.dq) + tok * a.ld_dq + (long long)h * HD + sub * HDT;
#pragma unroll
  for (int d = 0; d < HDT; ++d) dqp[d] = Cvt<T>::from_f(dq[d]);
}

// One thread group per key row; loops over the query heads that share this kv head (in-kernel, ordered GQA
// reduction) and over query tiles at or after the key position.
template <typename T, int HD, int TPR, int KT>
__global__ void __launch_bounds__(128) attn_bwd_dkv_kernel(const AttnArgs a) {
  constexpr int HDT = HD / TPR;
  constexpr int ROWS = 128 / TPR;
  extern __shared__ float smem[];
  float* sQ = smem;
  float* sG = smem + KT * HD;
  float* sLse = sG + KT * HD;
  float* sDl = sLse + KT;
  int* sSeg = reinterpret_cast<int*>(sDl + KT);
  const int b = blockIdx.z, kvh = blockIdx.y, j0 = blockIdx.x * ROWS;
  const int group = a.H / a.KV;
  const int r = threadIdx.x / TPR, sub = threadIdx.x % TPR;
  const int j = j0 + r;
  const bool row_ok = j < a.T;
  const long long tok = (long long)b * a.T + j;
  const bool has_seg = a.seg != nullptr;
  const int seg_j = (has_seg && row_ok) ? a.seg[tok] : 0;
  float k[HDT], v[HDT], dk[HDT], dv[HDT];
#pragma unroll
  for (int d = 0; d < HDT; ++d) { k[d] = 0.f; v[d] = 0.f; dk[d] = 0.f; dv[d] = 0.f; }
  if (row_ok) {
    const T* kp = reinterpret_cast<const T*>(a.k) + tok * a.ld_k + (long long)kvh * HD + sub * HDT;
    const T* vp = reinterpret_cast<const T*>(a.v) + tok * a.ld_v + (long long)kvh * HD + sub * HDT;
#pragma unroll
    for (int d = 0; d < HDT; ++d) { k[d] = Cvt<T>::to_f(kp[d]); v[d] = Cvt<T>::to_f(vp[d]); }
  }
  const int i_lo = (j0 / KT) * KT;
  int i_hi = a.T;
  if (a.window > 0) i_hi = min(a.T, j0 + ROWS - 1 + a.window);
  for (int hh = 0; hh < group; ++hh) {
    const int h = kvh * group + hh;
    const T* qb = reinterpret_cast<const T*>(a.q) + (long long)b * a.T * a.ld_q + (long long)h * HD;
    const T* gb = reinterpret_cast<const T*>(a.d_o) + (long long)b * a.T * a.ld_do + (long long)h * HD;
    for (int i0 = i_lo; i0 < i_hi; i0 += KT) {
      __syncthreads();
      stage_tile<T>(qb, a.ld_q, i0, KT, a.T, HD, sQ);
      stage_tile<T>(gb, a.ld_do, i0, KT, a.T, HD, sG);
      for (int t = threadIdx.x; t < KT; t += blockDim.x) {
        const bool in = i0 + t < a.T;
        const long long tt = (long long)b * a.T + i0 + t;
        sLse[t] = in ? a.lse[tt * a.H + h] : INFINITY;
        sDl[t] = in ? a.delta[tt * a.H + h] : 0.f;
        sSeg[t] = (in && has_seg) ? a.seg[tt] : 0;
      }
      __syncthreads();
      const int in_n = min(KT, i_hi - i0);
      for (int ii = 0; ii < in_n; ++ii) {
        const int i = i0 + ii;
        const float* qr = sQ + ii * HD + sub * HDT;
        const float* gr = sG + ii * HD + sub * HDT;
        float s = 0.f, dp = 0.f;
#pragma unroll
        for (int d = 0; d < HDT; ++d) { s += k[d] * qr[d]; dp += v[d] * gr[d]; }
        s = row_sum<TPR>(s);
        dp = row_sum<TPR>(dp);
        if (!row_ok || !visible(i, j, a.window, sSeg[ii], seg_j, has_seg)) continue;
        const float p = __expf(s * a.scale - sLse[ii]);
        const float ds = p * (dp - sDl[ii]) * a.scale;
#pragma unroll
        for (int d = 0; d < HDT; ++d) { dv[d] += p * gr[d]; dk[d] += ds * qr[d]; }
      }
    }
  }
  if (!row_ok) return;
  T* dkp = reinterpret_cast<T*>(a.dk) + tok * a.ld_dk + (long long)kvh * HD + sub * HDT;
  T* dvp = reinterpret_cast<T*>(a.dv) + tok * a.ld_dv + (long long)kvh * HD + sub * HDT;
#pragma unroll
  for (int d = 0; d < HDT; ++d) { dkp[d] = Cvt<T>::from_f(dk[d]); dvp[d] = Cvt<T>::from_f(dv[d]); }
}

template <typename T, int HD>
int launch_fwd(const AttnArgs& a, cudaStream_t st) {
  constexpr int TPR = HD / 16;   // 16 head dims per thread: small query tiles keep all SMs busy at short T
  constexpr int KT = HD <= 128 ? 32 : 16;
  constexpr int ROWS = 128 / TPR;
  const size_t smem = (size_t)2 * KT * HD * 4 + KT * 4;
  auto kern = attn_fwd_kernel<T, HD, TPR, KT>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid((a.T + ROWS - 1) / ROWS, a.H, a.B);
  kern<<<grid, 128, smem, st>>>(a);
  return gb_launch_rc();
}

template <typename T, int HD>
int launch_bwd(const AttnArgs& a, cudaStream_t st) {
  constexpr int TPR = HD / 16;
  constexpr int KT = HD <= 128 ? 32 : 16;
  constexpr int ROWS = 128 / TPR;
  const long long n_tok = (long long)a.B * a.T;
  attn_delta_kernel<T><<<(unsigned)((n_tok * a.H + 7) / 8), 256, 0, st>>>(
      reinterpret_cast<const T*>(a.d_o), a.ld_do, reinterpret_cast<const T*>(a.o), a.ld_o, a.delta, n_tok, a.H, HD);
  const size_t smem_q = (size_t)2 * KT * HD * 4 + KT * 4;
  const size_t smem_kv = (size_t)2 * KT * HD * 4 + KT * 12;
  auto kq = attn_bwd_dq_kernel<T, HD, TPR, KT>;
  auto kkv = attn_bwd_dkv_kernel<T, HD, TPR, KT>;
  if (smem_kv > 48 * 1024) {
    cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q);
    cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv);
  }
  dim3 gq((a.T + ROWS - 1) / ROWS, a.H, a.B), gkv((a.T + ROWS - 1) / ROWS, a.KV, a.B);
  kq<<<gq, 128, smem_q, st>>>(a);
  kkv<<<gkv, 128, smem_kv, st>>>(a);
  return gb_launch_rc();
}

}  // namespace gb

using namespace gb;

static int attn_check(const gb_attn_args* p) {
  if (!p || p->B <= 0 || p->T <= 0 || p->H <= 0 || p->KV <= 0 || p->H % p->KV) return -1;
  if (p->hd != 32 && p->hd != 64 && p->hd != 128 && p->hd != 256) return -2;
  return 0;
}

static AttnArgs to_args(const gb_attn_args* p) {
  AttnArgs a{};
  a.q = p->q; a.ld_q = p->ld_q; a.k = p->k; a.ld_k = p->ld_k; a.v = p->v; a.ld_v = p->ld_v;
  a.o = p->o; a.ld_o = p->ld_o; a.lse = p->lse; a.seg = p->seg;
  a.B = p->B; a.T = p->T; a.H = p->H; a.KV = p->KV; a.window = p->window; a.scale = p->scale;
  a.d_o = p->d_o; a.ld_do = p->ld_do; a.delta = p->delta;
  a.dq = p->dq; a.ld_dq = p->ld_dq; a.dk = p->dk; a.ld_dk = p->ld_dk; a.dv = p->dv; a.ld_dv = p->ld_dv;
  return a;
}

#define GB_ATTN_DISPATCH(FN)                                            \
  switch (p->hd) {                                                      \
    case 32: return p->is_bf16 ? FN<__nv_bfloat16, 32>(a, st) : FN<__half, 32>(a, st);     \
    case 64: return p->is_bf16 ? FN<__nv_bfloat16, 64>(a, st) : FN<__half, 64>(a, st);     \
    case 128: return p->is_bf16 ? FN<__nv_bfloat16, 128>(a, st) : FN<__half, 128>(a, st);  \
    case 256: return p->is_bf16 ? FN<__nv_bfloat16, 256>(a, st) : FN<__half, 256>(a, st);  \
  }

extern "C" int gb_attn_fwd(const gb_attn_args* p, cudaStream_t st) {
  int rc = attn_check(p);
  if (rc) return rc;
  AttnArgs a = to_args(p);
  GB_ATTN_DISPATCH(launch_fwd)
  return -2;
}

extern "C" int gb_attn_bwd(const gb_attn_args* p, cudaStream_t st) {
  int rc = attn_check(p);
  if (rc) return rc;
  if (!p->d_o || !p->delta || !p->lse || !p->dq || !p->dk || !p->dv) return -1;
  AttnArgs a = to_args(p);
  GB_ATTN_DISPATCH(launch_bwd)
  return -2;
}
