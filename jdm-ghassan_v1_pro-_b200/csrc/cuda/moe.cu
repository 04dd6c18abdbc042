// Mixture-of-experts routing and data movement around the grouped tcgen05 GEMMs.
//
//   route    : router logits (fp32 weights) + jitter hash + softmax + bias-on-selection top-k (ties -> lowest
//              index) + renormalised combine weights + per-block expert histograms       (one warp per token)
//   group    : device-side scan -> 128-row padded expert segments, tile->expert map, stable (token-order) row
//              positions, expert-sorted 16-bit copy of the activations; no host synchronisation anywhere
//   combine  : out = resid + shared(x) + sum_k w_k * y_k   gathered per token (deterministic, no atomics)
//   backward : weighted scatter of d(out) into sorted order, per-slot <d(out), y_k> for the router gradient,
//              softmax-Jacobian with top-k renormalisation (+ aux-loss term, + jitter), d(router weights)
// The semantics are the reference's (core/ops_cpu_moe.cpp:182-379, cuda/moe.cu:113-258, 601-970); the
// structure is not: the reference syncs the host once per layer per pass to read group offsets and loops
// over experts with one cuBLAS call each.
#include "sm100_common.cuh"
#include <algorithm>
#include <type_traits>

#include "gb_api.h"

namespace gb {

constexpr int BLK_TOK = 256;   // most tokens a routing block handles
// Tokens per routing block: small blocks for small batches so that the grid covers the GPU, large blocks for
// large batches so that the single-block scan over [blocks, experts] stays short.
__host__ __device__ inline int blk_tok(int n_tok) { return n_tok < 8192 ? 8 : (n_tok < 65536 ? 64 : BLK_TOK); }
constexpr int MAX_NE = 64;
constexpr int MAX_K = 8;

__device__ __forceinline__ float jitter_u(long long t, int e, unsigned long long seed) {
  unsigned long long h = (unsigned long long)t * 0x9E3779B97F4A7C15ULL;
  h ^= (unsigned long long)e * 0xC2B2AE3D27D4EB4FULL;
  h ^= (seed + 0x9E3779B97F4A7C15ULL);
  h ^= h >> 33; h *= 0xff51afd7ed558ccdULL;
  h ^= h >> 33; h *= 0xc4ceb9fe1a85ec53ULL;
  h ^= h >> 33;
  return (float)((h >> 40) & 0xFFFFFF) / (float)(1 << 24) - 0.5f;
}

// (value, index) arg-max over the warp; equal values keep the lower index
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

// NV8 > 0: d = 256 * NV8 and the activation row stays in registers (one 16-byte load per 256 columns and lane,
// 16-byte weight loads); NV8 = 0 is the loop for any even d.  With the row re-read for every expert in 4-byte
// pieces the kernel was bound by load instructions, at a tenth of the bandwidth its 2 bytes per element need.
template <typename T, int NV8>
__global__ void __launch_bounds__(256) moe_route_kernel(const gb_moe_args a) {
  __shared__ int s_hist[MAX_NE + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ne = a.ne, K = a.top_k, d = a.d;
  for (int i = threadIdx.x; i <= ne; i += blockDim.x) s_hist[i] = 0;
  __syncthreads();
  const int bt = blk_tok(a.n_tok);
  const int t0 = blockIdx.x * bt;
  const int t1 = min(a.n_tok, t0 + bt);
  const T* x16 = reinterpret_cast<const T*>(a.x16);
  const unsigned long long jseed = a.dyn_seed ? a.dyn_seed[0] : a.jitter_seed;   // device copy wins (graph replay)
  // The rest of a token after its logits: soft-max, bias-steered top-k, outputs and the block histogram.
  auto finish = [&](int t, float l0, float l1) {
    const float mx = warp_max(fmaxf(l0, l1));
    const float e0 = lane < ne ? __expf(l0 - mx) : 0.f;
    const float e1 = lane + 32 < ne ? __expf(l1 - mx) : 0.f;
    const float inv = 1.f / warp_sum(e0 + e1);
    const float p0 = e0 * inv, p1 = e1 * inv;
    if (lane < ne) a.probs[(size_t)t * ne + lane] = p0;
    if (lane + 32 < ne) a.probs[(size_t)t * ne + lane + 32] = p1;
    float s0 = lane < ne ? p0 + (a.bias ? a.bias[lane] : 0.f) : -INFINITY;
    float s1 = lane + 32 < ne ? p1 + (a.bias ? a.bias[lane + 32] : 0.f) : -INFINITY;
    float psel[MAX_K];
    int esel[MAX_K];
    float psum = 0.f;
#pragma unroll
    for (int k = 0; k < MAX_K; ++k) {
      if (k < K) {
        float bv = s0; int bi = lane;
        if (s1 > bv) { bv = s1; bi = lane + 32; }
        if (bv == -INFINITY) bi = 1 << 20;   // exhausted lanes never win a tie
        warp_argmax(bv, bi);
        esel[k] = bi;
        const float pw = __shfl_sync(0xffffffffu, bi < 32 ? p0 : p1, bi & 31);
        psel[k] = pw;
        psum += pw;
        if (bi == lane) s0 = -INFINITY;
        if (bi == lane + 32) s1 = -INFINITY;
      }
    }
    const float invs = psum > 1e-8f ? 1.f / psum : 0.f;
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < MAX_K; ++k)
        if (k < K) {
          a.idx[(size_t)t * K + k] = esel[k];
          a.w[(size_t)t * K + k] = psel[k] * invs;
          atomicAdd(&s_hist[esel[k]], 1);
        }
      if (a.shared) atomicAdd(&s_hist[ne], 1);
    }
  };
  if constexpr (NV8 > 0) {
    // Two tokens per warp and trip: the router rows (ne x d fp32, the same for every token) come through L1 once
    // for the pair.  With one token per trip the kernel moved 24 KB of router weights per token through L1 and ran
    // at a tenth of what its 1.5 KB of activations per token need.
    for (int t = t0 + 2 * warp; t < t1; t += 16) {
      const bool two = t + 1 < t1;
      float xf[2][NV8][8];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const T* xr = x16 + (size_t)(t + (u && two ? 1 : 0)) * d;
#pragma unroll
        for (int k = 0; k < NV8; ++k) {
          const uint4 q = *reinterpret_cast<const uint4*>(xr + k * 256 + lane * 8);
          const float2 v0 = Cvt<T>::unpack2(q.x), v1 = Cvt<T>::unpack2(q.y), v2 = Cvt<T>::unpack2(q.z), v3 = Cvt<T>::unpack2(q.w);
          xf[u][k][0] = v0.x; xf[u][k][1] = v0.y; xf[u][k][2] = v1.x; xf[u][k][3] = v1.y;
          xf[u][k][4] = v2.x; xf[u][k][5] = v2.y; xf[u][k][6] = v3.x; xf[u][k][7] = v3.y;
        }
      }
      float l0[2] = {-INFINITY, -INFINITY}, l1[2] = {-INFINITY, -INFINITY};
#pragma unroll 2
      for (int e = 0; e < ne; ++e) {
        const float* wr = a.router_w + (size_t)e * d + lane * 8;
        float s[2] = {0.f, 0.f};
#pragma unroll
        for (int k = 0; k < NV8; ++k) {
          const float4 w0 = *reinterpret_cast<const float4*>(wr + k * 256);
          const float4 w1 = *reinterpret_cast<const float4*>(wr + k * 256 + 4);
#pragma unroll
          for (int u = 0; u < 2; ++u)
            s[u] += xf[u][k][0] * w0.x + xf[u][k][1] * w0.y + xf[u][k][2] * w0.z + xf[u][k][3] * w0.w +
                    xf[u][k][4] * w1.x + xf[u][k][5] * w1.y + xf[u][k][6] * w1.z + xf[u][k][7] * w1.w;
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          s[u] = warp_sum(s[u]);
          const int tt = t + u;
          const int tj = a.seg_tokens > 0 ? tt % a.seg_tokens : tt;   // the jitter hash counts tokens inside a micro-batch
          if (a.use_jitter) s[u] *= 1.0f + a.jitter * 2.0f * jitter_u(tj, e, jseed);
          if (e == lane) l0[u] = s[u];
          if (e == lane + 32) l1[u] = s[u];
        }
      }
      finish(t, l0[0], l1[0]);
      if (two) finish(t + 1, l0[1], l1[1]);
    }
  } else {
    for (int t = t0 + warp; t < t1; t += 8) {
      const T* xr = x16 + (size_t)t * d;
      const int tj = a.seg_tokens > 0 ? t % a.seg_tokens : t;
      float l0 = -INFINITY, l1 = -INFINITY;   // lane holds the logits of experts `lane` and `lane + 32`
      for (int e = 0; e < ne; ++e) {
        const float* wr = a.router_w + (size_t)e * d;
        float s = 0.f;
        for (int i = lane * 2; i < d; i += 64) {
          const float2 xv = Cvt<T>::unpack2(*reinterpret_cast<const uint32_t*>(xr + i));
          const float2 wv = *reinterpret_cast<const float2*>(wr + i);
          s += xv.x * wv.x + xv.y * wv.y;
        }
        s = warp_sum(s);
        if (a.use_jitter) s *= 1.0f + a.jitter * 2.0f * jitter_u(tj, e, jseed);
        if (e == lane) l0 = s;
        if (e == lane + 32) l1 = s;
      }
      finish(t, l0, l1);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= ne; i += blockDim.x) a.block_hist[(size_t)blockIdx.x * (ne + 1) + i] = s_hist[i];
}

// ------------------------------------------------------------------------------------------------ router on tcgen05
// The router logits are a GEMM with a tiny N: logits[n_tok, ne] = x16[n_tok, d] * router_w[ne, d]^T.  For at most 8
// experts one CTA takes 128 tokens: warp 0 streams their activations through a 4-stage ring of [128 x 64] TMA tiles,
// warp 1 issues M = 128, N = 16, K = 16 MMAs into 16 tensor-memory columns, and warps 2-5 then finish one token per
// thread (thread = tensor-memory lane): soft-max, bias-steered top-k with the lowest index on ties, outputs, block
// histograms - the same rules as moe_route_kernel, which stays for everything this kernel does not cover.  The fp32 router
// rows are split into two 16-bit terms, hi = round16(w) in rows 0-7 of the B operand and lo = round16((w - hi) * S) in
// rows 8-15 (S = 2048 for fp16, 256 for bf16), and the logit is D[e] + D[8 + e] / S: 22 (fp16) or 16 (bf16) mantissa
// bits of the weight at the cost of columns the N = 16 instruction computes anyway.  (The CUDA-core kernel spent about
// 400 warp instructions per token on FMAs and lane reductions; this one is bound by reading x16 once.)
constexpr int RT_TOK = 128, RT_KC = 64, RT_ST = 4, RT_THREADS = 192;
constexpr uint32_t RT_XTILE = RT_TOK * RT_KC * 2, RT_WPANEL = 16 * RT_KC * 2;
__host__ __device__ inline size_t rt_smem_bytes(int d, int ne) {
  return (size_t)RT_ST * RT_XTILE + (size_t)(d / RT_KC) * RT_WPANEL + 128 + (size_t)(RT_TOK / 8) * (ne + 1) * 4 + 1024;
}

template <typename T>
__global__ void __launch_bounds__(RT_THREADS) moe_route_tc_kernel(const __grid_constant__ CUtensorMap tmX, const gb_moe_args a,
                                                                  int* status) {
  extern __shared__ __align__(1024) uint8_t rt_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(rt_raw) + 1023) & ~uintptr_t(1023));
  const int ne = a.ne, K = a.top_k, d = a.d;
  const int nkc = d / RT_KC;
  uint8_t* sX = smem;
  uint8_t* sW = sX + RT_ST * RT_XTILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sW + (size_t)nkc * RT_WPANEL);
  uint64_t* full = bars;                   // RT_ST
  uint64_t* empty = bars + RT_ST;          // RT_ST
  uint64_t* d_full = bars + 2 * RT_ST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * RT_ST + 1);
  int* s_hist = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bt = blk_tok(a.n_tok);                       // routing block (<= RT_TOK: checked by the launcher)
  const int nsub = RT_TOK / bt;
  const int t0 = blockIdx.x * RT_TOK;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr float SPLIT = kBf16 ? 256.f : 2048.f;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RT_ST; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(d_full, 1);
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 32); tmem_relinquish(); }
  for (int i = threadIdx.x; i < nsub * (ne + 1); i += RT_THREADS) s_hist[i] = 0;
  __syncthreads();
  // the first activation tiles are asked for before the weights are prepared, so that they arrive meanwhile
  const int pre = nkc < RT_ST ? nkc : RT_ST;
  if (threadIdx.x == 0)
    for (int kc = 0; kc < pre; ++kc) {
      mbar_arrive_expect_tx(&full[kc], RT_XTILE);
      tma_load_2d(&tmX, &full[kc], sX + kc * RT_XTILE, kc * RT_KC, t0);
    }
  // the B operand: 16 rows (8 hi, 8 lo) x d columns, K-major, 128-byte swizzle, one 2 KB panel per 64 columns
  for (int i = threadIdx.x; i < 8 * d; i += RT_THREADS) {
    const int e = i / d, c = i - e * d;
    const float w = e < ne ? a.router_w[(size_t)e * d + c] : 0.f;
    const T hi = Cvt<T>::from_f(w);
    const T lo = Cvt<T>::from_f((w - Cvt<T>::to_f(hi)) * SPLIT);
    uint8_t* panel = sW + (size_t)(c >> 6) * RT_WPANEL;
    const int cc = c & 63;
    const uint32_t off_hi = (uint32_t)(e * 128 + ((((cc >> 3) ^ (e & 7)) << 4) | ((cc & 7) << 1)));
    *reinterpret_cast<T*>(panel + off_hi) = hi;
    *reinterpret_cast<T*>(panel + off_hi + 1024) = lo;        // row e + 8: the next 8-row group, same swizzle phase
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_D = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kc = pre; kc < nkc; ++kc) {
        const int s = kc % RT_ST, ph = (kc / RT_ST) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1)) { atomicCAS(status, 0, ST_TIMEOUT_EMPTY); break; }
        mbar_arrive_expect_tx(&full[s], RT_XTILE);
        tma_load_2d(&tmX, &full[s], sX + s * RT_XTILE, kc * RT_KC, t0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(kBf16 ? 1 : 0, 0, 0, RT_TOK, 16);
      bool ok = true;
      for (int kc = 0; kc < nkc && ok; ++kc) {
        const int s = kc % RT_ST, ph = (kc / RT_ST) & 1;
        if (!mbar_wait(&full[s], ph)) { atomicCAS(status, 0, ST_TIMEOUT_FULL); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < RT_KC / 16; ++kk)
          umma_f16(tmem_D, make_smem_desc_sw128(smem_u32(sX + s * RT_XTILE) + kk * 32, 16, 1024),
                   make_smem_desc_sw128(smem_u32(sW + (size_t)kc * RT_WPANEL) + kk * 32, 16, 1024), idesc,
                   (kc > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(d_full);
    }
    __syncwarp();
  } else {
    // one token per thread; a warp reads the tensor-memory lane quarter (warp % 4)
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int t = t0 + r;
    const bool got = mbar_wait(d_full, 0);
    if (!got && lane == 0) atomicCAS(status, 0, ST_TIMEOUT_TMEM_FULL);
    if (got) {
      tc_fence_after();
      uint32_t v[16];
      tmem_ld_32x16(tmem_D + ((uint32_t)(q * 32) << 16), v);
      tmem_ld_wait();
      tc_fence_before();
      if (t < a.n_tok) {
        const unsigned long long jseed = a.dyn_seed ? a.dyn_seed[0] : a.jitter_seed;
        const int tj = a.seg_tokens > 0 ? t % a.seg_tokens : t;
        float l[8], pr[8], sc[8];
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          l[e] = __uint_as_float(v[e]) + __uint_as_float(v[8 + e]) * (1.f / SPLIT);
          if (a.use_jitter) l[e] *= 1.0f + a.jitter * 2.0f * jitter_u(tj, e, jseed);
          if (e >= ne) l[e] = -INFINITY;
          mx = fmaxf(mx, l[e]);
        }
        float sum = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) { pr[e] = e < ne ? __expf(l[e] - mx) : 0.f; sum += pr[e]; }
        const float inv = 1.f / sum;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          pr[e] *= inv;
          if (e < ne) a.probs[(size_t)t * ne + e] = pr[e];
          sc[e] = e < ne ? pr[e] + (a.bias ? a.bias[e] : 0.f) : -INFINITY;
        }
        int esel[MAX_K];
        float psel[MAX_K];
        float psum = 0.f;
#pragma unroll
        for (int k = 0; k < MAX_K; ++k)
          if (k < K) {
            float bv = sc[0];
            int bi = 0;
#pragma unroll
            for (int e = 1; e < 8; ++e)
              if (sc[e] > bv) { bv = sc[e]; bi = e; }       // strict: equal scores keep the lower index
            float pw = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (e == bi) { pw = pr[e]; sc[e] = -INFINITY; }
            esel[k] = bi;
            psel[k] = pw;
            psum += pw;
          }
        const float invs = psum > 1e-8f ? 1.f / psum : 0.f;
        int* hist = s_hist + (r / bt) * (ne + 1);
#pragma unroll
        for (int k = 0; k < MAX_K; ++k)
          if (k < K) {
            a.idx[(size_t)t * K + k] = esel[k];
            a.w[(size_t)t * K + k] = psel[k] * invs;
            atomicAdd(&hist[esel[k]], 1);
          }
        if (a.shared) atomicAdd(&hist[ne], 1);
      }
    }
  }
  __syncthreads();
  const int nb = (a.n_tok + bt - 1) / bt;
  for (int i = threadIdx.x; i < nsub * (ne + 1); i += RT_THREADS) {
    const int b = blockIdx.x * nsub + i / (ne + 1);
    if (b < nb) a.block_hist[(size_t)b * (ne + 1) + i % (ne + 1)] = s_hist[i];
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_D, 32); }
}

// Single block.  Totals, padded offsets, per-block bases, tile map, balance statistics.
// `staged` != 0: the histogram table fits the dynamic shared memory passed at launch and is scanned there
// (the per-expert scans are chains of dependent loads; in global memory they dominate the kernel).
__global__ void moe_scan_kernel(const gb_moe_args a, int n_blocks, int staged) {
  __shared__ int s_total[MAX_NE + 1];
  __shared__ int s_off[MAX_NE + 2];
  extern __shared__ int s_tab[];
  const int ne1 = a.ne + (a.shared ? 1 : 0);
  const int stride = a.ne + 1;
  const int e = threadIdx.x;
  const int cells = n_blocks * stride;
  if (staged) {
    for (int i = threadIdx.x; i < cells; i += blockDim.x) s_tab[i] = a.block_hist[i];
    __syncthreads();
  }
  // micro-batch segments of the pass: routed-slot shares (and further down the balance loss) are kept per segment,
  // as if every micro-batch had been routed on its own.  Blocks never straddle a segment (checked by the launcher).
  const int bt = blk_tok(a.n_tok);
  const int seg_tok = a.seg_tokens > 0 ? a.seg_tokens : a.n_tok;
  const int bps = (a.seg_tokens > 0 && a.seg_tokens < a.n_tok) ? seg_tok / bt : n_blocks;   // blocks per segment
  const int n_seg = (a.n_tok + seg_tok - 1) / seg_tok;
  if (staged) {
    // one warp per expert: exclusive scan of its column over the blocks, 32 blocks per trip (one thread per expert
    // walking all blocks was a chain of a thousand dependent shared-memory round trips, most of this kernel's time)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    for (int ex = warp; ex < ne1; ex += n_warps) {
      int run = 0;
      for (int b0 = 0; b0 < n_blocks; b0 += 32) {
        const int b = b0 + lane;
        const int c = b < n_blocks ? s_tab[b * stride + ex] : 0;
        int inc = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int n = __shfl_up_sync(0xffffffffu, inc, o);
          if (lane >= o) inc += n;
        }
        if (b < n_blocks) s_tab[b * stride + ex] = run + inc - c;
        run += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (lane == 0) {
        s_total[ex] = run;
        a.block_base[(size_t)n_blocks * stride + ex] = run;  // last row: totals
      }
    }
    __syncthreads();
    // routed-slot share of every (segment, expert): a difference of two scanned values
    if (a.f_frac)
      for (int idx = threadIdx.x; idx < n_seg * a.ne; idx += blockDim.x) {
        const int sgi = idx / a.ne, ex = idx - sgi * a.ne;
        const int b_lo = sgi * bps, b_hi = min(n_blocks, b_lo + bps);
        const int lo = s_tab[b_lo * stride + ex];
        const int hi = b_hi < n_blocks ? s_tab[b_hi * stride + ex] : s_total[ex];
        const int ntk = min(seg_tok, a.n_tok - sgi * seg_tok);
        a.f_frac[(size_t)sgi * a.ne + ex] = (float)(hi - lo) / (float)((long long)ntk * a.top_k);
      }
  } else if (e < ne1) {
    int run = 0, segsum = 0;
    for (int b = 0; b < n_blocks; ++b) {
      const int c = a.block_hist[(size_t)b * stride + e];
      a.block_base[(size_t)b * stride + e] = run;   // relative for now
      run += c;
      segsum += c;
      if (((b + 1) % bps == 0 || b == n_blocks - 1) && e < a.ne && a.f_frac) {
        const int sgi = b / bps;
        const int ntk = min(seg_tok, a.n_tok - sgi * seg_tok);
        a.f_frac[(size_t)sgi * a.ne + e] = (float)segsum / (float)((long long)ntk * a.top_k);
        segsum = 0;
      }
    }
    s_total[e] = run;
    a.block_base[(size_t)n_blocks * stride + e] = run;  // last row: totals
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int i = 0; i < ne1; ++i) {
      s_off[i] = off;
      off += (s_total[i] + GB_MOE_PAD - 1) / GB_MOE_PAD * GB_MOE_PAD;
    }
    s_off[ne1] = off;
    for (int i = 0; i <= ne1; ++i) a.seg_offsets[i] = s_off[i];
    if (!a.shared) a.seg_offsets[a.ne + 1] = off;
    a.num_tiles[0] = off / 128;
  }
  __syncthreads();
  if (staged) {
    for (int i = threadIdx.x; i < cells; i += blockDim.x) {
      const int col = i % stride;
      a.block_base[i] = s_tab[i] + (col < ne1 ? s_off[col] : 0);
    }
  } else if (e < ne1) {
    for (int b = 0; b < n_blocks; ++b) a.block_base[(size_t)b * stride + e] += s_off[e];
  }
  if (e < ne1)
    for (int tle = s_off[e] / 128; tle < s_off[e + 1] / 128; ++tle) a.tile_expert[tle] = e;
  if (e < a.ne) {
    if (a.counts) a.counts[e] += (float)s_total[e];
  }
  if (a.aux_acc && a.aux_m && a.f_frac) {                      // uniform over the block
    // balance loss of this call: per segment ne * sum_e mean_prob[e] * slot_share[e], weighted by seg_weight (the
    // segment's supervised tokens) when given.  f_frac was written above by this block (ordered by the barriers).
    // One thread per segment fetches its 2 * ne values (64 segments read by one thread were 1024 dependent loads, most
    // of this kernel's time); thread 0 then adds the segments in order, so the sum is the same as a serial loop's.
    __shared__ float s_seg[256];
    auto seg_term = [&](int sgi) {
      float raw = 0.f;
      for (int i = 0; i < a.ne; ++i) raw += a.aux_m[(size_t)sgi * a.ne + i] * a.f_frac[(size_t)sgi * a.ne + i];
      return (a.seg_weight ? a.seg_weight[sgi] : 1.f) * (float)a.ne * raw;
    };
    if (n_seg <= 256) {
      if ((int)threadIdx.x < n_seg) s_seg[threadIdx.x] = seg_term(threadIdx.x);
      __syncthreads();
      if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int sgi = 0; sgi < n_seg; ++sgi) tot += s_seg[sgi];
        a.aux_acc[0] += tot;
      }
    } else if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int sgi = 0; sgi < n_seg; ++sgi) tot += seg_term(sgi);
      a.aux_acc[0] += tot;
    }
  }
}

// mean over the tokens of segment blockIdx.y of probs[t, e] -> aux_m[segment, e]; one block per (expert, segment),
// fixed-order tree reduction
__global__ void moe_colmean_kernel(const float* __restrict__ probs, float* __restrict__ out, int n_tok_all, int ne,
                                   int seg_tok) {
  __shared__ float s[256];
  const int e = blockIdx.x;
  const int t_lo = blockIdx.y * seg_tok;
  const int n_tok = min(seg_tok, n_tok_all - t_lo);
  probs += (size_t)t_lo * ne;
  out += (size_t)blockIdx.y * ne;
  float acc = 0.f;
  for (int t = threadIdx.x; t < n_tok; t += 256) acc += probs[(size_t)t * ne + e];
  s[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) s[threadIdx.x] += s[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[e] = s[0] / (float)n_tok;
}

// Row positions (stable: token order inside every expert) and the expert-sorted copy.
template <typename T>
__global__ void __launch_bounds__(256) moe_pack_kernel(const gb_moe_args a) {
  __shared__ int s_idx[BLK_TOK * MAX_K];
  __shared__ int s_pos[BLK_TOK * (MAX_K + 1)];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ne = a.ne, K = a.top_k, S = K + (a.shared ? 1 : 0), d = a.d;
  const int bt = blk_tok(a.n_tok);
  const int t0 = blockIdx.x * bt;
  const int nt = min(a.n_tok, t0 + bt) - t0;
  for (int i = threadIdx.x; i < nt * K; i += blockDim.x) s_idx[i] = a.idx[(size_t)t0 * K + i];
  __syncthreads();
  const int* base = a.block_base + (size_t)blockIdx.x * (ne + 1);
  for (int e = warp; e < ne; e += 8) {
    int run = base[e];
    for (int c = 0; c < nt; c += 32) {
      const int tl = c + lane;
      int k_hit = -1;
      if (tl < nt)
        for (int k = 0; k < K; ++k)
          if (s_idx[tl * K + k] == e) k_hit = k;
      const unsigned bal = __ballot_sync(0xffffffffu, k_hit >= 0);
      if (k_hit >= 0) s_pos[tl * S + k_hit] = run + __popc(bal & ((1u << lane) - 1));
      run += __popc(bal);
    }
  }
  if (a.shared)
    for (int tl = threadIdx.x; tl < nt; tl += blockDim.x) s_pos[tl * S + K] = base[ne] + tl;
  __syncthreads();
  for (int i = threadIdx.x; i < nt * S; i += blockDim.x) a.slot_pos[(size_t)t0 * S + i] = s_pos[i];
  const T* x16 = reinterpret_cast<const T*>(a.x16);
  T* xp = reinterpret_cast<T*>(a.x_perm);
  const int vec = d / 8;
  for (int tl = warp; tl < nt; tl += 8) {
    const uint4* src = reinterpret_cast<const uint4*>(x16 + (size_t)(t0 + tl) * d);
    for (int i = lane; i < vec; i += 32) {
      const uint4 v = src[i];
      for (int s = 0; s < S; ++s) reinterpret_cast<uint4*>(xp + (size_t)s_pos[tl * S + s] * d)[i] = v;
    }
  }
}

// zero rows [seg_off[e] + total[e], seg_off[e+1]) of a sorted 16-bit buffer
template <typename T>
__global__ void moe_zero_pads_kernel(T* __restrict__ buf, const int* __restrict__ seg_offsets,
                                     const int* __restrict__ totals, int d) {
  const int e = blockIdx.x;
  const int r0 = seg_offsets[e] + totals[e], r1 = seg_offsets[e + 1];
  const int vec = d / 8;
  for (int i = threadIdx.x; i < (r1 - r0) * vec; i += blockDim.x)
    reinterpret_cast<uint4*>(buf + (size_t)r0 * d)[i] = make_uint4(0, 0, 0, 0);
}

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const gb_moe_args a) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= a.n_tok) return;
  const int K = a.top_k, S = K + (a.shared ? 1 : 0), d = a.d;
  const T* y = reinterpret_cast<const T*>(a.y_perm);
  int pos[MAX_K + 1];
  float w[MAX_K + 1];
#pragma unroll
  for (int s = 0; s <= MAX_K; ++s)
    if (s < S) {
      pos[s] = a.slot_pos[(size_t)t * S + s];
      w[s] = s < K ? a.w[(size_t)t * K + s] : 1.f;
    }
  for (int i = lane * 8; i < d; i += 256) {
    float acc[8];
    if (a.resid) {
      const float4 r0 = *reinterpret_cast<const float4*>(a.resid + (size_t)t * d + i);
      const float4 r1 = *reinterpret_cast<const float4*>(a.resid + (size_t)t * d + i + 4);
      acc[0] = r0.x; acc[1] = r0.y; acc[2] = r0.z; acc[3] = r0.w; acc[4] = r1.x; acc[5] = r1.y; acc[6] = r1.z; acc[7] = r1.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
#pragma unroll
    for (int s = 0; s <= MAX_K; ++s)
      if (s < S) {
        const uint4 q = *reinterpret_cast<const uint4*>(y + (size_t)pos[s] * d + i);
        const float2 v0 = Cvt<T>::unpack2(q.x), v1 = Cvt<T>::unpack2(q.y), v2 = Cvt<T>::unpack2(q.z), v3 = Cvt<T>::unpack2(q.w);
        acc[0] += w[s] * v0.x; acc[1] += w[s] * v0.y; acc[2] += w[s] * v1.x; acc[3] += w[s] * v1.y;
        acc[4] += w[s] * v2.x; acc[5] += w[s] * v2.y; acc[6] += w[s] * v3.x; acc[7] += w[s] * v3.y;
      }
    *reinterpret_cast<float4*>(a.out + (size_t)t * d + i) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(a.out + (size_t)t * d + i + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

// dy_perm[pos(t,k)] = w_k * dout[t]; dy_perm[pos(t,shared)] = dout[t]; gdot[t,k] = <dout[t], y_perm[pos(t,k)]>
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_bwd_kernel(const gb_moe_args a) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= a.n_tok) return;
  const int K = a.top_k, S = K + (a.shared ? 1 : 0), d = a.d;
  const T* y = reinterpret_cast<const T*>(a.y_perm);
  T* dy = reinterpret_cast<T*>(a.dy_perm);
  int pos[MAX_K + 1];
  float w[MAX_K + 1], dot[MAX_K];
#pragma unroll
  for (int s = 0; s <= MAX_K; ++s)
    if (s < S) {
      pos[s] = a.slot_pos[(size_t)t * S + s];
      w[s] = s < K ? a.w[(size_t)t * K + s] : 1.f;
    }
#pragma unroll
  for (int k = 0; k < MAX_K; ++k) dot[k] = 0.f;
  for (int i = lane * 8; i < d; i += 256) {
    const float4 g0 = *reinterpret_cast<const float4*>(a.dout + (size_t)t * d + i);
    const float4 g1 = *reinterpret_cast<const float4*>(a.dout + (size_t)t * d + i + 4);
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
    for (int s = 0; s <= MAX_K; ++s)
      if (s < S) {
        if (s < K) {
          const uint4 q = *reinterpret_cast<const uint4*>(y + (size_t)pos[s] * d + i);
          const float2 v0 = Cvt<T>::unpack2(q.x), v1 = Cvt<T>::unpack2(q.y), v2 = Cvt<T>::unpack2(q.z), v3 = Cvt<T>::unpack2(q.w);
          dot[s] += g[0] * v0.x + g[1] * v0.y + g[2] * v1.x + g[3] * v1.y + g[4] * v2.x + g[5] * v2.y + g[6] * v3.x + g[7] * v3.y;
        }
        uint4 o;
        o.x = Cvt<T>::pack2(w[s] * g[0], w[s] * g[1]); o.y = Cvt<T>::pack2(w[s] * g[2], w[s] * g[3]);
        o.z = Cvt<T>::pack2(w[s] * g[4], w[s] * g[5]); o.w = Cvt<T>::pack2(w[s] * g[6], w[s] * g[7]);
        *reinterpret_cast<uint4*>(dy + (size_t)pos[s] * d + i) = o;
      }
  }
#pragma unroll
  for (int k = 0; k < MAX_K; ++k)
    if (k < K) {
      const float s = warp_sum(dot[k]);
      if (lane == 0) a.gdot[(size_t)t * K + k] = s;
    }
}

// Per token: sum the sorted-order input gradients of its slots, add the router path, write 16-bit dx and the
// router-logit gradients (into `part`, [n_tok, ne]).
template <typename T>
__global__ void __launch_bounds__(256, 4) moe_router_bwd_kernel(const gb_moe_args a) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= a.n_tok) return;
  const int ne = a.ne, K = a.top_k, S = K + (a.shared ? 1 : 0), d = a.d;
  // ---- router-logit gradient (lane e and e+32 hold expert e / e+32)
  // the slot positions first: they do not depend on the router part, and after its stores the compiler could not
  // move these loads up by itself
  int pos[MAX_K + 1];
#pragma unroll
  for (int s = 0; s <= MAX_K; ++s)
    if (s < S) pos[s] = a.slot_pos[(size_t)t * S + s];
  const float p0 = lane < ne ? a.probs[(size_t)t * ne + lane] : 0.f;
  const float p1 = lane + 32 < ne ? a.probs[(size_t)t * ne + lane + 32] : 0.f;
  float dp0 = 0.f, dp1 = 0.f;
  const int sgi = a.seg_tokens > 0 ? t / a.seg_tokens : 0;       // micro-batch segment of this token
  const int tj = a.seg_tokens > 0 ? t - sgi * a.seg_tokens : t;
  const float aux_coef = a.dyn_aux_coef ? a.dyn_aux_coef[sgi] : a.aux_coef;   // one coefficient per segment
  const unsigned long long jseed = a.dyn_seed ? a.dyn_seed[0] : a.jitter_seed;
  if (a.f_frac && aux_coef != 0.f) {
    const float* ff = a.f_frac + (size_t)sgi * ne;
    if (lane < ne) dp0 = aux_coef * ff[lane];
    if (lane + 32 < ne) dp1 = aux_coef * ff[lane + 32];
  }
  float ssum = 0.f, gbar = 0.f;
  for (int k = 0; k < K; ++k) {
    const int e = a.idx[(size_t)t * K + k];
    const float pe = __shfl_sync(0xffffffffu, e < 32 ? p0 : p1, e & 31);   // probs[t, e], already in a lane
    ssum += pe;
    gbar += a.gdot[(size_t)t * K + k] * a.w[(size_t)t * K + k];
  }
  if (ssum > 1e-8f) {
    const float invs = 1.f / ssum;
    for (int k = 0; k < K; ++k) {
      const int e = a.idx[(size_t)t * K + k];
      const float v = (a.gdot[(size_t)t * K + k] - gbar) * invs;
      if (e == lane) dp0 += v;
      if (e == lane + 32) dp1 += v;
    }
  }
  const float pdp = warp_sum(p0 * dp0 + p1 * dp1);
  float dl0 = p0 * (dp0 - pdp), dl1 = p1 * (dp1 - pdp);
  if (a.use_jitter) {
    dl0 *= 1.0f + a.jitter * 2.0f * jitter_u(tj, lane, jseed);
    dl1 *= 1.0f + a.jitter * 2.0f * jitter_u(tj, lane + 32, jseed);
  }
  if (lane < ne) a.part[(size_t)t * ne + lane] = dl0;
  if (lane + 32 < ne) a.part[(size_t)t * ne + lane + 32] = dl1;
  // ---- input gradient
  const T* dxp = reinterpret_cast<const T*>(a.dx_perm);
  T* dx = reinterpret_cast<T*>(a.dx16);
  for (int i = lane * 8; i < d; i += 256) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int s = 0; s <= MAX_K; ++s)
      if (s < S) {
        const uint4 q = *reinterpret_cast<const uint4*>(dxp + (size_t)pos[s] * d + i);
        const float2 v0 = Cvt<T>::unpack2(q.x), v1 = Cvt<T>::unpack2(q.y), v2 = Cvt<T>::unpack2(q.z), v3 = Cvt<T>::unpack2(q.w);
        acc[0] += v0.x; acc[1] += v0.y; acc[2] += v1.x; acc[3] += v1.y; acc[4] += v2.x; acc[5] += v2.y; acc[6] += v3.x; acc[7] += v3.y;
      }
#pragma unroll 4
    for (int e = 0; e < ne; ++e) {
      const float dl = __shfl_sync(0xffffffffu, e < 32 ? dl0 : dl1, e & 31);
      const float4 w0 = *reinterpret_cast<const float4*>(a.router_w + (size_t)e * d + i);
      const float4 w1 = *reinterpret_cast<const float4*>(a.router_w + (size_t)e * d + i + 4);
      acc[0] += dl * w0.x; acc[1] += dl * w0.y; acc[2] += dl * w0.z; acc[3] += dl * w0.w;
      acc[4] += dl * w1.x; acc[5] += dl * w1.y; acc[6] += dl * w1.z; acc[7] += dl * w1.w;
    }
    uint4 o;
    o.x = Cvt<T>::pack2(acc[0], acc[1]); o.y = Cvt<T>::pack2(acc[2], acc[3]);
    o.z = Cvt<T>::pack2(acc[4], acc[5]); o.w = Cvt<T>::pack2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(dx + (size_t)t * d + i) = o;
  }
}

// The same for at most 8 experts, in two kernels.  moe_router_dlogit_kernel is the router-logit part above (one thread
// per token, a few hundred bytes); moe_router_dx_kernel then streams the input gradient with the router rows held in
// registers: a lane owns 8 columns of all (<= 8) experts for the life of the block, 4 token groups x 96 lanes per
// block, blocks walk the tokens with a grid stride.  Per token a lane issues its slot rows' 16-byte loads and two
// broadcast loads of the logit gradients; the 24 KB of router rows are no longer re-read from L1 for every token
// (sixteen 16-byte loads per 8 columns, three quarters of the one-kernel form's load instructions).
__global__ void __launch_bounds__(256) moe_router_dlogit_kernel(const gb_moe_args a) {
  // one thread per token: with at most 8 experts everything of a token fits a thread's registers, and its dozen
  // loads are independent (a warp per token waited for them in sequence, round after round)
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= a.n_tok) return;
  const int ne = a.ne, K = a.top_k;
  float p[8], dp[8];
  int idx[MAX_K];
  float gd[MAX_K], wk[MAX_K];
#pragma unroll
  for (int e = 0; e < 8; ++e) p[e] = e < ne ? a.probs[(size_t)t * ne + e] : 0.f;
#pragma unroll
  for (int k = 0; k < MAX_K; ++k)
    if (k < K) { idx[k] = a.idx[(size_t)t * K + k]; gd[k] = a.gdot[(size_t)t * K + k]; wk[k] = a.w[(size_t)t * K + k]; }
  const int sgi = a.seg_tokens > 0 ? t / a.seg_tokens : 0;       // micro-batch segment of this token
  const int tj = a.seg_tokens > 0 ? t - sgi * a.seg_tokens : t;
  const float aux_coef = a.dyn_aux_coef ? a.dyn_aux_coef[sgi] : a.aux_coef;
  const unsigned long long jseed = a.dyn_seed ? a.dyn_seed[0] : a.jitter_seed;
  const bool aux = a.f_frac && aux_coef != 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) dp[e] = (aux && e < ne) ? aux_coef * a.f_frac[(size_t)sgi * ne + e] : 0.f;
  float ssum = 0.f, gbar = 0.f;
#pragma unroll
  for (int k = 0; k < MAX_K; ++k)
    if (k < K) {
#pragma unroll
      for (int e = 0; e < 8; ++e) ssum += idx[k] == e ? p[e] : 0.f;
      gbar += gd[k] * wk[k];
    }
  if (ssum > 1e-8f) {
    const float invs = 1.f / ssum;
#pragma unroll
    for (int k = 0; k < MAX_K; ++k)
      if (k < K) {
        const float v = (gd[k] - gbar) * invs;
#pragma unroll
        for (int e = 0; e < 8; ++e) dp[e] += idx[k] == e ? v : 0.f;
      }
  }
  float pdp = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) pdp += p[e] * dp[e];
#pragma unroll
  for (int e = 0; e < 8; ++e)
    if (e < ne) {
      float dl = p[e] * (dp[e] - pdp);
      if (a.use_jitter) dl *= 1.0f + a.jitter * 2.0f * jitter_u(tj, e, jseed);
      a.part[(size_t)t * ne + e] = dl;
    }
}

constexpr int RD_LANES = 96, RD_GROUPS = 4;
template <typename T, int NS>       // NS = slots per token (top_k + shared), so that the row buffers are exactly that long
__global__ void __launch_bounds__(RD_LANES * RD_GROUPS) moe_router_dx_kernel(const gb_moe_args a) {
  const int g = threadIdx.x / RD_LANES, l = threadIdx.x - g * RD_LANES;
  const int c0 = (blockIdx.y * RD_LANES + l) * 8;
  const int ne = a.ne, d = a.d;
  constexpr int S = NS;
  if (c0 >= d) return;                            // no block-wide barrier below
  float w[8][8];                                  // router rows of this lane's 8 columns (zero beyond ne)
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f), w1 = w0;
    if (e < ne) {
      w0 = *reinterpret_cast<const float4*>(a.router_w + (size_t)e * d + c0);
      w1 = *reinterpret_cast<const float4*>(a.router_w + (size_t)e * d + c0 + 4);
    }
    w[e][0] = w0.x; w[e][1] = w0.y; w[e][2] = w0.z; w[e][3] = w0.w;
    w[e][4] = w1.x; w[e][5] = w1.y; w[e][6] = w1.z; w[e][7] = w1.w;
  }
  const T* dxp = reinterpret_cast<const T*>(a.dx_perm);
  T* dx = reinterpret_cast<T*>(a.dx16);
  const bool vec = ne == 8;
  // Two tokens in flight: a token's slot rows depend on its slot positions, a chain of two global loads.  The positions
  // are fetched two tokens ahead and the rows one token ahead, so that every trip waits for one load, not two.
  const int stride = gridDim.x * RD_GROUPS;
  auto load_pos = [&](int t, int (&pos)[NS]) {
#pragma unroll
    for (int s = 0; s < NS; ++s)
      pos[s] = t < a.n_tok ? a.slot_pos[(size_t)t * S + s] : 0;
  };
  auto load_rows = [&](int t, const int (&pos)[NS], uint4 (&q)[NS], float (&dl)[8]) {
    if (t >= a.n_tok) return;
#pragma unroll
    for (int s = 0; s < NS; ++s)
      q[s] = *reinterpret_cast<const uint4*>(dxp + (size_t)pos[s] * d + c0);
    if (vec) {
      const float4 a4 = *reinterpret_cast<const float4*>(a.part + (size_t)t * 8);
      const float4 b4 = *reinterpret_cast<const float4*>(a.part + (size_t)t * 8 + 4);
      dl[0] = a4.x; dl[1] = a4.y; dl[2] = a4.z; dl[3] = a4.w; dl[4] = b4.x; dl[5] = b4.y; dl[6] = b4.z; dl[7] = b4.w;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) dl[e] = e < ne ? a.part[(size_t)t * ne + e] : 0.f;
    }
  };
  int t0 = blockIdx.x * RD_GROUPS + g;
  int pos0[NS], pos1[NS];
  uint4 q0[NS], q1[NS];
  float dl0[8], dl1[8];
  load_pos(t0, pos0);
  load_pos(t0 + stride, pos1);
  load_rows(t0, pos0, q0, dl0);
  for (; t0 < a.n_tok; t0 += stride) {
    load_rows(t0 + stride, pos1, q1, dl1);          // the next token's rows
    load_pos(t0 + 2 * stride, pos0);                // positions of the one after (pos0 is free: its rows are loaded)
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int s = 0; s < NS; ++s)
      {
        const float2 v0 = Cvt<T>::unpack2(q0[s].x), v1 = Cvt<T>::unpack2(q0[s].y), v2 = Cvt<T>::unpack2(q0[s].z),
                     v3 = Cvt<T>::unpack2(q0[s].w);
        acc[0] += v0.x; acc[1] += v0.y; acc[2] += v1.x; acc[3] += v1.y; acc[4] += v2.x; acc[5] += v2.y; acc[6] += v3.x; acc[7] += v3.y;
      }
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += dl0[e] * w[e][j];
    uint4 o;
    o.x = Cvt<T>::pack2(acc[0], acc[1]); o.y = Cvt<T>::pack2(acc[2], acc[3]);
    o.z = Cvt<T>::pack2(acc[4], acc[5]); o.w = Cvt<T>::pack2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(dx + (size_t)t0 * d + c0) = o;
    // hand over: next token's rows become current, the freshly loaded positions become next
#pragma unroll
    for (int s = 0; s < NS; ++s)
      { q0[s] = q1[s]; const int tmp = pos0[s]; pos0[s] = pos1[s]; pos1[s] = tmp; }
#pragma unroll
    for (int e = 0; e < 8; ++e) dl0[e] = dl1[e];
  }
}

// d_router_w[e, c] += sum_t dlogit[t, e] * x16[t, c], in a fixed order (deterministic).
// grid (column groups / 96, token chunks, expert groups of 8), 384 threads = 4 token groups x 96 lanes.  A lane owns 8
// columns (one 16-byte load of the activations per token) and 8 experts, 64 sums in registers; token group g takes
// tokens ta + g, ta + g + 4, ... of the chunk, four per trip, and the four groups are added in group order through
// shared memory.  With more than one token chunk `dw` is a partial buffer [chunks, ne, d] that
// moe_router_wgrad_fold_kernel adds up in chunk order.  (One column per thread with eight scalar dlogit loads per token
// ran at 0.14 of the copy bandwidth.)
constexpr int RW_LANES = 96, RW_GROUPS = 4;
template <typename T>
__global__ void __launch_bounds__(RW_LANES * RW_GROUPS) moe_router_wgrad_kernel(const float* __restrict__ dlogit,
                                                                              const T* __restrict__ x16, float* __restrict__ dw,
                                                                              int n_tok, int ne, int d) {
  __shared__ float red[RW_LANES][65];
  const int g = threadIdx.x / RW_LANES, l = threadIdx.x - g * RW_LANES;
  const int c0 = (blockIdx.x * RW_LANES + l) * 8;
  const bool live = c0 < d;                       // d % 8 == 0: a live lane has all 8 columns
  const int e0 = blockIdx.z * 8;
  const int chunks = gridDim.y;
  const int per = (n_tok + chunks - 1) / chunks;
  const int ta = blockIdx.y * per, tb = min(n_tok, ta + per);
  const bool vec = (ne % 4 == 0) && (e0 + 8 <= ne);
  float acc[8][8];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[j][k] = 0.f;
  auto load_dl = [&](int t, float (&dl)[8]) {
    if (vec) {
      const float4 a4 = *reinterpret_cast<const float4*>(dlogit + (size_t)t * ne + e0);
      const float4 b4 = *reinterpret_cast<const float4*>(dlogit + (size_t)t * ne + e0 + 4);
      dl[0] = a4.x; dl[1] = a4.y; dl[2] = a4.z; dl[3] = a4.w; dl[4] = b4.x; dl[5] = b4.y; dl[6] = b4.z; dl[7] = b4.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) dl[j] = e0 + j < ne ? dlogit[(size_t)t * ne + e0 + j] : 0.f;
    }
  };
  auto fma_tok = [&](const uint4& xq, const float (&dl)[8]) {
    float xv[8];
    const uint32_t* xu = reinterpret_cast<const uint32_t*>(&xq);
#pragma unroll
    for (int k = 0; k < 4; ++k) { const float2 f = Cvt<T>::unpack2(xu[k]); xv[2 * k] = f.x; xv[2 * k + 1] = f.y; }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[j][k] += dl[j] * xv[k];
  };
  if (live) {
    int t = ta + g;
    for (; t + 3 * RW_GROUPS < tb; t += 4 * RW_GROUPS) {  // four tokens' loads in flight; the additions keep token order
      const uint4 x0 = *reinterpret_cast<const uint4*>(x16 + (size_t)t * d + c0);
      const uint4 x1 = *reinterpret_cast<const uint4*>(x16 + (size_t)(t + RW_GROUPS) * d + c0);
      const uint4 x2 = *reinterpret_cast<const uint4*>(x16 + (size_t)(t + 2 * RW_GROUPS) * d + c0);
      const uint4 x3 = *reinterpret_cast<const uint4*>(x16 + (size_t)(t + 3 * RW_GROUPS) * d + c0);
      float d0[8], d1[8], d2[8], d3[8];
      load_dl(t, d0);
      load_dl(t + RW_GROUPS, d1);
      load_dl(t + 2 * RW_GROUPS, d2);
      load_dl(t + 3 * RW_GROUPS, d3);
      fma_tok(x0, d0);
      fma_tok(x1, d1);
      fma_tok(x2, d2);
      fma_tok(x3, d3);
    }
    for (; t < tb; t += RW_GROUPS) {
      const uint4 x0 = *reinterpret_cast<const uint4*>(x16 + (size_t)t * d + c0);
      float d0[8];
      load_dl(t, d0);
      fma_tok(x0, d0);
    }
  }
  // groups 1..3 hand their sums to group 0, in group order
  for (int gg = 1; gg < RW_GROUPS; ++gg) {
    if (g == gg) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int k = 0; k < 8; ++k) red[l][j * 8 + k] = acc[j][k];
    }
    __syncthreads();
    if (g == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[j][k] += red[l][j * 8 + k];
    }
    __syncthreads();
  }
  if (g != 0 || !live) return;
  float* out = dw + (chunks > 1 ? (size_t)blockIdx.y * ne * d : 0);
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (e0 + j < ne) {
      float4* o = reinterpret_cast<float4*>(out + (size_t)(e0 + j) * d + c0);
      if (chunks > 1) {
        o[0] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
        o[1] = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
      } else {
        float4 p0 = o[0], p1 = o[1];
        p0.x += acc[j][0]; p0.y += acc[j][1]; p0.z += acc[j][2]; p0.w += acc[j][3];
        p1.x += acc[j][4]; p1.y += acc[j][5]; p1.z += acc[j][6]; p1.w += acc[j][7];
        o[0] = p0; o[1] = p1;
      }
    }
}

// dw[i] += sum over the chunks of part[z, i], in chunk order: 8 threads per output take a contiguous eighth of the
// chunks each (their loads independent), and the eight partial sums are added in order.
__global__ void __launch_bounds__(256) moe_router_wgrad_fold_kernel(const float* __restrict__ part, float* __restrict__ dw,
                                                                    int chunks, int n) {
  __shared__ float red[8][32];
  const int o = threadIdx.x & 31, q = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + o;
  const int per = (chunks + 7) / 8;
  const int za = q * per, zb = min(chunks, za + per);
  float s = 0.f;
  if (i < n)
    for (int z = za; z < zb; ++z) s += part[(size_t)z * n + i];
  red[q][o] = s;
  __syncthreads();
  if (q == 0 && i < n) {
    float t = red[0][o];
#pragma unroll
    for (int k = 1; k < 8; ++k) t += red[k][o];
    dw[i] += t;
  }
}

}  // namespace gb

using namespace gb;

template <typename T>
static void launch_router_dx(const gb_moe_args& a, int n_slots, dim3 grid, cudaStream_t st) {
  switch (n_slots) {
    case 1: moe_router_dx_kernel<T, 1><<<grid, RD_LANES * RD_GROUPS, 0, st>>>(a); break;
    case 2: moe_router_dx_kernel<T, 2><<<grid, RD_LANES * RD_GROUPS, 0, st>>>(a); break;
    case 3: moe_router_dx_kernel<T, 3><<<grid, RD_LANES * RD_GROUPS, 0, st>>>(a); break;
    case 4: moe_router_dx_kernel<T, 4><<<grid, RD_LANES * RD_GROUPS, 0, st>>>(a); break;
    case 5: moe_router_dx_kernel<T, 5><<<grid, RD_LANES * RD_GROUPS, 0, st>>>(a); break;
    default: moe_router_dx_kernel<T, 6><<<grid, RD_LANES * RD_GROUPS, 0, st>>>(a); break;
  }
}

static int moe_check(const gb_moe_args* a) {
  if (!a || a->n_tok <= 0 || a->d <= 0 || a->d % 8) return -1;
  if (a->ne <= 0 || a->ne > MAX_NE || a->top_k <= 0 || a->top_k > MAX_K || a->top_k > a->ne) return -2;
  if (a->seg_tokens < 0 || (a->seg_tokens > 0 && a->seg_tokens < a->n_tok && a->seg_tokens % blk_tok(a->n_tok))) return -4;
  return 0;
}

extern "C" int gb_moe_seg_ok(int n_tok, int seg_tokens) {
  return seg_tokens > 0 && (seg_tokens >= n_tok || seg_tokens % blk_tok(n_tok) == 0) ? 1 : 0;
}

extern "C" int gb_moe_num_blocks(int n_tok) { return (n_tok + blk_tok(n_tok) - 1) / blk_tok(n_tok); }

extern "C" int gb_moe_capacity(int n_tok, int ne, int top_k, int shared) {
  const long long slots = (long long)n_tok * (top_k + (shared ? 1 : 0));
  const long long cap = slots + (long long)(ne + (shared ? 1 : 0)) * (GB_MOE_PAD - 1);
  return (int)((cap + GB_MOE_PAD - 1) / GB_MOE_PAD * GB_MOE_PAD);
}

#define GB_OK() (gb_launch_rc())

extern "C" int gb_moe_route(const gb_moe_args* a, cudaStream_t st) {
  int rc = moe_check(a);
  if (rc) return rc;
  const int nb = gb_moe_num_blocks(a->n_tok);
  // tensor-core router: up to 8 experts, whole 64-column panels, routing blocks that divide the 128-token tile
  const bool tc = a->status && a->ne <= 8 && a->d % RT_KC == 0 && a->d <= 4096 && a->n_tok >= 256 && blk_tok(a->n_tok) <= RT_TOK &&
                  ((uintptr_t)a->x16 & 15) == 0;
  if (tc) {
    CUtensorMap tm;
    if (gb_make_tmap_2d_16b(&tm, a->x16, (uint64_t)a->n_tok, (uint64_t)a->d, (uint64_t)a->d, RT_TOK, RT_KC, a->is_bf16)) return -20;
    const size_t smem = rt_smem_bytes(a->d, a->ne);
    const unsigned grid = (unsigned)((a->n_tok + RT_TOK - 1) / RT_TOK);
    if (a->is_bf16) {
      auto kern = moe_route_tc_kernel<__nv_bfloat16>;
      static size_t set_b = 0;                   // the attribute only ever grows
      if (smem > set_b) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -10;
        set_b = smem;
      }
      kern<<<grid, RT_THREADS, smem, st>>>(tm, *a, a->status);
    } else {
      auto kern = moe_route_tc_kernel<__half>;
      static size_t set_h = 0;
      if (smem > set_h) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -10;
        set_h = smem;
      }
      kern<<<grid, RT_THREADS, smem, st>>>(tm, *a, a->status);
    }
  }
  const bool vec = a->d % 256 == 0 && a->d <= 1024 && (((uintptr_t)a->x16 | (uintptr_t)a->router_w) & 15) == 0;
#define GB_ROUTE(T)                                                           \
  switch (vec ? a->d / 256 : 0) {                                             \
    case 1: moe_route_kernel<T, 1><<<nb, 256, 0, st>>>(*a); break;            \
    case 2: moe_route_kernel<T, 2><<<nb, 256, 0, st>>>(*a); break;            \
    case 3: moe_route_kernel<T, 3><<<nb, 256, 0, st>>>(*a); break;            \
    case 4: moe_route_kernel<T, 4><<<nb, 256, 0, st>>>(*a); break;            \
    default: moe_route_kernel<T, 0><<<nb, 256, 0, st>>>(*a); break;           \
  }
  if (!tc) {
    if (a->is_bf16) { GB_ROUTE(__nv_bfloat16) } else { GB_ROUTE(__half) }
  }
#undef GB_ROUTE
  if (a->aux_m) {
    const int seg_tok = a->seg_tokens > 0 ? a->seg_tokens : a->n_tok;
    moe_colmean_kernel<<<dim3(a->ne, (a->n_tok + seg_tok - 1) / seg_tok), 256, 0, st>>>(a->probs, a->aux_m, a->n_tok, a->ne,
                                                                                       seg_tok);
  }
  return GB_OK();
}

extern "C" int gb_moe_group(const gb_moe_args* a, cudaStream_t st) {
  int rc = moe_check(a);
  if (rc) return rc;
  const int nb = gb_moe_num_blocks(a->n_tok);
  if (nb > 4096) return -3;
  const int ne1 = a->ne + (a->shared ? 1 : 0);
  const size_t tab_bytes = (size_t)nb * (a->ne + 1) * sizeof(int);
  const int staged = tab_bytes <= 40 * 1024;
  moe_scan_kernel<<<1, 256, staged ? tab_bytes : 0, st>>>(*a, nb, staged);
  const int* totals = a->block_base + (size_t)nb * (a->ne + 1);
  if (a->is_bf16) {
    moe_pack_kernel<__nv_bfloat16><<<nb, 256, 0, st>>>(*a);
    moe_zero_pads_kernel<__nv_bfloat16><<<ne1, 256, 0, st>>>((__nv_bfloat16*)a->x_perm, a->seg_offsets, totals, a->d);
  } else {
    moe_pack_kernel<__half><<<nb, 256, 0, st>>>(*a);
    moe_zero_pads_kernel<__half><<<ne1, 256, 0, st>>>((__half*)a->x_perm, a->seg_offsets, totals, a->d);
  }
  return GB_OK();
}

extern "C" int gb_moe_combine(const gb_moe_args* a, cudaStream_t st) {
  int rc = moe_check(a);
  if (rc) return rc;
  const int grid = (a->n_tok + 7) / 8;
  if (a->is_bf16) moe_combine_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(*a);
  else moe_combine_kernel<__half><<<grid, 256, 0, st>>>(*a);
  return GB_OK();
}

extern "C" int gb_moe_combine_bwd(const gb_moe_args* a, cudaStream_t st) {
  int rc = moe_check(a);
  if (rc) return rc;
  const int nb = gb_moe_num_blocks(a->n_tok);
  const int grid = (a->n_tok + 7) / 8;
  const int ne1 = a->ne + (a->shared ? 1 : 0);
  const int* totals = a->block_base + (size_t)nb * (a->ne + 1);
  if (a->is_bf16) {
    moe_combine_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(*a);
    moe_zero_pads_kernel<__nv_bfloat16><<<ne1, 256, 0, st>>>((__nv_bfloat16*)a->dy_perm, a->seg_offsets, totals, a->d);
  } else {
    moe_combine_bwd_kernel<__half><<<grid, 256, 0, st>>>(*a);
    moe_zero_pads_kernel<__half><<<ne1, 256, 0, st>>>((__half*)a->dy_perm, a->seg_offsets, totals, a->d);
  }
  return GB_OK();
}

extern "C" int gb_moe_router_bwd(const gb_moe_args* a, cudaStream_t st) {
  int rc = moe_check(a);
  if (rc) return rc;
  const int grid = (a->n_tok + 7) / 8;
  // token chunks for the router weight gradient: partials in part2 ([chunks, ne, d]) when it is provided
  int chunks = a->part2 ? (a->n_tok + 31) / 32 : 1;   // 32 tokens per thread: 8192 tokens fill 1536 blocks
  if (chunks > GB_ROUTER_WGRAD_CHUNKS) chunks = GB_ROUTER_WGRAD_CHUNKS;
  dim3 g2((a->d / 8 + RW_LANES - 1) / RW_LANES, chunks, (a->ne + 7) / 8);
  float* wout = chunks > 1 ? a->part2 : a->d_router_w;
  // up to 8 experts: logit gradients first, then the input gradient with the router rows in registers
  const int n_slots = a->top_k + (a->shared ? 1 : 0);
  const bool split = a->ne <= 8 && n_slots <= 6;
  int sms = 0, dev = 0;
  if (split && (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess))
    return -10;
  dim3 gdx(std::max(1, std::min(sms, (a->n_tok + RD_GROUPS - 1) / RD_GROUPS)), (a->d / 8 + RD_LANES - 1) / RD_LANES);   // one resident block per SM
  if (a->is_bf16) {
    if (split) {
      moe_router_dlogit_kernel<<<(a->n_tok + 255) / 256, 256, 0, st>>>(*a);
      launch_router_dx<__nv_bfloat16>(*a, n_slots, gdx, st);
    } else {
      moe_router_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(*a);
    }
    if (a->d_router_w)
      moe_router_wgrad_kernel<__nv_bfloat16><<<g2, RW_LANES * RW_GROUPS, 0, st>>>(a->part, (const __nv_bfloat16*)a->x16, wout, a->n_tok,
                                                                 a->ne, a->d);
  } else {
    if (split) {
      moe_router_dlogit_kernel<<<(a->n_tok + 255) / 256, 256, 0, st>>>(*a);
      launch_router_dx<__half>(*a, n_slots, gdx, st);
    } else {
      moe_router_bwd_kernel<__half><<<grid, 256, 0, st>>>(*a);
    }
    if (a->d_router_w)
      moe_router_wgrad_kernel<__half><<<g2, RW_LANES * RW_GROUPS, 0, st>>>(a->part, (const __half*)a->x16, wout, a->n_tok, a->ne, a->d);
  }
  if (a->d_router_w && chunks > 1) {
    const int n = a->ne * a->d;
    moe_router_wgrad_fold_kernel<<<(n + 31) / 32, 256, 0, st>>>(a->part2, a->d_router_w, chunks, n);
  }
  return GB_OK();
}
