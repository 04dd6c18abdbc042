// Device sampler: repetition / frequency / presence penalties, then greedy arg-max or top-k -> temperature softmax
// -> min-p -> top-p -> renormalise -> draw, in that order (the order of inference/sampler.cpp:119-257 in the
// reference).  One block per sequence.  The uniform number of each draw comes from the host's generator, so a run
// with a fixed seed consumes the same stream as a host-side sampler would.
//
// Top-k: radix select over order-preserving 32-bit keys (four 8-bit passes over the logits) finds the k-th largest
// value; everything at or above it (up to MAX_CAND entries) is sorted by (value descending, index ascending) in
// shared memory, and the first k survive.  The softmax over at most k values runs in double precision on one thread.
#include "sm100_common.cuh"
#include "gb_decode.h"

namespace gb {

constexpr int SM_THREADS = 1024;
constexpr int MAX_CAND = 2048;     // >= the largest supported top_k (1024) plus room for ties at the threshold
constexpr int MAX_WINDOW = 1024;   // penalty window handled on the device

__device__ __forceinline__ unsigned int order_key(float f) {
  unsigned int u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float <=> larger key; NaN sorts above +inf
}

__global__ void __launch_bounds__(SM_THREADS) sample_kernel(gb_sample_args a) {
  pdl_wait();
  __shared__ unsigned int hist[256];
  __shared__ unsigned int s_prefix, s_need, s_count;
  __shared__ float cand_v[MAX_CAND];
  __shared__ int cand_i[MAX_CAND];
  __shared__ float red_v[32];
  __shared__ int red_i[32];
  __shared__ int s_tok;
  const int b = blockIdx.x, tid = threadIdx.x;
  float* lg = const_cast<float*>(a.logits) + (long long)b * a.ld;
  const int V = a.V;

  // ---- penalties over the last `rep_window` tokens of this sequence's history (each distinct token once)
  const int hl = a.hist_len ? a.hist_len[b] : 0;
  const bool pen = hl > 0 && (a.rep_penalty != 1.f || a.freq_penalty != 0.f || a.presence_penalty != 0.f);
  if (pen) {
    int win = a.rep_window > 0 ? min(hl, a.rep_window) : hl;
    win = min(win, MAX_WINDOW);
    const int* h = a.history + (long long)b * a.hist_cap + (hl - win);
    for (int i = tid; i < win; i += SM_THREADS) {
      const int t = h[i];
      if (t < 0 || t >= V) continue;
      bool first = true;
      int n = 0;
      for (int j = 0; j < win; ++j) {
        if (h[j] == t) {
          if (j < i) { first = false; break; }
          ++n;
        }
      }
      if (!first) continue;
      float l = lg[t];
      if (a.rep_penalty != 1.f) l = l > 0.f ? l / a.rep_penalty : l * a.rep_penalty;
      if (a.freq_penalty != 0.f) l -= a.freq_penalty * (float)n;
      if (a.presence_penalty != 0.f) l -= a.presence_penalty;
      lg[t] = l;
    }
    __syncthreads();
  }

  const bool greedy = a.greedy || !(a.temperature > 0.f) || a.top_k == 1;
  if (greedy) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < V; i += SM_THREADS) {
      const float v = lg[i];
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_down_sync(0xffffffffu, bv, o);
      const int oi = __shfl_down_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { red_v[tid >> 5] = bv; red_i[tid >> 5] = bi; }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < SM_THREADS / 32; ++w)
        if (red_v[w] > bv || (red_v[w] == bv && red_i[w] < bi)) { bv = red_v[w]; bi = red_i[w]; }
      s_tok = bi == 0x7fffffff ? 0 : bi;
    }
    __syncthreads();
  } else {
    const int k = min(min(a.top_k > 0 ? a.top_k : 1024, 1024), V);
    // ---- radix select: key of the k-th largest logit
    if (tid == 0) { s_prefix = 0; s_need = (unsigned)k; }
    __syncthreads();
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      const unsigned int prefix = s_prefix;
      const unsigned int mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
      for (int i = tid; i < V; i += SM_THREADS) {
        const unsigned int key = order_key(lg[i]);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xFF], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned int need = s_need, bin = 255;
        for (;; --bin) {   // walk from the largest bin down until the k-th element is inside
          if (hist[bin] >= need || bin == 0) break;
          need -= hist[bin];
        }
        s_need = need;
        s_prefix = prefix | (bin << shift);
      }
      __syncthreads();
    }
    const unsigned int thr = s_prefix;
    if (tid == 0) s_count = 0;
    __syncthreads();
    for (int i = tid; i < V; i += SM_THREADS) {
      const float v = lg[i];
      if (order_key(v) >= thr) {
        const unsigned int at = atomicAdd(&s_count, 1u);
        if (at < MAX_CAND) { cand_v[at] = v; cand_i[at] = i; }
      }
    }
    __syncthreads();
    const int n = min((int)s_count, MAX_CAND);
    for (int i = n + tid; i < MAX_CAND; i += SM_THREADS) { cand_v[i] = -INFINITY; cand_i[i] = 0x7fffffff; }
    __syncthreads();
    // ---- bitonic sort, descending by value then ascending by index
    for (int size = 2; size <= MAX_CAND; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int t = tid; t < MAX_CAND / 2; t += SM_THREADS) {
          const int lo = 2 * t - (t & (stride - 1));
          const int hi = lo + stride;
          const bool desc = (lo & size) == 0;
          const float v0 = cand_v[lo], v1 = cand_v[hi];
          const int i0 = cand_i[lo], i1 = cand_i[hi];
          const bool first_is_better = v0 > v1 || (v0 == v1 && i0 < i1);
          if (first_is_better != desc) {
            cand_v[lo] = v1; cand_v[hi] = v0;
            cand_i[lo] = i1; cand_i[hi] = i0;
          }
        }
        __syncthreads();
      }
    }
    if (tid == 0) {
      const int m = min(k, n);
      const float inv_t = 1.f / a.temperature;
      const float mx = cand_v[0];
      double sum = 0.0;
      for (int i = 0; i < m; ++i) sum += exp((double)((cand_v[i] - mx) * inv_t));
      int tok = cand_i[0];
      if (isfinite(sum) && sum > 0.0) {
        // probabilities are recomputed on the fly instead of stored: p_i = exp(...) / sum
        int limit = m;
        if (a.min_p > 0.f) {
          const double thresh = (double)a.min_p * (1.0 / sum);   // p_0 = exp(0)/sum
          int c = 0;
          while (c < m && exp((double)((cand_v[c] - mx) * inv_t)) / sum >= thresh) ++c;
          limit = max(1, c);
        }
        if (a.top_p > 0.f && a.top_p < 1.f) {
          double cum = 0.0;
          int c = 0;
          while (c < limit) {
            cum += exp((double)((cand_v[c] - mx) * inv_t)) / sum;
            ++c;
            if (cum >= (double)a.top_p) break;
          }
          limit = max(1, c);
        }
        double renorm = 0.0;
        for (int i = 0; i < limit; ++i) renorm += exp((double)((cand_v[i] - mx) * inv_t)) / sum;
        // with a device step counter the draws of a whole run sit in one [steps, B] table filled ahead of time
        int ustep = a.step ? a.step[0] : 0;
        if (a.step && ustep >= a.log_cap) ustep = a.log_cap - 1;
        const double r = (double)a.uniforms[(long long)ustep * a.B + b] * renorm;
        double acc = 0.0;
        tok = cand_i[limit - 1];
        for (int i = 0; i < limit; ++i) {
          acc += exp((double)((cand_v[i] - mx) * inv_t)) / sum;
          if (r <= acc) { tok = cand_i[i]; break; }
        }
      }
      s_tok = tok;
    }
    __syncthreads();
  }

  if (tid == 0) {
    const int tok = s_tok;
    a.out_tok[b] = tok;
    if (a.hist_len && hl < a.hist_cap) {
      const_cast<int*>(a.history)[(long long)b * a.hist_cap + hl] = tok;
      a.hist_len[b] = hl + 1;
    }
    if (a.state) {
      for (int i = 0; i < a.n_stop; ++i)
        if (a.stop[i] == tok) a.state[b].done = 1;
    }
    if (a.tok_log && a.step) {
      const int s = a.step[0];
      if (s >= 0 && s < a.log_cap) a.tok_log[(long long)b * a.log_cap + s] = tok;
    }
  }
}

__global__ void step_inc_kernel(int* step) {
  pdl_wait();
  step[0] += 1;
}

}  // namespace gb

extern "C" int gb_sample(const gb_sample_args* a, cudaStream_t st) {
  if (!a || !a->logits || !a->out_tok || a->B <= 0 || a->V <= 0) return -1;
  const bool greedy = a->greedy || !(a->temperature > 0.f) || a->top_k == 1;
  if (!greedy && (!a->uniforms || a->top_k <= 0 || a->top_k > 1024)) return -2;   // unbounded / larger candidate sets: host sampler
  if (a->n_stop > 0 && !a->stop) return -1;
  GB_PDL_LAUNCH(gb::sample_kernel, dim3(a->B), dim3(gb::SM_THREADS), st, *a);
  if (a->tok_log && a->step) GB_PDL_LAUNCH(gb::step_inc_kernel, dim3(1), dim3(1), st, const_cast<int*>(a->step));
  return gb_launch_rc();
}
