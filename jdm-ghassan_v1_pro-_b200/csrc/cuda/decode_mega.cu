// The whole token step of one sequence as ONE cooperative kernel: embedding row, every layer (RMSNorm + fused QKV
// projection, QK-norm + RoPE + cache append + split-KV attention, merge + output projection + residual, RMSNorm +
// router + gate/up + SwiGLU of the selected experts, down projection + residual), final norm and the vocabulary
// projection.  One CTA of 16 warps per SM; the phases of a layer are separated by grid-wide barriers (five per layer)
// instead of kernel boundaries (eight per layer in decode.cu), and every warp starts the bulk asynchronous copies of
// the weight rows of its next piece of work into shared memory BEFORE it arrives at the barrier: the weights do not
// depend on the activations, so their DRAM round trip hides behind the barrier instead of following it.  The reference's decode loop (inference/generator.cpp:97-193,
// cuda/kernels.cu:876-1019) launches about fifteen kernels per layer.
//
// Work split.  Output rows of a projection are dealt to the CTAs round robin (row r belongs to CTA r mod grid); inside
// a CTA a row goes to one warp, or, when the CTA has fewer rows than warps, to KS warps that split the row's K range
// and meet in shared memory.  Rows are read in "super-units" of 256 stored values: a whole number of quantisation
// blocks in every format (512 B fp16/bf16, 272 B Q8_0, 144 B Q4_0, 272 B Q8_0(64), 160 B Q4_1) and a multiple of 16 bytes,
// so a run of super-units is one bulk copy and lane l expands values 8l..8l+7 of a super-unit from shared memory.
// (The vocabulary projection, too many rows per CTA to stage, pulls its rows through registers instead.)
//
// Every wait is bounded: a grid barrier that does not open within about two seconds writes status 401, a copy that
// never signals its mbarrier 402; the CTA then skips the rest of the step (the others follow when their own waits run
// out) and waits, again bounded, for its copies in flight before it leaves.  The launch is cooperative, so either all CTAs are
// resident or the launch fails.
#include <algorithm>
#include <type_traits>

#include "sm100_common.cuh"
#include "gb_decode.h"
#include "decode_fmt.cuh"

namespace gb {
namespace mg {

constexpr int WARPS = 16;
constexpr int THREADS = WARPS * 32;
constexpr int GROUP = 4;              // super-units a warp keeps in flight
constexpr int SU = 256;               // values per super-unit
constexpr int MAX_SLOTS = 9;          // top_k <= 8 routed experts plus the shared one
constexpr int MAX_HEADS = 128;
constexpr int ST_TIMEOUT_GRID = 401;
constexpr int ST_TIMEOUT_COPY = 402;      // a bulk copy of weight rows never signalled its barrier

template <int FMT> struct Fmt {
  static constexpr bool k16 = FMT == GB_W_F16 || FMT == GB_W_BF16;
  static constexpr int bytes = k16 ? 512 : FMT == GB_W_GGML_Q8_0 ? 272 : FMT == GB_W_Q4_0 ? 144 : FMT == GB_W_Q8_64 ? 272 : 160;
  static constexpr int words = bytes / 16;    // 16-byte words per super-unit (<= 32: one per lane)
};

__device__ __forceinline__ uint4 ld_stream(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
template <typename XT> __device__ __forceinline__ float ld16(const XT* p) {       // L2 read of one 16-bit activation
  const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(p));
  if constexpr (std::is_same<XT, __half>::value) return __half2float(__ushort_as_half(u));
  else return __bfloat162float(__ushort_as_bfloat16(u));
}

// ------------------------------------------------------------------------------------------------ grid barrier
// Arrivals are counted in sync[0], which only ever grows; barrier k of a launch opens at base + k * grid, where base
// (sync[1]) is the count the previous launch left behind.
struct GridBar {
  unsigned* cnt;
  int* status;
  int* dead;          // shared memory: set once a wait of this CTA ran out
  unsigned next;      // count at which the next barrier opens
};

__device__ __forceinline__ bool grid_sync(GridBar& gb) {
  __syncthreads();
  if (threadIdx.x == 0 && !*gb.dead) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(gb.cnt), "r"(1u) : "memory");
    unsigned it = 0;
    unsigned long long t0 = 0;
    for (;;) {
      // A relaxed load on purpose.  An acquire at GPU scope empties this SM's L1, and with it the registers the kernel
      // has spilled to local memory: every phase then began with their reload from L2 (ncu: 65 % of the local loads
      // missed L1).  What other CTAs wrote before they arrived is read with ld.global.cg or by bulk copies, both of
      // which go to L2 and never to this L1, and the writers release (red.release.gpu) after their stores; the
      // __syncthreads below keeps every thread's reads behind thread 0's observation of the count.
      unsigned v;
      asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(gb.cnt) : "memory");
      if ((int)(v - gb.next) >= 0) break;
      ++it;
      if (it == 2048) t0 = globaltimer_ns();
      if (it > 2048) {
        __nanosleep(64);
        if ((it & 1023) == 0 && globaltimer_ns() - t0 > 2000000000ull) {
          *gb.dead = 1;
          atomicCAS(gb.status, 0, ST_TIMEOUT_GRID);
          break;
        }
      }
    }
  }
  gb.next += gridDim.x;
  __syncthreads();
  return !*gb.dead;
}

// ------------------------------------------------------------------------------------------------ row engine
// One projection phase: every output is a sum over P super-units.  Super-unit p of an output lives at
//   W + row_off(output) + off[p / nsu] + (p % nsu) * bytes,
// is multiplied with the 256 activations at xs + (x_mod ? p % nsu : p) * 256, weighted by wt[p / nsu], and added to
// accumulator (acc_split ? p / nsu : 0).  That covers a plain row (off, wt absent), a gate/up pair (two rows, two
// accumulators) and the down projection of several experts into one output (one stored row per slot, weighted).
struct Phase {
  const uint8_t* W;
  const long long* off;
  const float* wt;
  int nsu, P;
  bool x_mod, acc_split;
};

// Which outputs of the CTA a warp computes: local output i = first + k * stride for k < n, super-units [pb, pe).
struct Plan {
  int n, first, stride, KS, rows, pb, pe;
};
__device__ __forceinline__ Plan make_plan(int N, int P) {
  const int warp = threadIdx.x >> 5;
  const int grid = gridDim.x, cta = blockIdx.x;
  Plan pl;
  pl.rows = N > cta ? (N - cta + grid - 1) / grid : 0;
  pl.KS = 1; pl.first = warp; pl.stride = WARPS; pl.pb = 0; pl.pe = P; pl.n = 0;
  if (pl.rows == 0) return pl;
  const int ks = min(P, WARPS / pl.rows);
  if (ks >= 2) {
    pl.KS = ks;
    pl.first = warp / ks;
    const int k = warp - pl.first * ks;
    pl.pb = k * P / ks;
    pl.pe = (k + 1) * P / ks;
    pl.n = pl.first < pl.rows ? 1 : 0;
  } else {
    pl.n = warp < pl.rows ? (pl.rows - warp + WARPS - 1) / WARPS : 0;
  }
  return pl;
}

template <int FMT>
__device__ __forceinline__ void load_group(const Phase& ph, const uint8_t* row, int p0, int pe, uint4 (&r)[GROUP]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < GROUP; ++i) {
    const int p = p0 + i;
    if (p < pe && lane < Fmt<FMT>::words) {
      const int s = p / ph.nsu, su = p - s * ph.nsu;
      r[i] = ld_stream(row + (ph.off ? ph.off[s] : 0ll) + (long long)su * Fmt<FMT>::bytes + 16 * lane);
    }
  }
}

template <int FMT, typename XT>
__device__ __forceinline__ float su_dot(const uint4& q, const uint8_t* slot, const XT* __restrict__ x) {
  const int lane = threadIdx.x & 31;
  float w[8];
  if constexpr (FMT == GB_W_F16) {
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); w[2 * i] = f.x; w[2 * i + 1] = f.y; }
  } else if constexpr (FMT == GB_W_BF16) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); w[2 * i] = f.x; w[2 * i + 1] = f.y; }
  } else {
    load8<FMT>(slot, lane, w);
  }
  const uint4 xv = *reinterpret_cast<const uint4*>(x + 8 * lane);
  float s = 0.f;
  const uint32_t* xu = reinterpret_cast<const uint32_t*>(&xv);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = Cvt<XT>::unpack2(xu[i]); s += w[2 * i] * f.x + w[2 * i + 1] * f.y; }
  return s;
}

template <int FMT, typename XT>
__device__ __forceinline__ void dot_group(const Phase& ph, const XT* xs, int p0, int pe, const uint4 (&r)[GROUP], uint8_t* stage,
                                          float (&acc)[2]) {
  const int lane = threadIdx.x & 31;
  if constexpr (!Fmt<FMT>::k16) {
#pragma unroll
    for (int i = 0; i < GROUP; ++i)
      if (p0 + i < pe && lane < Fmt<FMT>::words) *reinterpret_cast<uint4*>(stage + i * Fmt<FMT>::bytes + 16 * lane) = r[i];
    __syncwarp();
  }
#pragma unroll
  for (int i = 0; i < GROUP; ++i) {
    const int p = p0 + i;
    if (p < pe) {
      const int s = p / ph.nsu, su = p - s * ph.nsu;
      const float v = su_dot<FMT, XT>(r[i], stage + i * Fmt<FMT>::bytes, xs + (ph.x_mod ? su : p) * SU);
      if (ph.acc_split && s == 1) acc[1] += v;
      else acc[0] += (ph.wt ? ph.wt[s] : 1.f) * v;
    }
  }
  if constexpr (!Fmt<FMT>::k16) __syncwarp();
}

// The first group of the warp's first output, issued before the barrier that precedes the phase.
template <int FMT, class RowOff>
__device__ __forceinline__ void preload(const Phase& ph, const Plan& pl, RowOff row_off, uint4 (&cur)[GROUP]) {
  if (pl.n > 0) load_group<FMT>(ph, ph.W + row_off(blockIdx.x + pl.first * (int)gridDim.x), pl.pb, pl.pe, cur);
}

// Runs the warp's outputs.  row_off(o): byte offset of output o's stored row; epi(o, a0, a1): called by one thread
// per finished output.  `cur` holds the preloaded first group.
template <int FMT, typename XT, class RowOff, class Epi>
__device__ __forceinline__ void run_phase(const Phase& ph, const Plan& pl, const XT* xs, uint8_t* stage, float (*red)[WARPS],
                                          uint4 (&cur)[GROUP], RowOff row_off, Epi epi) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grid = gridDim.x, cta = blockIdx.x;
  const int gpi = (pl.pe - pl.pb + GROUP - 1) / GROUP;
  const int total = pl.n * gpi;
  float acc[2] = {0.f, 0.f};
  int k = 0, g = 0;
  for (int t = 0; t < total; ++t) {
    uint4 nxt[GROUP];
    int k2 = k, g2 = g + 1;
    if (g2 == gpi) { g2 = 0; ++k2; }
    if (t + 1 < total)
      load_group<FMT>(ph, ph.W + row_off(cta + (pl.first + k2 * pl.stride) * grid), pl.pb + GROUP * g2, pl.pe, nxt);
    dot_group<FMT, XT>(ph, xs, pl.pb + GROUP * g, pl.pe, cur, stage, acc);
    if (g == gpi - 1) {
      const float a0 = warp_sum(acc[0]);
      const float a1 = ph.acc_split ? warp_sum(acc[1]) : 0.f;
      if (lane == 0) {
        if (pl.KS == 1) epi(cta + (pl.first + k * pl.stride) * grid, a0, a1);
        else { red[0][warp] = a0; red[1][warp] = a1; }
      }
      acc[0] = acc[1] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < GROUP; ++i) cur[i] = nxt[i];
    k = k2; g = g2;
  }
  if (pl.KS > 1) {                        // uniform over the CTA: rows and P are
    __syncthreads();
    if ((int)threadIdx.x < pl.rows) {
      float a0 = 0.f, a1 = 0.f;
      for (int j = 0; j < pl.KS; ++j) { a0 += red[0][threadIdx.x * pl.KS + j]; a1 += red[1][threadIdx.x * pl.KS + j]; }
      epi(cta + (int)threadIdx.x * grid, a0, a1);
    }
  }
}

// ------------------------------------------------------------------------------------------------ row streaming
// The layer phases do not pull their rows through registers: lane 0 of a warp issues one bulk asynchronous copy per
// contiguous run of super-units of ALL the warp's work in the phase into the warp's own slice of shared memory (no
// other warp touches it), signalled on the warp's own mbarriers, and it does so right after the warp has finished the
// phase before: the weights of a phase are in flight while the previous phase's results cross the grid barrier.
constexpr int MAXI = 4;               // outputs a warp stages at once (checked on the host)
constexpr int MAX_DYN = 220 * 1024;   // dynamic shared memory the kernel may ask for (227 KB per CTA, 3 KB static)

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}

struct Stage {
  uint8_t* base;        // this warp's slice
  uint64_t* bars;       // this warp's MAXI barriers
  uint32_t parity;      // bit k: parity that the next completion of bars[k] is waited with
  uint32_t pending;     // bit k: a copy onto bars[k] was issued and not yet waited for
  int* dead;
  int* status;
};

// Per-warp bytes of the staging slice for one phase: N outputs of P super-units each, dealt as make_plan does.
__host__ __device__ inline long long stage_need(long long N, int P, int grid, int su_bytes, int* items_out) {
  const long long rows = (N + grid - 1) / grid;
  long long items = 1, sus = P;
  if (rows == 0) { if (items_out) *items_out = 0; return 0; }
  const int ks = (int)(WARPS / rows) < P ? (int)(WARPS / rows) : P;
  if (ks >= 2) sus = (P + ks - 1) / ks;
  else items = (rows + WARPS - 1) / WARPS;
  if (items_out) *items_out = (int)items;
  return items * sus * su_bytes;
}

template <int FMT, class RowOff>
__device__ __forceinline__ void stream_issue(const Phase& ph, const Plan& pl, Stage& st, RowOff row_off) {
  constexpr int SB = Fmt<FMT>::bytes;
  __syncwarp();                                  // every lane has finished reading the slice
  if (pl.n > 0 && !*st.dead) st.pending |= (1u << pl.n) - 1u;
  if ((threadIdx.x & 31) == 0 && !*st.dead) {
    fence_proxy_async();                         // those reads are ordered before the copies that overwrite them
    const int item_bytes = (pl.pe - pl.pb) * SB;
    for (int k = 0; k < pl.n; ++k) {
      const uint8_t* row = ph.W + row_off((int)blockIdx.x + (pl.first + k * pl.stride) * (int)gridDim.x);
      uint8_t* dst = st.base + (size_t)k * item_bytes;
      mbar_arrive_expect_tx(st.bars + k, (uint32_t)item_bytes);
      for (int p = pl.pb; p < pl.pe;) {
        const int s = p / ph.nsu, su = p - s * ph.nsu;
        const int run = min(pl.pe - p, ph.nsu - su);
        bulk_g2s(smem_u32(dst + (size_t)(p - pl.pb) * SB), row + (ph.off ? ph.off[s] : 0ll) + (long long)su * SB,
                 (uint32_t)(run * SB), smem_u32(st.bars + k));
        p += run;
      }
    }
  }
}

template <int FMT, typename XT, class Epi>
__device__ __forceinline__ void stream_run(const Phase& ph, const Plan& pl, const XT* xs, Stage& st, float (*red)[WARPS], Epi epi) {
  constexpr int SB = Fmt<FMT>::bytes;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grid = gridDim.x, cta = blockIdx.x;
  const int item_bytes = (pl.pe - pl.pb) * SB;
  for (int k = 0; k < pl.n; ++k) {
    const bool got = mbar_wait(st.bars + k, (st.parity >> k) & 1u);
    if (!got) {                                  // bounded: the copy never landed
      if (lane == 0) { *st.dead = 1; atomicCAS(st.status, 0, ST_TIMEOUT_COPY); }
      break;
    }
    st.parity ^= 1u << k;
    st.pending &= ~(1u << k);
    const uint8_t* src = st.base + (size_t)k * item_bytes;
    float acc[2] = {0.f, 0.f};
    for (int p = pl.pb; p < pl.pe; ++p) {
      const int s = p / ph.nsu, su = p - s * ph.nsu;
      const uint8_t* slot = src + (size_t)(p - pl.pb) * SB;
      uint4 q = make_uint4(0u, 0u, 0u, 0u);
      if constexpr (Fmt<FMT>::k16) q = *reinterpret_cast<const uint4*>(slot + 16 * lane);
      const float v = su_dot<FMT, XT>(q, slot, xs + (ph.x_mod ? su : p) * SU);
      if (ph.acc_split && s == 1) acc[1] += v;
      else acc[0] += (ph.wt ? ph.wt[s] : 1.f) * v;
    }
    const float a0 = warp_sum(acc[0]);
    const float a1 = ph.acc_split ? warp_sum(acc[1]) : 0.f;
    if (lane == 0) {
      if (pl.KS == 1) epi(cta + (pl.first + k * pl.stride) * grid, a0, a1);
      else { red[0][warp] = a0; red[1][warp] = a1; }
    }
  }
  if (pl.KS > 1) {                               // uniform over the CTA
    __syncthreads();
    if ((int)threadIdx.x < pl.rows) {
      float a0 = 0.f, a1 = 0.f;
      for (int j = 0; j < pl.KS; ++j) { a0 += red[0][threadIdx.x * pl.KS + j]; a1 += red[1][threadIdx.x * pl.KS + j]; }
      epi(cta + (int)threadIdx.x * grid, a0, a1);
    }
  }
}

// ------------------------------------------------------------------------------------------------ pieces
// RMSNorm of an fp32 row in global memory into 16-bit shared memory, by the whole CTA.
template <typename XT>
__device__ __forceinline__ void block_norm(const float* x, const float* __restrict__ w, XT* xs, int d, float eps, float* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // d <= 4 * THREADS * 2: at most two float4 per thread, read once and kept
  float4 v[2];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int i = threadIdx.x + k * THREADS;
    v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < d / 4) v[k] = __ldcg(reinterpret_cast<const float4*>(x) + i);
    ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  }
  float4 g[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int i = threadIdx.x + k * THREADS;
    g[k] = i < d / 4 ? reinterpret_cast<const float4*>(w)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < WARPS; ++i) tot += red[i];
  float inv = rsqrtf(tot / (float)d + eps);
  if (!isfinite(inv)) inv = 0.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int i = threadIdx.x + k * THREADS;
    if (i < d / 4) {
      uint2 o;
      o.x = Cvt<XT>::pack2(v[k].x * inv * g[k].x, v[k].y * inv * g[k].y);
      o.y = Cvt<XT>::pack2(v[k].z * inv * g[k].z, v[k].w * inv * g[k].w);
      *reinterpret_cast<uint2*>(xs + 4 * i) = o;
    }
  }
  __syncthreads();
}

// QK-norm + rotation of one head by one warp (the arithmetic of qk_rope_append_kernel in decode.cu); st(i, value).
template <typename XT, class Store>
__device__ __forceinline__ void rope_head(const XT* src, const float* __restrict__ w, const float* __restrict__ csr, int hd, int rope_type,
                                          float eps, Store st) {
  const int lane = threadIdx.x & 31;
  const int pairs = hd / 2;
  float a[2], b[2];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int p = lane + 32 * k;
    a[k] = b[k] = 0.f;
    if (p < pairs) {
      const int i0 = rope_type == 0 ? 2 * p : p, i1 = rope_type == 0 ? 2 * p + 1 : p + pairs;
      a[k] = ld16<XT>(src + i0);
      b[k] = ld16<XT>(src + i1);
      ss += a[k] * a[k] + b[k] * b[k];
    }
  }
  float inv = 1.f;
  if (w) {
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)hd + eps);
    if (!isfinite(inv)) inv = 0.f;
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int p = lane + 32 * k;
    if (p < pairs) {
      const int i0 = rope_type == 0 ? 2 * p : p, i1 = rope_type == 0 ? 2 * p + 1 : p + pairs;
      float x0 = a[k], x1 = b[k];
      if (w) { x0 *= inv * w[i0]; x1 *= inv * w[i1]; }
      const float c = csr[p], sn = csr[pairs + p];
      st(i0, x0 * c - x1 * sn);
      st(i1, x0 * sn + x1 * c);
    }
  }
}

// epl (1, 2 or 4) consecutive 16-bit values of a cache row
template <typename XT>
__device__ __forceinline__ void ld_epl(const XT* p, int epl, float (&f)[4]) {
  if (epl == 2) {
    const float2 v = Cvt<XT>::unpack2(__ldcg(reinterpret_cast<const unsigned int*>(p)));
    f[0] = v.x; f[1] = v.y;
  } else if (epl == 4) {
    const uint2 u = __ldcg(reinterpret_cast<const uint2*>(p));
    const float2 v0 = Cvt<XT>::unpack2(u.x), v1 = Cvt<XT>::unpack2(u.y);
    f[0] = v0.x; f[1] = v0.y; f[2] = v1.x; f[3] = v1.y;
  } else {
    f[0] = ld16<XT>(p);
  }
}

struct Smem {          // static shared memory of the kernel
  float red[2][WARPS];
  float lg[64];
  float linv[MAX_HEADS];
  float q[4][128];
  long long off_e[MAX_SLOTS];
  long long off_gu[2];
  float wsel[MAX_SLOTS];
  int esel[MAX_SLOTS];
  int dead;
};

// ------------------------------------------------------------------------------------------------ attention
// CTA `item` < KV * S serves key/value head item % KV over slots [lo, hi) of the cache (split item / KV): all query
// heads of the group in one walk.  The CTA whose range holds the step's own slot writes the new K (normalised,
// rotated) and V there first.  Partial (max, sum, output) per (head, split) go to `scratch`.
template <typename XT>
__device__ __noinline__ void attention_phase(const gb_mega_args& a, const gb_mega_layer& L, int S, Smem& sm, float* amerge,
                                             const gb_seq_state s, int pos_now, unsigned long long*& prof) {
  const int item = blockIdx.x;
  if (item >= a.KV * S) {
    if (prof) { const unsigned long long t = globaltimer_ns(); *prof++ = t; *prof++ = t; }
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hd = a.hd, G = a.H / a.KV, epl = hd / 32;
  const int kvh = item % a.KV, split = item / a.KV;
  const int n_slots = min(a.cap, s.cache_len + 1);       // s: the sequence state, read once per step by the caller
  const int slot_new = s.cache_len < a.cap ? s.cache_len : a.pinned + s.ring_start;
  const int per = (n_slots + S - 1) / S;
  const int lo = split * per, hi = min(n_slots, lo + per);
  const bool owner = slot_new >= lo && slot_new < hi;
  const XT* qkv = reinterpret_cast<const XT*>(a.qkv);
  const long long kvd = (long long)a.KV * hd;
  XT* cK = reinterpret_cast<XT*>(L.cache_k);
  XT* cV = reinterpret_cast<XT*>(L.cache_v);
  const float* csr = a.cos_sin + (size_t)pos_now * hd;
  float* am = amerge;                         // [WARPS][4]
  float* al = amerge + WARPS * 4;             // [WARPS][4]
  float* ao = amerge + WARPS * 8;             // [WARPS][4][hd]

  for (int g0 = 0; g0 < G; g0 += 4) {
    const int gc = min(4, G - g0);
    if (warp < gc) {
      float* qd = sm.q[warp];
      const float scale = a.scale;
      rope_head<XT>(qkv + (size_t)(kvh * G + g0 + warp) * hd, L.q_norm, csr, hd, a.rope_type, a.eps,
                    [&](int i, float v) { qd[i] = Cvt<XT>::to_f(Cvt<XT>::from_f(v)) * scale; });
    } else if (g0 == 0 && owner && warp == 4) {
      XT* dk = cK + (size_t)slot_new * kvd + (size_t)kvh * hd;
      rope_head<XT>(qkv + (size_t)(a.H + kvh) * hd, L.k_norm, csr, hd, a.rope_type, a.eps,
                    [&](int i, float v) { dk[i] = Cvt<XT>::from_f(v); });
      if (kvh == 0 && lane == 0) a.slot_pos[slot_new] = s.abs_pos;
    } else if (g0 == 0 && owner && warp == 5) {
      const XT* sv = qkv + (size_t)(a.H + a.KV + kvh) * hd;
      XT* dv = cV + (size_t)slot_new * kvd + (size_t)kvh * hd;
      for (int i = lane * 2; i < hd; i += 64)
        *reinterpret_cast<unsigned int*>(dv + i) = __ldcg(reinterpret_cast<const unsigned int*>(sv + i));
    }
    __syncthreads();
    if (prof && g0 == 0) *prof++ = globaltimer_ns();          // queries rotated, the step's key and value stored

    float qv[4][4], m[4], l[4], o[4][4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o[g][e] = 0.f;
        qv[g][e] = (g < gc && e < epl) ? sm.q[g][lane * epl + e] : 0.f;
      }
    }
    auto live = [&](int j) {
      if (j >= hi) return false;
      if (a.window <= 0 || j == slot_new) return true;
      return s.abs_pos - __ldcg(a.slot_pos + j) < a.window;
    };
    for (int j = lo + warp; j < hi; j += 4 * WARPS) {
      bool ok[4];
      float kf[4][4], vf[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int ju = j + u * WARPS;
        ok[u] = live(ju);
#pragma unroll
        for (int e = 0; e < 4; ++e) kf[u][e] = vf[u][e] = 0.f;
        if (ok[u]) {
          ld_epl<XT>(cK + (size_t)ju * kvd + (size_t)kvh * hd + lane * epl, epl, kf[u]);
          ld_epl<XT>(cV + (size_t)ju * kvd + (size_t)kvh * hd + lane * epl, epl, vf[u]);
        }
      }
      // the dot products of all four slots with all heads of the group first, reduced over the lanes together (sixteen
      // independent shuffles per step instead of one chain per slot and head), then the soft-max updates in slot order
      float dots[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float dsum = 0.f;
#pragma unroll
          for (int e = 0; e < 4; ++e) if (e < epl) dsum += qv[g][e] * kf[u][e];
          dots[u][g] = dsum;
        }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int g = 0; g < 4; ++g) dots[u][g] += __shfl_xor_sync(0xffffffffu, dots[u][g], off);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (!ok[u]) continue;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (g < gc) {
            const float dsum = dots[u][g];
            const float mn = fmaxf(m[g], dsum);
            const float c = __expf(m[g] - mn), p = __expf(dsum - mn);
            l[g] = l[g] * c + p;
#pragma unroll
            for (int e = 0; e < 4; ++e) if (e < epl) o[g][e] = o[g][e] * c + p * vf[u][e];
            m[g] = mn;
          }
        }
      }
    }
    if (prof && g0 == 0) *prof++ = globaltimer_ns();          // this warp's slots walked
    // the sixteen warps meet in shared memory, in warp order
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g < gc) {
        if (lane == 0) { am[warp * 4 + g] = m[g]; al[warp * 4 + g] = l[g]; }
#pragma unroll
        for (int e = 0; e < 4; ++e) if (e < epl) ao[(size_t)(warp * 4 + g) * hd + lane * epl + e] = o[g][e];
      }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < gc * hd; t += THREADS) {
      const int g = t / hd, c = t - g * hd;
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, am[w * 4 + g]);
      float ll = 0.f, oo = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float mw = am[w * 4 + g];
        const float f = mw == -INFINITY ? 0.f : __expf(mw - mm);
        ll += al[w * 4 + g] * f;
        oo += ao[(size_t)(w * 4 + g) * hd + c] * f;
      }
      float* dst = a.att_scratch + ((size_t)(kvh * G + g0 + g) * S + split) * (hd + 2);
      dst[2 + c] = oo;
      if (c == 0) { dst[0] = mm; dst[1] = ll; }
    }
    __syncthreads();
  }
}

// Every CTA merges the S partial results of all heads into the 16-bit attention output in shared memory.
template <typename XT>
__device__ __forceinline__ void merge_phase(const gb_mega_args& a, int S, Smem& sm, float* ftab, XT* xs, float* part,
                                            unsigned long long*& prof) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hd = a.hd, st = hd + 2;
  for (int h = warp; h < a.H; h += WARPS) {
    const float* base = a.att_scratch + (size_t)h * S * st;
    // S <= 64: at most two splits per lane, (max, sum) read once
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    if (lane < S) { const float2 t = __ldcg(reinterpret_cast<const float2*>(base + (size_t)lane * st)); m0 = t.x; l0 = t.y; }
    if (lane + 32 < S) { const float2 t = __ldcg(reinterpret_cast<const float2*>(base + (size_t)(lane + 32) * st)); m1 = t.x; l1 = t.y; }
    const float M = warp_max(fmaxf(m0, m1));
    const float f0 = m0 == -INFINITY ? 0.f : __expf(m0 - M), f1 = m1 == -INFINITY ? 0.f : __expf(m1 - M);
    if (lane < S) ftab[h * S + lane] = f0;
    if (lane + 32 < S) ftab[h * S + lane + 32] = f1;
    const float ls = warp_sum(l0 * f0 + l1 * f1);
    if (lane == 0) sm.linv[h] = ls;
  }
  __syncthreads();
  if (prof) *prof++ = globaltimer_ns();                       // factors of every (head, split)
  const int qd = a.H * hd;
  if (2 * qd <= WARPS * 8 + WARPS * 4 * hd) {
    // two threads per output, each over half of the splits, all loads of a half in flight at once; the halves meet in
    // shared memory (the attention phase's merge area, free by now)
    const int half = (S + 1) / 2;
    // a thread's items are THREADS apart; the partial outputs of up to three items (twelve splits each) are fetched
    // before any is used, so that one memory round trip covers them all; larger cases go through the loops again
    // Every CTA reads all partial outputs.  Walking them in the same order at the same time would put all 148 SMs on
    // the same few L2 lines at every moment, so each CTA starts at its own offset into the item list.
    const int rot = (int)((blockIdx.x * 53u) % (unsigned)(2 * qd));
    auto item_of = [&](int i) { const int r = i + rot; return r >= 2 * qd ? r - 2 * qd : r; };
    for (int it0 = threadIdx.x; it0 < 2 * qd; it0 += 3 * THREADS) {
      for (int sc = 0; sc < half; sc += 12) {
        float v[3][12];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          const int iu = it0 + k * THREADS;
          const int it = iu < 2 * qd ? item_of(iu) : iu;
          const int hf = it >= qd ? 1 : 0, c = it - hf * qd;
          const int h = c / hd, cc = c - h * hd;
          const int s0 = hf * half + sc, s1 = min(S, hf * half + half);
          const float* base = a.att_scratch + (size_t)h * S * st + 2 + cc;
#pragma unroll
          for (int j = 0; j < 12; ++j) v[k][j] = (it < 2 * qd && s0 + j < s1) ? __ldcg(base + (size_t)(s0 + j) * st) : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          const int iu = it0 + k * THREADS;
          if (iu >= 2 * qd) continue;
          const int it = item_of(iu);
          const int hf = it >= qd ? 1 : 0, c = it - hf * qd;
          const int h = c / hd;
          const int s0 = hf * half + sc, s1 = min(S, hf * half + half);
          float oo = sc == 0 ? 0.f : part[it];
#pragma unroll
          for (int j = 0; j < 12; ++j)
            if (s0 + j < s1) oo += v[k][j] * ftab[h * S + s0 + j];
          part[it] = oo;
        }
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < qd; c += THREADS) {
      const float ll = sm.linv[c / hd];
      xs[c] = Cvt<XT>::from_f(ll > 0.f ? (part[c] + part[qd + c]) / ll : 0.f);
    }
  } else {
    for (int c = threadIdx.x; c < qd; c += THREADS) {
      const int h = c / hd, cc = c - h * hd;
      const float* base = a.att_scratch + (size_t)h * S * st + 2 + cc;
      float oo = 0.f;
      for (int sc = 0; sc < S; sc += 16) {
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = sc + j < S ? __ldcg(base + (size_t)(sc + j) * st) : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (sc + j < S) oo += v[j] * ftab[h * S + sc + j];
      }
      const float ll = sm.linv[h];
      xs[c] = Cvt<XT>::from_f(ll > 0.f ? oo / ll : 0.f);
    }
  }
  __syncthreads();
}

// Router of the normalised activations in shared memory (rules of route_in_block in decode.cu), then the tables the
// expert phases index by slot: expert, weight, byte offset of the expert's down-projection block.
template <typename XT>
__device__ __forceinline__ void route_phase(const gb_mega_args& a, const gb_mega_layer& L, const XT* xs, Smem& sm, long long rb_E,
                                            const float* router_rows) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = a.d, ne = a.ne, top_k = a.top_k;
  if (ne > 0) {
    // logits: `split` warps per expert, each over a contiguous part of the row with all its 16-byte loads in flight
    // (a rolled loop of 8-byte loads per expert was most of this phase's time)
    const int split = (2 * ne <= WARPS && d % 256 == 0) ? 2 : 1;
    float* lg2 = sm.q[0];                                   // partial sums of the second halves (free in this phase)
    for (int t = warp; t < ne * split; t += WARPS) {
      const int e = t / split, hf = t - e * split;
      const int len = d / split;                            // multiple of 128 when split == 2
      const float* wr = router_rows + (size_t)e * d + hf * len;    // shared memory when staged, else the global rows
      const XT* xr = xs + hf * len;
      float s = 0.f;
      if (d % 256 == 0) {
        float4 w[4];
        uint2 xq[4];
        const int n4 = len / 128;                           // 16-byte weight loads per lane (<= 4 per trip)
        for (int c0 = 0; c0 < n4; c0 += 4) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (c0 + j < n4) {
              w[j] = *reinterpret_cast<const float4*>(wr + (size_t)(c0 + j) * 128 + lane * 4);
              xq[j] = *reinterpret_cast<const uint2*>(xr + (size_t)(c0 + j) * 128 + lane * 4);
            }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (c0 + j < n4) {
              const float2 x0 = Cvt<XT>::unpack2(xq[j].x), x1 = Cvt<XT>::unpack2(xq[j].y);
              s += x0.x * w[j].x + x0.y * w[j].y + x1.x * w[j].z + x1.y * w[j].w;
            }
        }
      } else {
        for (int i = lane * 2; i < len; i += 64) {
          const float2 xv = Cvt<XT>::unpack2(*reinterpret_cast<const uint32_t*>(xr + i));
          const float2 wv = *reinterpret_cast<const float2*>(wr + i);
          s += xv.x * wv.x + xv.y * wv.y;
        }
      }
      s = warp_sum(s);
      if (lane == 0) { if (hf == 0) sm.lg[e] = s; else lg2[e] = s; }
    }
    __syncthreads();
    // softmax and the top_k picks by one warp, lane e holding experts e and e + 32 in registers (a single thread
    // walking the table in shared memory took most of this phase); ties go to the lower index, as in the serial rule
    if (warp == 0) {
      const unsigned full = 0xffffffffu;
      const bool h0 = lane < ne, h1 = lane + 32 < ne;
      const float l0 = h0 ? sm.lg[lane] + (split == 2 ? lg2[lane] : 0.f) : -INFINITY;
      const float l1 = h1 ? sm.lg[lane + 32] + (split == 2 ? lg2[lane + 32] : 0.f) : -INFINITY;
      float mx = fmaxf(l0, l1);
#pragma unroll
      for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(full, mx, o));
      float p0 = h0 ? __expf(l0 - mx) : 0.f, p1 = h1 ? __expf(l1 - mx) : 0.f;
      const float inv = 1.f / warp_sum(p0 + p1);
      p0 *= inv;
      p1 *= inv;
      float s0 = h0 ? p0 + (L.bias ? L.bias[lane] : 0.f) : -INFINITY;
      float s1 = h1 ? p1 + (L.bias ? L.bias[lane + 32] : 0.f) : -INFINITY;
      float psum = 0.f, my_w = 0.f;
      int my_e = 0;
      for (int k = 0; k < top_k; ++k) {
        float bv = s0;
        int bi = lane;
        if (s1 > bv) { bv = s1; bi = lane + 32; }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
          const float ov = __shfl_xor_sync(full, bv, o);
          const int oi = __shfl_xor_sync(full, bi, o);
          if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        bi = min(bi, ne - 1);
        const float w0 = __shfl_sync(full, p0, bi & 31), w1 = __shfl_sync(full, p1, bi & 31);
        const float w = bi < 32 ? w0 : w1;
        if (lane == k) { my_e = bi; my_w = w; }
        psum += w;
        if (bi == lane) s0 = -INFINITY;
        if (bi == lane + 32) s1 = -INFINITY;
      }
      const float invs = psum > 1e-8f ? 1.f / psum : 0.f;
      if (lane < top_k) {
        sm.esel[lane] = my_e;
        sm.wsel[lane] = my_w * invs;
        sm.off_e[lane] = (long long)my_e * d * rb_E;
        if (blockIdx.x == 0 && a.r_idx) { a.r_idx[lane] = my_e; a.r_w[lane] = my_w * invs; }
      }
      if (a.shared && lane == top_k) { sm.esel[top_k] = ne; sm.wsel[top_k] = 1.f; sm.off_e[top_k] = (long long)ne * d * rb_E; }
    }
  } else if (threadIdx.x == 0) {
    sm.esel[0] = 0;
    sm.wsel[0] = 1.f;
    sm.off_e[0] = 0;
  }
  if (threadIdx.x == THREADS - 1) {      // byte offsets of the gate and the up block, for the projection that follows
    sm.off_gu[0] = 0;
    sm.off_gu[1] = reinterpret_cast<const uint8_t*>(L.wu) - reinterpret_cast<const uint8_t*>(L.wg);
  }
  __syncthreads();
}

// Vocabulary projection.  A warp has far more rows here than its staging slice holds, so the slice is a ring of
// `items` row slots (as many whole rows as fit, at most MAXI): row k lands in slot k % items, and the slot is refilled
// with row k + items as soon as the warp has read it.  head_issue before the last grid barrier starts the first rows.
// (Pulling the rows through registers one group ahead ran this phase at a fifth of the memory bandwidth.)
template <int FMT>
__device__ __forceinline__ int head_items(const gb_mega_args& a) {
  const long long rb = (long long)(a.d / SU) * Fmt<FMT>::bytes;
  const long long fit = a.stage_bytes / rb;
  return (int)(fit < MAXI ? fit : MAXI);
}

template <int FMT>
__device__ __forceinline__ void head_issue(const gb_mega_args& a, const Plan& pl, Stage& st, int items, int k0, int k1) {
  const uint32_t rb = (uint32_t)(a.d / SU) * Fmt<FMT>::bytes;
  k1 = min(k1, pl.n);
  if (k0 >= k1 || *st.dead) return;
  __syncwarp();                                  // every lane has finished reading the slots that are refilled
  for (int k = k0; k < k1; ++k) st.pending |= 1u << (k % items);
  if ((threadIdx.x & 31) == 0) {
    fence_proxy_async();
    for (int k = k0; k < k1; ++k) {
      const int slot = k % items;
      const long long o = (long long)blockIdx.x + (long long)(pl.first + k * pl.stride) * gridDim.x;
      mbar_arrive_expect_tx(st.bars + slot, rb);
      bulk_g2s(smem_u32(st.base + (size_t)slot * rb), reinterpret_cast<const uint8_t*>(a.head) + o * rb, rb,
               smem_u32(st.bars + slot));
    }
  }
}

template <int FMT, typename XT>
__device__ __noinline__ void head_phase(const gb_mega_args& a, const XT* xs, uint8_t* stage, Smem& sm, Stage& st,
                                           int issued) {
  constexpr int SB = Fmt<FMT>::bytes;
  const int nsu = a.d / SU;
  const long long rb = (long long)nsu * SB;
  Phase ph{reinterpret_cast<const uint8_t*>(a.head), nullptr, nullptr, nsu, nsu, false, false};
  const Plan pl = make_plan(a.V, ph.P);
  const int items = head_items<FMT>(a);
  if (items < 1) {                               // a row does not fit the slice: through registers
    auto row = [&](int o) { return (long long)o * rb; };
    uint4 cur[GROUP];
    preload<FMT>(ph, pl, row, cur);
    run_phase<FMT, XT>(ph, pl, xs, stage, sm.red, cur, row, [&](int o, float v, float) { a.logits[o] = v; });
    return;
  }
  const int lane = threadIdx.x & 31;
  head_issue<FMT>(a, pl, st, items, issued, items);
  for (int k = 0; k < pl.n; ++k) {
    const int slot = k % items;
    if (!mbar_wait(st.bars + slot, (st.parity >> slot) & 1u)) {
      if (lane == 0) { *st.dead = 1; atomicCAS(st.status, 0, ST_TIMEOUT_COPY); }
      break;
    }
    st.parity ^= 1u << slot;
    st.pending &= ~(1u << slot);
    const uint8_t* src = st.base + (size_t)slot * rb;
    float acc = 0.f;
    for (int p = 0; p < nsu; ++p) {
      const uint8_t* su = src + (size_t)p * SB;
      uint4 q = make_uint4(0u, 0u, 0u, 0u);
      if constexpr (Fmt<FMT>::k16) q = *reinterpret_cast<const uint4*>(su + 16 * lane);
      acc += su_dot<FMT, XT>(q, su, xs + p * SU);
    }
    head_issue<FMT>(a, pl, st, items, k + items, k + items + 1);
    acc = warp_sum(acc);
    if (lane == 0) a.logits[blockIdx.x + (pl.first + k * pl.stride) * (int)gridDim.x] = acc;
  }
}

// ------------------------------------------------------------------------------------------------ the kernel
template <int FMT, typename XT>
__global__ void __launch_bounds__(THREADS, 1) decode_mega_kernel(const __grid_constant__ gb_mega_args a) {
  extern __shared__ __align__(16) uint8_t dyn[];
  __shared__ Smem sm;
  const int d = a.d, hd = a.hd, qd = a.H * hd, kvd = a.KV * hd, E = a.E;
  const int slots = a.ne > 0 ? a.top_k + (a.shared ? 1 : 0) : 1;
  const int xs_vals = max(max(d, qd), slots * E);
  XT* xs = reinterpret_cast<XT*>(dyn);
  uint8_t* stage_all = dyn + (((size_t)xs_vals * 2 + 15) & ~(size_t)15);
  uint8_t* stage = stage_all + (size_t)(threadIdx.x >> 5) * GROUP * 512;
  float* ftab = reinterpret_cast<float*>(stage_all + (size_t)WARPS * GROUP * 512);
  float* amerge = ftab + ((a.H * a.max_splits + 3) & ~3);
  uint8_t* wstage = reinterpret_cast<uint8_t*>(amerge + WARPS * 8 + WARPS * 4 * hd);   // 16-byte aligned: see dyn_bytes
  const int nsu_d = d / SU, nsu_q = qd / SU, nsu_E = E / SU;
  const long long rb_d = (long long)nsu_d * Fmt<FMT>::bytes, rb_q = (long long)nsu_q * Fmt<FMT>::bytes,
                  rb_E = (long long)nsu_E * Fmt<FMT>::bytes;

  if (threadIdx.x == 0) sm.dead = 0;
  GridBar gb{a.sync, a.status, &sm.dead, a.sync[1] + gridDim.x};
  __syncthreads();

  int tok = a.cur_tok[0];
  if (tok < 0 || tok >= a.V) tok = 0;
  const float* x_in = a.emb + (size_t)tok * d;
  float* x_mid = a.xbuf;
  float* x_out = a.xbuf + d;
  XT* qkv = reinterpret_cast<XT*>(a.qkv);
  XT* act = reinterpret_cast<XT*>(a.act);

  // number of cache splits: about 64 slots per CTA (four per warp, fetched in one trip), at most what the grid and
  // the scratch hold
  const gb_seq_state s0 = a.state[0];
  const int pos_now = a.pos[0];
  const int n_slots = min(a.cap, s0.cache_len + 1);
  const int S = max(1, min(min(a.max_splits, (int)gridDim.x / a.KV), (n_slots + 63) / 64));

  // optional trace: CTA 0 records the global timer before and after every barrier and at six points inside the phases
  // (16 marks per layer + start and end)
  unsigned long long* prof = (blockIdx.x == 0 && threadIdx.x == 0) ? a.prof : nullptr;
  auto mark = [&]() { if (prof) *prof++ = globaltimer_ns(); };
  mark();

  // per-warp staging slice and barriers
  __shared__ __align__(8) uint64_t bars[WARPS * MAXI];
  // the router rows of a layer (ne x d fp32, the same for every token) are staged a phase and a half ahead too, into the
  // area that only the vocabulary projection of block formats uses
  __shared__ __align__(8) uint64_t rbar;
  const uint32_t router_bytes = a.ne > 0 ? (uint32_t)a.ne * (uint32_t)d * 4u : 0u;
  const bool router_staged = router_bytes > 0 && router_bytes <= (uint32_t)(WARPS * GROUP * 512);
  uint32_t rparity = 0;
  bool rpending = false;
  if (threadIdx.x == 0) mbar_init(&rbar, 1);
  const int warp_id = threadIdx.x >> 5;
  Stage st{wstage + (size_t)warp_id * a.stage_bytes, bars + warp_id * MAXI, 0u, 0u, &sm.dead, a.status};
  if ((threadIdx.x & 31) == 0) {
    for (int k = 0; k < MAXI; ++k) mbar_init(st.bars + k, 1);
    fence_barrier_init();
  }
  __syncthreads();

  bool ok = true;
  const int n_qkv = qd + 2 * kvd;
  auto rowA = [&](int o) { return (long long)o * rb_d; };
  auto rowC = [&](int o) { return (long long)o * rb_q; };
  auto rowE = [&](int o) { return (long long)o * rb_E; };
  const Plan plA = make_plan(n_qkv, nsu_d), plC = make_plan(d, nsu_q), plE = make_plan(d, slots * nsu_E);
  {   // rows of the first projection of the first layer: nothing to wait for
    Phase ph{reinterpret_cast<const uint8_t*>(a.layers[0].wqkv), nullptr, nullptr, nsu_d, nsu_d, false, false};
    stream_issue<FMT>(ph, plA, st, rowA);
  }
  for (int li = 0; li < a.n_layers && ok; ++li) {
    const gb_mega_layer& L = a.layers[li];
    Phase phC{reinterpret_cast<const uint8_t*>(L.wo), nullptr, nullptr, nsu_q, nsu_q, false, false};
    // ---- A: RMSNorm + fused QKV projection; then this warp's rows of wo start to arrive
    {
      block_norm<XT>(x_in, L.attn_norm, xs, d, a.eps, sm.red[0]);
      Phase ph{reinterpret_cast<const uint8_t*>(L.wqkv), nullptr, nullptr, nsu_d, nsu_d, false, false};
      stream_run<FMT, XT>(ph, plA, xs, st, sm.red, [&](int o, float v, float) { qkv[o] = Cvt<XT>::from_f(v); });
      stream_issue<FMT>(phC, plC, st, rowC);
      if ((int)blockIdx.x < a.KV * S) {
        // this CTA's slice of the cache is known before the queries are: ask L2 for its rows now (a cache row was last
        // touched a token ago, 1.2 GB of weights back, so it would otherwise come from DRAM inside the walk)
        const int kvh = blockIdx.x % a.KV, split = blockIdx.x / a.KV;
        const int per = (n_slots + S - 1) / S;
        const int lo = split * per, hi = min(n_slots, lo + per);
        const int lane = threadIdx.x & 31;
        const size_t row_elems = (size_t)a.KV * hd;
        if (lane * 64 < hd)                                    // one 128-byte line per 64 values
          for (int j = lo + warp_id; j < hi; j += WARPS) {
            const XT* kp = reinterpret_cast<const XT*>(L.cache_k) + (size_t)j * row_elems + (size_t)kvh * hd + lane * 64;
            const XT* vp = reinterpret_cast<const XT*>(L.cache_v) + (size_t)j * row_elems + (size_t)kvh * hd + lane * 64;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(kp));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(vp));
          }
      }
      if (router_staged) {
        if (threadIdx.x == THREADS - 32) {       // every thread's reads of the previous layer's rows lie barriers back
          fence_proxy_async();
          mbar_arrive_expect_tx(&rbar, router_bytes);
          bulk_g2s(smem_u32(stage_all), L.router, router_bytes, smem_u32(&rbar));
        }
        rpending = true;
      }
    }
    mark();
    if (!(ok = grid_sync(gb))) break;
    mark();
    // ---- B: attention over the cache
    {   // a copy for the call: the cursor itself must not have its address taken, or it lives in local memory
      unsigned long long* pp = prof;
      attention_phase<XT>(a, L, S, sm, amerge, s0, pos_now, pp);
      prof = pp;
    }
    mark();
    if (!(ok = grid_sync(gb))) break;
    mark();
    // ---- C: merge of the splits + output projection + residual (the residual value is fetched ahead of the merge by
    // the thread that will write the output)
    const bool ownC = plC.KS > 1 && (int)threadIdx.x < plC.rows;
    const float resC = ownC ? __ldcg(x_in + blockIdx.x + threadIdx.x * gridDim.x) : 0.f;
    merge_phase<XT>(a, S, sm, ftab, xs, amerge, prof);
    mark();                                                     // merged attention output in shared memory
    stream_run<FMT, XT>(phC, plC, xs, st, sm.red,
                        [&](int o, float v, float) { x_mid[o] = (ownC ? resC : __ldcg(x_in + o)) + v; });
    mark();
    if (!(ok = grid_sync(gb))) break;
    mark();
    // ---- D: RMSNorm + router + gate/up of the chosen experts + SwiGLU; then the down-projection rows start to arrive
    Phase phE{reinterpret_cast<const uint8_t*>(L.wd), sm.off_e, sm.wsel, nsu_E, slots * nsu_E, false, false};
    {
      block_norm<XT>(x_mid, L.ffn_norm, xs, d, a.eps, sm.red[0]);
      mark();
      const float* router_rows = L.router;
      if (rpending) {
        if (!mbar_wait(&rbar, rparity)) {
          if (threadIdx.x == 0) { sm.dead = 1; atomicCAS(a.status, 0, ST_TIMEOUT_COPY); }
        } else {
          router_rows = reinterpret_cast<const float*>(stage_all);
        }
        rparity ^= 1u;
        rpending = false;
      }
      route_phase<XT>(a, L, xs, sm, rb_E, router_rows);
      mark();
      Phase ph{reinterpret_cast<const uint8_t*>(L.wg), sm.off_gu, nullptr, nsu_d, 2 * nsu_d, true, true};
      const Plan pl = make_plan(slots * E, ph.P);
      auto row = [&](int o) {
        const int slot = o / E, j = o - slot * E;
        return ((long long)sm.esel[slot] * E + j) * rb_d;
      };
      stream_issue<FMT>(ph, pl, st, row);
      stream_run<FMT, XT>(ph, pl, xs, st, sm.red,
                          [&](int o, float g, float u) { act[o] = Cvt<XT>::from_f(g / (1.f + __expf(-g)) * u); });
      stream_issue<FMT>(phE, plE, st, rowE);
    }
    mark();
    if (!(ok = grid_sync(gb))) break;
    mark();
    // ---- E: down projection of the chosen experts, weighted, + residual; then the next layer's QKV rows
    const bool ownE = plE.KS > 1 && (int)threadIdx.x < plE.rows;
    const float resE = ownE ? __ldcg(x_mid + blockIdx.x + threadIdx.x * gridDim.x) : 0.f;
    for (int i = threadIdx.x; i < slots * E / 8; i += THREADS)
      reinterpret_cast<uint4*>(xs)[i] = __ldcg(reinterpret_cast<const uint4*>(act) + i);
    __syncthreads();
    stream_run<FMT, XT>(phE, plE, xs, st, sm.red,
                        [&](int o, float v, float) { x_out[o] = (ownE ? resE : __ldcg(x_mid + o)) + v; });
    const bool last = li + 1 == a.n_layers;
    int head_pre = 0;
    if (!last) {
      Phase ph{reinterpret_cast<const uint8_t*>(a.layers[li + 1].wqkv), nullptr, nullptr, nsu_d, nsu_d, false, false};
      stream_issue<FMT>(ph, plA, st, rowA);
    } else {                              // the first rows of the vocabulary projection
      const Plan plH = make_plan(a.V, nsu_d);
      if (a.head_fmt == FMT) { head_pre = head_items<FMT>(a); head_issue<FMT>(a, plH, st, head_pre, 0, head_pre); }
      else if (a.head_fmt == GB_W_F16) { head_pre = head_items<GB_W_F16>(a); head_issue<GB_W_F16>(a, plH, st, head_pre, 0, head_pre); }
      else { head_pre = head_items<GB_W_BF16>(a); head_issue<GB_W_BF16>(a, plH, st, head_pre, 0, head_pre); }
      head_pre = max(0, min(head_pre, plH.n));
    }
    mark();
    if (!(ok = grid_sync(gb))) break;
    mark();
    x_in = x_out;
    if (last) {
      // ---- final norm + vocabulary projection
      block_norm<XT>(x_in, a.final_norm, xs, d, a.eps, sm.red[0]);
      Stage sh = st;                      // a copy for the call, as above
      if (a.head_fmt == FMT) head_phase<FMT, XT>(a, xs, stage, sm, sh, head_pre);
      else if (a.head_fmt == GB_W_F16) head_phase<GB_W_F16, XT>(a, xs, stage, sm, sh, head_pre);
      else head_phase<GB_W_BF16, XT>(a, xs, stage, sm, sh, head_pre);
      st = sh;
    }
  }
  // a step that was given up: the copies this warp still has in flight must land (or run out of time) before the
  // shared memory they target goes away
  for (int k = 0; k < MAXI; ++k)
    if (st.pending >> k & 1u) (void)mbar_wait(st.bars + k, (st.parity >> k) & 1u);
  if (rpending) (void)mbar_wait(&rbar, rparity);
  mark();
  // ---- bookkeeping: the last CTA out records where the arrival count stands; CTA 0 advances the sequence state
  __syncthreads();
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0 && ok) {
      gb_seq_state s = a.state[0];
      if (s.cache_len < a.cap) s.cache_len += 1;
      else s.ring_start = (s.ring_start + 1) % max(1, a.cap - a.pinned);
      s.abs_pos += 1;
      a.state[0] = s;
      a.pos[0] = s.abs_pos;
    }
    __threadfence();
    const unsigned t = atomicAdd(&a.sync[2], 1u);
    if (t == gridDim.x - 1) {
      a.sync[1] = atomicAdd(&a.sync[0], 0u);
      a.sync[2] = 0u;
      __threadfence();
    }
  }
}

static size_t dyn_bytes(const gb_mega_args& a, long long stage_per_warp) {
  const int slots = a.ne > 0 ? a.top_k + (a.shared ? 1 : 0) : 1;
  const int xs_vals = std::max(std::max(a.d, a.H * a.hd), slots * a.E);
  size_t b = ((size_t)xs_vals * 2 + 15) & ~(size_t)15;
  b += (size_t)WARPS * GROUP * 512;
  b += (size_t)((a.H * a.max_splits + 3) & ~3) * 4;
  b += (size_t)(WARPS * 8 + WARPS * 4 * a.hd) * 4;
  b += (size_t)WARPS * (size_t)stage_per_warp;
  return b;
}

static int su_bytes_of(int fmt) {
  switch (fmt) {
    case GB_W_F16: case GB_W_BF16: return 512;
    case GB_W_GGML_Q8_0: case GB_W_Q8_64: return 272;
    case GB_W_Q4_0: return 144;
    default: return 160;
  }
}

// Bytes of one warp's staging slice (the largest of the four layer phases and of the vocabulary ring), or -1 when a
// warp would have to stage more than MAXI outputs at once.
static long long stage_bytes_per_warp(const gb_mega_args& a, int grid, int su_bytes) {
  const int slots = a.ne > 0 ? a.top_k + (a.shared ? 1 : 0) : 1;
  const int nsu_d = a.d / SU, nsu_q = a.H * a.hd / SU, nsu_E = a.E / SU;
  const long long n[4] = {(long long)(a.H + 2 * a.KV) * a.hd, a.d, (long long)slots * a.E, a.d};
  const int P[4] = {nsu_d, nsu_q, 2 * nsu_d, slots * nsu_E};
  long long need = 16;
  for (int i = 0; i < 4; ++i) {
    int items = 0;
    need = std::max(need, stage_need(n[i], P[i], grid, su_bytes, &items));
    if (items > MAXI) return -1;
  }
  need = (need + 15) & ~15ll;
  // room for a ring of up to MAXI rows of the vocabulary projection, as far as the shared memory allows
  const long long head_row = (long long)nsu_d * su_bytes_of(a.head_fmt);
  const long long head_rows = ((long long)a.V + (long long)grid * WARPS - 1) / ((long long)grid * WARPS);
  for (long long r = std::min<long long>(MAXI, head_rows); r >= 1; --r)
    if (dyn_bytes(a, std::max(need, r * head_row)) <= (size_t)MAX_DYN) { need = std::max(need, r * head_row); break; }
  return need;
}

}  // namespace mg
}  // namespace gb

using namespace gb;

extern "C" int gb_decode_mega_ok(const gb_mega_args* a) {
  if (!a || a->n_layers <= 0) return -1;
  if (a->d % mg::SU || (a->H * a->hd) % mg::SU || a->E % mg::SU) return -2;          // whole super-units per stored row
  if (a->hd != 32 && a->hd != 64 && a->hd != 128) return -3;
  if (a->KV <= 0 || a->H % a->KV || a->H > mg::MAX_HEADS) return -3;
  if (a->ne > 64 || a->ne < 0 || (a->ne > 0 && (a->top_k < 1 || a->top_k > 8 || a->top_k > a->ne))) return -4;
  if (a->fmt < GB_W_F16 || a->fmt > GB_W_Q4_1) return -5;
  if (a->head_fmt != a->fmt && a->head_fmt != GB_W_F16 && a->head_fmt != GB_W_BF16) return -5;
  if (a->d > 8 * mg::THREADS || a->max_splits > 64) return -6;
  if (a->max_splits < 1 || a->cap < 1 || a->pinned < 0 || a->pinned >= a->cap) return -6;
  const int grid = gb_decode_mega_grid();
  if (grid <= 0 || grid < a->KV) return -9;
  const long long per_warp = mg::stage_bytes_per_warp(*a, grid, mg::su_bytes_of(a->fmt));
  if (per_warp < 0 || mg::dyn_bytes(*a, per_warp) > mg::MAX_DYN) return -7;
  return 0;
}

// Number of CTAs of the launch: one per SM (a cooperative launch needs all of them resident at once).
extern "C" int gb_decode_mega_grid() {
  static const int n = []() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
  }();
  return n;
}

template <int FMT, typename XT>
static int launch_mega(const gb_mega_args& a_in, cudaStream_t st) {
  auto kern = mg::decode_mega_kernel<FMT, XT>;
  const int grid = gb_decode_mega_grid();
  if (grid <= 0 || grid < a_in.KV) return -9;
  gb_mega_args a = a_in;
  a.stage_bytes = (int)mg::stage_bytes_per_warp(a, grid, mg::Fmt<FMT>::bytes);
  const size_t smem = mg::dyn_bytes(a, a.stage_bytes);
  static bool attr_done = false;                 // one process drives one device
  if (!attr_done) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, mg::MAX_DYN) != cudaSuccess) return -8;
    attr_done = true;
  }
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeCooperative;
  attr.val.cooperative = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(mg::THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return -(1000 + (int)e); }
  return 0;
}

extern "C" int gb_decode_mega(const gb_mega_args* a, cudaStream_t st) {
  const int rc = gb_decode_mega_ok(a);
  if (rc) return rc;
#define GB_MEGA_CASE(F)                                                    \
  case F:                                                                  \
    return a->is_bf16 ? launch_mega<F, __nv_bfloat16>(*a, st) : launch_mega<F, __half>(*a, st);
  switch (a->fmt) {
    GB_MEGA_CASE(GB_W_F16)
    GB_MEGA_CASE(GB_W_BF16)
    GB_MEGA_CASE(GB_W_GGML_Q8_0)
    GB_MEGA_CASE(GB_W_Q4_0)
    GB_MEGA_CASE(GB_W_Q8_64)
    GB_MEGA_CASE(GB_W_Q4_1)
  }
#undef GB_MEGA_CASE
  return -5;
}
