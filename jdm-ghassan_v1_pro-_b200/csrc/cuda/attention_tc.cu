// Causal flash attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), head_dim 64 or 128.
//
// Forward, one CTA per (batch, head, 128 query rows):
//   warp 4 : TMA producer  - Q tile once, then K/V tiles of 128 keys through a 2-stage ring
//   warp 5 : MMA issuer    - S = Q K^T into tensor memory, then O_part = P V (P read from shared memory)
//   warps 0-3 (one thread per query row): tcgen05.ld of S, scale + causal/window/segment mask, online softmax,
//            P (16-bit) written to shared memory in the 128-byte-swizzled operand layout, O rescaled and
//            accumulated in registers, final normalisation, O and log-sum-exp stored.
// The backward pass (further down) uses the same tile machinery: a dQ kernel per query tile and a dK/dV kernel
// per key tile that loops over the query heads of its group, both recomputing P from the saved log-sum-exp.
// Scores are never written to global memory (the reference materialises B*H*T^2 floats and re-runs the forward
// in its backward, cuda/attention.cu:297-550, 805-898).
//
// Segment masks are passed as `lo[i]` = first key position visible to query i (start of its packed document,
// or 0): visible(i, j) <=> max(lo[i], i - window + 1) <= j <= i.  Every wait is bounded (status word on expiry).
#include <algorithm>
#include <type_traits>

#include "sm100_common.cuh"
#include "gb_api.h"

namespace gb {

template <typename T> struct OperandFmt { static constexpr int value = std::is_same<T, __nv_bfloat16>::value ? 1 : 0; };

constexpr int AT_M = 128;        // query rows per tile
constexpr int AT_N = 128;        // keys per tile
constexpr int AT_THREADS = 192;
// Backward kernels: sixteen compute warps.  Warp w owns the 32 tile rows of TMEM lane quarter w % 4 and the 32-column
// chunk w / 4, so a 128 x 128 score tile is one tcgen05.ld per thread and every scheduler has four warps to switch
// between (with four compute warps in all, the exp / multiply / pack chain of a tile ran at one warp per scheduler
// and its latencies were exposed: the tensor pipe sat idle 94 % of the time).  Warp 16 = TMA producer, 17 = MMA issuer.
constexpr int AT_BWD_CW = 16;
constexpr int AT_BWD_THREADS = (AT_BWD_CW + 2) * 32;
constexpr int AT_BWD_W_TMA = AT_BWD_CW, AT_BWD_W_MMA = AT_BWD_CW + 1;

struct AttnTcParams {
  int B, T, H, KV, window;
  float scale;
  const int* lo;          // [B*T] or null
  void* o; long long ld_o;
  float* lse;             // [B*T, H]
  // backward
  const float* delta;     // [B*T, H]
  void* dq; long long ld_dq;
  void* dk; long long ld_dk;
  void* dv; long long ld_dv;
  int* status;
};

__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity, int* status, int code, volatile int* abort_flag) {
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 1024; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > 4000000000LL) {
      atomicCAS(status, 0, code);
      *abort_flag = 1;
      return false;
    }
  }
}

// [rows x 64] 16-bit tile with 128-byte rows, 128B swizzle: byte offset of element (r, c), c < 64
__device__ __forceinline__ uint32_t sw128_off(int r, int c) {
  return (uint32_t)(r * 128 + ((((c >> 3) ^ (r & 7)) << 4) | ((c & 7) << 1)));
}

// write 32 consecutive columns [c0, c0+32) of row r into a [128 x 128] operand buffer made of two 64-column panels
template <typename T>
__device__ __forceinline__ void store_p_chunk(uint8_t* sP, int r, int c0, const float (&v)[32]) {
  uint8_t* panel = sP + (c0 >> 6) * (AT_M * 128);
  const int cc = c0 & 63;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 q;
    q.x = Cvt<T>::pack2(v[8 * j + 0], v[8 * j + 1]);
    q.y = Cvt<T>::pack2(v[8 * j + 2], v[8 * j + 3]);
    q.z = Cvt<T>::pack2(v[8 * j + 4], v[8 * j + 5]);
    q.w = Cvt<T>::pack2(v[8 * j + 6], v[8 * j + 7]);
    *reinterpret_cast<uint4*>(panel + sw128_off(r, cc + 8 * j)) = q;
  }
}

// TMA load of a [128 rows x HD] tile as HD/64 panels
template <int HD>
__device__ __forceinline__ void load_tile(const CUtensorMap* tm, uint64_t* bar, uint8_t* dst, int col0, int row0) {
#pragma unroll
  for (int p = 0; p < HD / 64; ++p) tma_load_2d(tm, bar, dst + p * (AT_M * 128), col0 + 64 * p, row0);
}

// D[128 x N] (+)= A[128 x K] * B, all operands in the panelled SW128 layout.
//   a_kmajor tile: K runs along the 64-column panels.   b_mn: B given as [K rows x N cols] (N contiguous).
template <int KDIM>
__device__ __forceinline__ void mma_kmajor_kmajor(uint32_t tmem_d, uint32_t sa, uint32_t sb, uint32_t idesc, bool accumulate) {
  // A: [128 x KDIM] K-major, B: [N x KDIM] K-major
#pragma unroll
  for (int kk = 0; kk < KDIM / 16; ++kk) {
    const uint32_t off = (kk >> 2) * (AT_M * 128) + (kk & 3) * 32;
    umma_f16(tmem_d, make_smem_desc_sw128(sa + off, 16, 1024), make_smem_desc_sw128(sb + off, 16, 1024), idesc,
             (accumulate || kk > 0) ? 1u : 0u);
  }
}
template <int KDIM>
__device__ __forceinline__ void mma_kmajor_mnmajor(uint32_t tmem_d, uint32_t sa, uint32_t sb, uint32_t idesc, bool accumulate) {
  // A: [128 x KDIM] K-major (panels of 64 along K), B: [KDIM rows x N] with N contiguous (panels of 64 along N)
#pragma unroll
  for (int kk = 0; kk < KDIM / 16; ++kk) {
    const uint32_t aoff = (kk >> 2) * (AT_M * 128) + (kk & 3) * 32;
    const uint32_t boff = kk * 2048;   // 16 rows of 128 bytes
    umma_f16(tmem_d, make_smem_desc_sw128(sa + aoff, 16, 1024), make_smem_desc_sw128(sb + boff, AT_N * 128, 1024), idesc,
             (accumulate || kk > 0) ? 1u : 0u);
  }
}

// ============================================================================================ forward
template <typename T, int HD>
__global__ void __launch_bounds__(AT_THREADS) attn_tc_fwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                 const __grid_constant__ CUtensorMap tmK,
                                                                 const __grid_constant__ CUtensorMap tmV,
                                                                 const AttnTcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t TILE = AT_M * HD * 2;
  uint8_t* smem;
  if constexpr (HD == 64) {
    // 112 KB of tiles + barriers and not a byte more: two CTAs of this kernel share an SM (143 registers, 256 TMEM
    // columns each), which hides the latency of the short causal loops at T = 512.  That leaves no slack to align
    // the base by hand; the kernel has no static shared memory, so the dynamic window starts 1024-aligned.  Checked,
    // not assumed: a misaligned base reports and returns before any barrier or TMEM is touched.
    if (smem_u32(smem_raw) & 1023u) {
      if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_BAD_ARGUMENT);
      return;
    }
    smem = smem_raw;
  } else {
    smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE;            // 2 stages
  uint8_t* sV = sK + 2 * TILE;        // 2 stages
  uint8_t* sP = sV + 2 * TILE;        // [128 x 128] 16-bit
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + AT_M * AT_N * 2);
  uint64_t* q_full = bars;            // 1
  uint64_t* kv_full = bars + 1;       // 2
  uint64_t* kv_empty = bars + 3;      // 2
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;
  uint64_t* o_full = bars + 7;
  uint64_t* q_empty = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Work items: (query tile, batch, head), the query tile slowest and from the last one down: under a causal mask that
  // tile visits the most key tiles, so the long items are dealt first and the short ones fill the tail.  A CTA stays
  // on its SM and walks items blockIdx.x, blockIdx.x + gridDim.x, ...: tensor memory, barriers and tensor maps are set
  // up once, the producer warp runs ahead into the next item's Q, K and V while the soft-max warps finish the current
  // one, and the first score tile of the next item is computed under the current item's output store.
  const int n_qt = (p.T + AT_M - 1) / AT_M, BH = p.B * p.H;
  const int n_items = n_qt * BH;
  const int rep = p.H / p.KV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 4);             // one arrival per soft-max warp
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + AT_N;

  // Visible key tiles of an item: [k_lo, k_lo + n_tiles * AT_N).  `lo` (start of the packed document) and the window
  // bound are both non-decreasing along a sequence, so the first row of the tile has the smallest of them.
  auto item_range = [&](int item, int& b, int& h, int& q0, int& k_lo, int& n_tiles) {
    const int zt = item / BH, bh = item - zt * BH;
    b = bh / p.H;
    h = bh - b * p.H;
    q0 = (n_qt - 1 - zt) * AT_M;
    int lo0 = p.lo ? p.lo[(long long)b * p.T + q0] : 0;
    if (p.window > 0) lo0 = max(lo0, q0 - p.window + 1);
    const int k_hi = min(p.T, q0 + AT_M);
    k_lo = (min(lo0, k_hi - 1) / AT_N) * AT_N;
    n_tiles = (k_hi - k_lo + AT_N - 1) / AT_N;
  };

  if (warp == 4) {
    if (lane == 0) {
      uint32_t kv_it = 0, q_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++q_it) {
        int b, h, q0, k_lo, n_tiles;
        item_range(item, b, h, q0, k_lo, n_tiles);
        const int kvh = h / rep;
        const int row_base = b * p.T;
        // the tensor core has read the previous item's Q (committed after its last score tile)
        if (!at_wait(q_empty, (q_it & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) break;
        mbar_arrive_expect_tx(q_full, TILE);
        load_tile<HD>(&tmQ, q_full, sQ, h * HD, row_base + q0);
        for (int t = 0; t < n_tiles; ++t, ++kv_it) {
          const int s = kv_it & 1, ph = (kv_it >> 1) & 1;
          if (!at_wait(&kv_empty[s], ph ^ 1, p.status, ST_TIMEOUT_EMPTY, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&kv_full[s], 2 * TILE);
          load_tile<HD>(&tmK, &kv_full[s], sK + s * TILE, kvh * HD, row_base + k_lo + t * AT_N);
          load_tile<HD>(&tmV, &kv_full[s], sV + s * TILE, kvh * HD, row_base + k_lo + t * AT_N);
        }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr int fmt = OperandFmt<T>::value;
      const uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, AT_M, AT_N);
      const uint32_t idesc_o = make_idesc_f16(fmt, 0, 1, AT_M, HD);
      uint32_t kv_it = 0, q_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++q_it) {
        int b, h, q0, k_lo, n_tiles;
        item_range(item, b, h, q0, k_lo, n_tiles);
        if (!at_wait(q_full, q_it & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) break;
        for (int t = 0; t < n_tiles; ++t, ++kv_it) {
          const int s = kv_it & 1, ph = (kv_it >> 1) & 1;
          if (!at_wait(&kv_full[s], ph, p.status, ST_TIMEOUT_FULL, abort_flag)) { ok = false; break; }
          tc_fence_after();
          // S(t) may overwrite S(t-1) only after the softmax threads have read it: p_ready(t-1) was waited below
          mma_kmajor_kmajor<HD>(tmem_S, smem_u32(sQ), smem_u32(sK + s * TILE), idesc_s, false);
          umma_commit(s_full);
          if (t == n_tiles - 1) umma_commit(q_empty);
          if (!at_wait(p_ready, kv_it & 1u, p.status, ST_TIMEOUT_TMEM_EMPTY, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_kmajor_mnmajor<AT_N>(tmem_O, smem_u32(sP), smem_u32(sV + s * TILE), idesc_o, t > 0);
          umma_commit(o_full);
          umma_commit(&kv_empty[s]);
        }
      }
    }
    __syncwarp();
  } else {
    // Soft-max warps, one thread per query row.  The output accumulates in tensor memory over the key tiles of an item
    // (the P V product adds to it), so a thread touches it only at the end of the item, and in the rare tile where the
    // running maximum of a row of its warp has grown by more than 2^8: only then are the accumulator rows rescaled
    // (until then the probabilities are taken against the older, smaller maximum, at most 256 times larger than with the
    // true one; the final division by the row sum, kept against the same maximum, is exact either way).
    const int r = threadIdx.x;                  // query row of the tile
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float sc2 = p.scale * 1.4426950408889634f;       // scores in log2 units: exp(x * scale) = 2^(x * sc2)
    uint32_t tile_it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      int b, h, q0, k_lo, n_tiles;
      item_range(item, b, h, q0, k_lo, n_tiles);
      const long long row_base = (long long)b * p.T;
      const int i = q0 + r;
      const bool row_ok = i < p.T;
      int lo_i = 0;
      if (row_ok) {
        if (p.lo) lo_i = p.lo[row_base + i];
        if (p.window > 0) lo_i = max(lo_i, i - p.window + 1);
      }
      float m2 = -INFINITY, l = 0.f;            // maximum in use (log2 units) and the row sum against it
      for (int t = 0; t < n_tiles; ++t, ++tile_it) {
        const int j0 = k_lo + t * AT_N;
        if (!at_wait(s_full, tile_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const bool need_mask = (j0 + AT_N - 1 > q0) || (j0 < lo_i);
        // pass A: row maximum of the raw scores (the scale is positive: checked by the launcher)
        float mr[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
        for (int c = 0; c < AT_N / 32; ++c) {
          uint32_t rg[32];
          tmem_ld_32x32(tmem_S + lane_base + c * 32, rg);
          tmem_ld_wait();
          if (!need_mask) {
#pragma unroll
            for (int k = 0; k < 32; ++k) mr[k & 3] = fmaxf(mr[k & 3], __uint_as_float(rg[k]));
          } else {
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const int j = j0 + c * 32 + k;
              if (j <= i && j >= lo_i) mr[k & 3] = fmaxf(mr[k & 3], __uint_as_float(rg[k]));
            }
          }
        }
        float mt = fmaxf(fmaxf(mr[0], mr[1]), fmaxf(mr[2], mr[3])) * sc2;
        if (!row_ok) mt = 0.f;
        // a new maximum is taken when some row of the warp needs it (the accumulator rows are reached by warp-wide
        // tensor-memory loads and stores, so the decision is the warp's)
        const bool grow = mt > m2 + 8.f || (m2 == -INFINITY && mt != -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = fmaxf(m2, mt);
          if (t > 0) {
            const float corr = (m2 == -INFINITY) ? 1.f : exp2f(m2 - m_new);   // nothing accumulated yet on a -inf row
            l *= corr;
            // the previous tile's P V has to be in the accumulator before it is rescaled
            if (!at_wait(o_full, (tile_it - 1u) & 1u, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < HD / 16; ++c) {
              uint32_t rg[16];
              tmem_ld_32x16(tmem_O + lane_base + c * 16, rg);
              tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 16; ++k) rg[k] = __float_as_uint(__uint_as_float(rg[k]) * corr);
              tmem_st_32x16(tmem_O + lane_base + c * 16, rg);
            }
            tmem_st_wait();
          }
          m2 = m_new;
        }
        float ls[2] = {0.f, 0.f};
        const bool dead = m2 == -INFINITY;       // no visible key so far in this row
        // pass B: probabilities -> shared memory (operand layout)
#pragma unroll 1
        for (int c = 0; c < AT_N / 32; ++c) {
          uint32_t rg[32];
          tmem_ld_32x32(tmem_S + lane_base + c * 32, rg);
          tmem_ld_wait();
          float pv[32];
          if (!need_mask) {
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const float e = exp2f(fmaf(__uint_as_float(rg[k]), sc2, -m2));
              pv[k] = e;
              ls[k & 1] += e;
            }
          } else {
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const int j = j0 + c * 32 + k;
              const bool vis = row_ok && !dead && j <= i && j >= lo_i;
              const float e = vis ? exp2f(fmaf(__uint_as_float(rg[k]), sc2, -m2)) : 0.f;
              pv[k] = e;
              ls[k & 1] += e;
            }
          }
          store_p_chunk<T>(sP, r, c * 32, pv);
        }
        l += ls[0] + ls[1];
        tc_fence_before();
        fence_proxy_async();          // generic-proxy writes of P must be visible to the tensor core
        __syncwarp();                 // every lane's writes and fences, then one arrival for the warp
        if (lane == 0) mbar_arrive(p_ready);
      }
      if (!ok) break;
      // the item's last P V
      if (!at_wait(o_full, (tile_it - 1u) & 1u, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      T* op = reinterpret_cast<T*>(p.o) + (row_base + i) * p.ld_o + (long long)h * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t rg[32];
        tmem_ld_32x32(tmem_O + lane_base + c * 32, rg);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 q;
            q.x = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 0]) * inv_l, __uint_as_float(rg[8 * k + 1]) * inv_l);
            q.y = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 2]) * inv_l, __uint_as_float(rg[8 * k + 3]) * inv_l);
            q.z = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 4]) * inv_l, __uint_as_float(rg[8 * k + 5]) * inv_l);
            q.w = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 6]) * inv_l, __uint_as_float(rg[8 * k + 7]) * inv_l);
            reinterpret_cast<uint4*>(op)[c * 4 + k] = q;
          }
        }
      }
      tc_fence_before();              // the next item's first P V overwrites the accumulator
      if (row_ok && p.lse) p.lse[(row_base + i) * p.H + h] = l > 0.f ? (m2 + log2f(l)) * 0.6931471805599453f : INFINITY;
    }
  }
  __syncthreads();
  if (*abort_flag) {
    for (int k = 0; k < 64; ++k) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// ============================================================================================ backward: dQ
// One CTA per (batch, head, 128 query rows).  Per key tile: S = Q K^T and dP = dO V^T into tensor memory,
// dS = P o (dP - delta) * scale written to shared memory (16-bit operand layout), dQ += dS K accumulated in
// tensor memory over the whole key loop and read out once.
template <typename T, int HD, int STAGES>
__global__ void __launch_bounds__(AT_BWD_THREADS) attn_tc_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                    const __grid_constant__ CUtensorMap tmK,
                                                                    const __grid_constant__ CUtensorMap tmV,
                                                                    const __grid_constant__ CUtensorMap tmDO,
                                                                    const AttnTcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t TILE = AT_M * HD * 2;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + TILE;
  uint8_t* sK = sDO + TILE;                 // STAGES
  uint8_t* sV = sK + STAGES * TILE;         // STAGES
  uint8_t* sDS = sV + STAGES * TILE;        // [128 x 128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + AT_M * AT_N * 2);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;             // STAGES (<= 2)
  uint64_t* kv_empty = bars + 3;
  uint64_t* sdp_full = bars + 5;
  uint64_t* ds_ready = bars + 6;
  uint64_t* dq_full = bars + 7;
  uint64_t* q_empty = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Persistent, like the forward kernel: items are (query tile, batch, head) with the last query tile (the longest key
  // loop) first; a CTA walks items blockIdx.x, blockIdx.x + gridDim.x, ... with tensor memory and barriers set up once,
  // the producer running ahead into the next item and the next item's first S / dP under the current dQ read-out.
  const int n_qt = (p.T + AT_M - 1) / AT_M, BH = p.B * p.H;
  const int n_items = n_qt * BH;
  const int rep = p.H / p.KV;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(sdp_full, 1);
    mbar_init(ds_ready, AT_BWD_CW);      // one arrival per compute warp
    mbar_init(dq_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == AT_BWD_W_MMA) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + AT_N, tmem_dQ = tmem_base + 2 * AT_N;

  // visible key tiles of an item (`lo` and the window bound are non-decreasing along a sequence: the first row of the
  // tile has the smallest)
  auto item_range = [&](int item, int& b, int& h, int& q0, int& k_lo, int& n_tiles) {
    const int zt = item / BH, bh = item - zt * BH;
    b = bh / p.H;
    h = bh - b * p.H;
    q0 = (n_qt - 1 - zt) * AT_M;
    int lo0 = p.lo ? p.lo[(long long)b * p.T + q0] : 0;
    if (p.window > 0) lo0 = max(lo0, q0 - p.window + 1);
    const int k_hi = min(p.T, q0 + AT_M);
    k_lo = (min(lo0, k_hi - 1) / AT_N) * AT_N;
    n_tiles = (k_hi - k_lo + AT_N - 1) / AT_N;
  };

  if (warp == AT_BWD_W_TMA) {
    if (lane == 0) {
      uint32_t kv_it = 0, q_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++q_it) {
        int b, h, q0, k_lo, n_tiles;
        item_range(item, b, h, q0, k_lo, n_tiles);
        const int kvh = h / rep;
        const int row_base = b * p.T;
        // Q and dO of the previous item have been read (committed after its last S / dP)
        if (!at_wait(q_empty, (q_it & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) break;
        mbar_arrive_expect_tx(q_full, 2 * TILE);
        load_tile<HD>(&tmQ, q_full, sQ, h * HD, row_base + q0);
        load_tile<HD>(&tmDO, q_full, sDO, h * HD, row_base + q0);
        for (int t = 0; t < n_tiles; ++t, ++kv_it) {
          const int s = kv_it % STAGES, ph = (kv_it / STAGES) & 1;
          if (!at_wait(&kv_empty[s], ph ^ 1, p.status, ST_TIMEOUT_EMPTY, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&kv_full[s], 2 * TILE);
          load_tile<HD>(&tmK, &kv_full[s], sK + s * TILE, kvh * HD, row_base + k_lo + t * AT_N);
          load_tile<HD>(&tmV, &kv_full[s], sV + s * TILE, kvh * HD, row_base + k_lo + t * AT_N);
        }
      }
    }
    __syncwarp();
  } else if (warp == AT_BWD_W_MMA) {
    if (lane == 0) {
      constexpr int fmt = OperandFmt<T>::value;
      const uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, AT_M, AT_N);
      const uint32_t idesc_dq = make_idesc_f16(fmt, 0, 1, AT_M, HD);
      uint32_t kv_it = 0, q_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++q_it) {
        int b, h, q0, k_lo, n_tiles;
        item_range(item, b, h, q0, k_lo, n_tiles);
        if (!at_wait(q_full, q_it & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) break;
        for (int t = 0; t < n_tiles; ++t, ++kv_it) {
          const int s = kv_it % STAGES, ph = (kv_it / STAGES) & 1;
          if (!at_wait(&kv_full[s], ph, p.status, ST_TIMEOUT_FULL, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_kmajor_kmajor<HD>(tmem_S, smem_u32(sQ), smem_u32(sK + s * TILE), idesc_s, false);
          mma_kmajor_kmajor<HD>(tmem_dP, smem_u32(sDO), smem_u32(sV + s * TILE), idesc_s, false);
          umma_commit(sdp_full);
          if (t == n_tiles - 1) umma_commit(q_empty);
          if (!at_wait(ds_ready, kv_it & 1u, p.status, ST_TIMEOUT_TMEM_EMPTY, abort_flag)) { ok = false; break; }
          tc_fence_after();
          // the first dQ of an item overwrites the accumulator: the compute warps have read the previous item's dQ
          // before they arrived on ds_ready for this tile
          mma_kmajor_mnmajor<AT_N>(tmem_dQ, smem_u32(sDS), smem_u32(sK + s * TILE), idesc_dq, t > 0);
          umma_commit(&kv_empty[s]);
        }
        if (ok) umma_commit(dq_full);
      }
    }
    __syncwarp();
  } else {
    const int cq = warp >> 2;                     // 32-column chunk of a compute warp
    const int r = (warp & 3) * 32 + lane;         // query row of a compute thread (its TMEM lane)
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const float sc = p.scale;
    const float sc2 = sc * 1.4426950408889634f;   // exp(x * scale - lse) = 2^(x * sc2 - lse * log2 e)
    uint32_t tile_it = 0, item_it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_it) {
      int b, h, q0, k_lo, n_tiles;
      item_range(item, b, h, q0, k_lo, n_tiles);
      const long long row_base = (long long)b * p.T;
      const int i = q0 + r;
      const bool row_ok = i < p.T;
      int lo_i = 0;
      float lse2 = INFINITY, dls = 0.f;
      if (row_ok) {
        if (p.lo) lo_i = p.lo[row_base + i];
        if (p.window > 0) lo_i = max(lo_i, i - p.window + 1);
        lse2 = p.lse[(row_base + i) * p.H + h] * 1.4426950408889634f;
        dls = p.delta[(row_base + i) * p.H + h] * sc;      // delta times the scale: dS = P (dP * scale - dls)
      }
      for (int t = 0; t < n_tiles; ++t, ++tile_it) {
        const int j0 = k_lo + t * AT_N;
        if (!at_wait(sdp_full, tile_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const bool need_mask = !row_ok || (j0 + AT_N - 1 > q0) || (j0 < lo_i);
        {
          const int c = cq;
          uint32_t rs[32], rp[32];
          tmem_ld_32x32(tmem_S + lane_base + c * 32, rs);
          tmem_ld_32x32(tmem_dP + lane_base + c * 32, rp);
          tmem_ld_wait();
          float ds[32];
          if (!need_mask) {
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const float pr = exp2f(fmaf(__uint_as_float(rs[k]), sc2, -lse2));
              ds[k] = pr * fmaf(__uint_as_float(rp[k]), sc, -dls);
            }
          } else {
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const int j = j0 + c * 32 + k;
              const bool vis = row_ok && j <= i && j >= lo_i;
              const float pr = vis ? exp2f(fmaf(__uint_as_float(rs[k]), sc2, -lse2)) : 0.f;
              ds[k] = pr * fmaf(__uint_as_float(rp[k]), sc, -dls);
            }
          }
          store_p_chunk<T>(sDS, r, c * 32, ds);
        }
        tc_fence_before();
        fence_proxy_async();
        __syncwarp();                 // every lane's writes and fences, then one arrival for the warp
        if (lane == 0) mbar_arrive(ds_ready);
      }
      if (!ok || !at_wait(dq_full, item_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) { ok = false; break; }
      tc_fence_after();
      T* dqp = reinterpret_cast<T*>(p.dq) + (row_base + i) * p.ld_dq + (long long)h * HD;
      if (cq < HD / 32) {
        const int c = cq;
        uint32_t rg[32];
        tmem_ld_32x32(tmem_dQ + lane_base + c * 32, rg);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 q;
            q.x = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 0]), __uint_as_float(rg[8 * k + 1]));
            q.y = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 2]), __uint_as_float(rg[8 * k + 3]));
            q.z = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 4]), __uint_as_float(rg[8 * k + 5]));
            q.w = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 6]), __uint_as_float(rg[8 * k + 7]));
            reinterpret_cast<uint4*>(dqp + c * 32)[k] = q;
          }
        }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (*abort_flag) {
    for (int k = 0; k < 64; ++k) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == AT_BWD_W_MMA) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ============================================================================================ backward: dQ (head_dim 64)
// The same product with key steps of 64 instead of 128.  A step is then S 64 + dP 64 + dQ 64 = 192 tensor-memory
// columns and 96 KB of shared memory, so two CTAs (8 compute warps each) share an SM: what bounds these kernels is the
// round trip tensor core -> barrier -> compute warps -> barrier -> tensor core of every step, not arithmetic, and two
// independent chains per SM hide each other's waits (the forward kernel gets its rate the same way).
constexpr int AT_DQ64_CW = 8;
constexpr int AT_DQ64_THREADS = (AT_DQ64_CW + 2) * 32;
constexpr int AT_DQ64_STAGES = 3;

template <typename T>
__global__ void __launch_bounds__(AT_DQ64_THREADS, 2) attn_tc_bwd_dq64_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                          const __grid_constant__ CUtensorMap tmK,
                                                                          const __grid_constant__ CUtensorMap tmV,
                                                                          const __grid_constant__ CUtensorMap tmDO,
                                                                          const AttnTcParams p) {
  constexpr int HD = 64, KN = 64, ST = AT_DQ64_STAGES;
  constexpr int W_TMA = AT_DQ64_CW, W_MMA = AT_DQ64_CW + 1;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t TILE = AT_M * HD * 2;          // Q, dO and dS: [128 x 64] 16-bit
  constexpr uint32_t KTILE = KN * HD * 2;           // K, V of a step: [64 x 64]
  // no static shared memory: the dynamic window starts 1024-aligned (checked, as in the forward kernel)
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_BAD_ARGUMENT);
    return;
  }
  uint8_t* sQ = smem_raw;
  uint8_t* sDO = sQ + TILE;
  uint8_t* sDS = sDO + TILE;
  uint8_t* sK = sDS + TILE;                 // ST
  uint8_t* sV = sK + ST * KTILE;            // ST
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + ST * KTILE);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;
  uint64_t* sdp_full = bars + 2;
  uint64_t* ds_ready = bars + 3;
  uint64_t* dq_full = bars + 4;
  uint64_t* kv_full = bars + 5;             // ST
  uint64_t* kv_empty = bars + 5 + ST;       // ST
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5 + 2 * ST);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.T + AT_M - 1) / AT_M, BH = p.B * p.H;
  const int n_items = n_qt * BH;
  const int rep = p.H / p.KV;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(ds_ready, AT_DQ64_CW);
    mbar_init(dq_full, 1);
    for (int s = 0; s < ST; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == W_MMA) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + KN, tmem_dQ = tmem_base + 2 * KN;

  // visible key steps of an item: [k_lo, k_lo + n_steps * 64)
  auto item_range = [&](int item, int& b, int& h, int& q0, int& k_lo, int& n_steps) {
    const int zt = item / BH, bh = item - zt * BH;
    b = bh / p.H;
    h = bh - b * p.H;
    q0 = (n_qt - 1 - zt) * AT_M;
    int lo0 = p.lo ? p.lo[(long long)b * p.T + q0] : 0;
    if (p.window > 0) lo0 = max(lo0, q0 - p.window + 1);
    const int k_hi = min(p.T, q0 + AT_M);
    k_lo = (min(lo0, k_hi - 1) / KN) * KN;
    n_steps = (k_hi - k_lo + KN - 1) / KN;
  };

  if (warp == W_TMA) {
    if (lane == 0) {
      uint32_t kv_it = 0, q_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++q_it) {
        int b, h, q0, k_lo, n_steps;
        item_range(item, b, h, q0, k_lo, n_steps);
        const int kvh = h / rep;
        const int row_base = b * p.T;
        if (!at_wait(q_empty, (q_it & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) break;
        mbar_arrive_expect_tx(q_full, 2 * TILE);
        load_tile<HD>(&tmQ, q_full, sQ, h * HD, row_base + q0);
        load_tile<HD>(&tmDO, q_full, sDO, h * HD, row_base + q0);
        for (int t = 0; t < n_steps; ++t, ++kv_it) {
          const int s = kv_it % ST, ph = (kv_it / ST) & 1;
          if (!at_wait(&kv_empty[s], ph ^ 1, p.status, ST_TIMEOUT_EMPTY, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&kv_full[s], 2 * KTILE);
          tma_load_2d(&tmK, &kv_full[s], sK + s * KTILE, kvh * HD, row_base + k_lo + t * KN);
          tma_load_2d(&tmV, &kv_full[s], sV + s * KTILE, kvh * HD, row_base + k_lo + t * KN);
        }
      }
    }
    __syncwarp();
  } else if (warp == W_MMA) {
    if (lane == 0) {
      constexpr int fmt = OperandFmt<T>::value;
      const uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, AT_M, KN);
      const uint32_t idesc_dq = make_idesc_f16(fmt, 0, 1, AT_M, HD);
      uint32_t kv_it = 0, q_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++q_it) {
        int b, h, q0, k_lo, n_steps;
        item_range(item, b, h, q0, k_lo, n_steps);
        if (!at_wait(q_full, q_it & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) break;
        for (int t = 0; t < n_steps; ++t, ++kv_it) {
          const int s = kv_it % ST, ph = (kv_it / ST) & 1;
          if (!at_wait(&kv_full[s], ph, p.status, ST_TIMEOUT_FULL, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_kmajor_kmajor<HD>(tmem_S, smem_u32(sQ), smem_u32(sK + s * KTILE), idesc_s, false);
          mma_kmajor_kmajor<HD>(tmem_dP, smem_u32(sDO), smem_u32(sV + s * KTILE), idesc_s, false);
          umma_commit(sdp_full);
          if (t == n_steps - 1) umma_commit(q_empty);
          if (!at_wait(ds_ready, kv_it & 1u, p.status, ST_TIMEOUT_TMEM_EMPTY, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_kmajor_mnmajor<KN>(tmem_dQ, smem_u32(sDS), smem_u32(sK + s * KTILE), idesc_dq, t > 0);
          umma_commit(&kv_empty[s]);
        }
        if (ok) umma_commit(dq_full);
      }
    }
    __syncwarp();
  } else {
    const int cq = warp >> 2;                     // 32-column chunk (of the 64 keys of a step, of the 64 of dQ)
    const int r = (warp & 3) * 32 + lane;         // query row of a compute thread (its TMEM lane)
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const float sc = p.scale;
    const float sc2 = sc * 1.4426950408889634f;
    uint32_t step_it = 0, item_it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_it) {
      int b, h, q0, k_lo, n_steps;
      item_range(item, b, h, q0, k_lo, n_steps);
      const long long row_base = (long long)b * p.T;
      const int i = q0 + r;
      const bool row_ok = i < p.T;
      int lo_i = 0;
      float lse2 = INFINITY, dls = 0.f;
      if (row_ok) {
        if (p.lo) lo_i = p.lo[row_base + i];
        if (p.window > 0) lo_i = max(lo_i, i - p.window + 1);
        lse2 = p.lse[(row_base + i) * p.H + h] * 1.4426950408889634f;
        dls = p.delta[(row_base + i) * p.H + h] * sc;      // delta times the scale: dS = P (dP * scale - dls)
      }
      for (int t = 0; t < n_steps; ++t, ++step_it) {
        const int j0 = k_lo + t * KN;
        if (!at_wait(sdp_full, step_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const bool need_mask = !row_ok || (j0 + KN - 1 > q0) || (j0 < lo_i);
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(tmem_S + lane_base + cq * 32, rs);
        tmem_ld_32x32(tmem_dP + lane_base + cq * 32, rp);
        tmem_ld_wait();
        float ds[32];
        if (!need_mask) {
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const float pr = exp2f(fmaf(__uint_as_float(rs[k]), sc2, -lse2));
            ds[k] = pr * fmaf(__uint_as_float(rp[k]), sc, -dls);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const int j = j0 + cq * 32 + k;
            const bool vis = row_ok && j <= i && j >= lo_i;
            const float pr = vis ? exp2f(fmaf(__uint_as_float(rs[k]), sc2, -lse2)) : 0.f;
            ds[k] = pr * fmaf(__uint_as_float(rp[k]), sc, -dls);
          }
        }
        store_p_chunk<T>(sDS, r, cq * 32, ds);
        tc_fence_before();
        fence_proxy_async();
        __syncwarp();                 // every lane's writes and fences, then one arrival for the warp
        if (lane == 0) mbar_arrive(ds_ready);
      }
      if (!ok || !at_wait(dq_full, item_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) { ok = false; break; }
      tc_fence_after();
      T* dqp = reinterpret_cast<T*>(p.dq) + (row_base + i) * p.ld_dq + (long long)h * HD;
      uint32_t rg[32];
      tmem_ld_32x32(tmem_dQ + lane_base + cq * 32, rg);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint4 q;
          q.x = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 0]), __uint_as_float(rg[8 * k + 1]));
          q.y = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 2]), __uint_as_float(rg[8 * k + 3]));
          q.z = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 4]), __uint_as_float(rg[8 * k + 5]));
          q.w = Cvt<T>::pack2(__uint_as_float(rg[8 * k + 6]), __uint_as_float(rg[8 * k + 7]));
          reinterpret_cast<uint4*>(dqp + cq * 32)[k] = q;
        }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (*abort_flag) {
    for (int k = 0; k < 64; ++k) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == W_MMA) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// ============================================================================================ backward: dK, dV
// One CTA per (batch, kv head, 128 key rows).  Loops over the query heads that share the kv head and over the
// query tiles at or after the key tile.  Per iteration: S^T = K Q^T and dP^T = V dO^T into tensor memory (rows =
// keys, columns = queries), P^T and dS^T written to shared memory, dV += P^T dO and dK += dS^T Q accumulated in
// tensor memory over all iterations (ordered, so the GQA reduction is deterministic) and read out once.
template <typename T, int HD, int STAGES>
__global__ void __launch_bounds__(AT_BWD_THREADS) attn_tc_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                     const __grid_constant__ CUtensorMap tmK,
                                                                     const __grid_constant__ CUtensorMap tmV,
                                                                     const __grid_constant__ CUtensorMap tmDO,
                                                                     const AttnTcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t TILE = AT_M * HD * 2;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE;
  uint8_t* sQ = sV + TILE;                  // STAGES
  uint8_t* sDO = sQ + STAGES * TILE;        // STAGES
  uint8_t* sPT = sDO + STAGES * TILE;       // [128 keys x 128 queries]
  uint8_t* sDST = sPT + AT_M * AT_N * 2;
  float* sLse = reinterpret_cast<float*>(sDST + AT_M * AT_N * 2);   // [2][128]
  float* sDl = sLse + 2 * AT_N;
  int* sLo = reinterpret_cast<int*>(sDl + 2 * AT_N);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sLo + 2 * AT_N);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;              // 2
  uint64_t* q_empty = bars + 3;             // 2
  uint64_t* st_full = bars + 5;
  uint64_t* pt_ready = bars + 6;
  uint64_t* dkv_full = bars + 7;
  uint64_t* kv_empty = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Persistent: items are (key tile, batch, kv head), the first key tile first (every query tile reads it: the longest
  // loop); a CTA walks items blockIdx.x, blockIdx.x + gridDim.x, ... with tensor memory and barriers set up once.
  const int group = p.H / p.KV;
  const int n_kt = (p.T + AT_N - 1) / AT_N, BKV = p.B * p.KV;
  const int n_items = n_kt * BKV;
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(kv_empty, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    mbar_init(st_full, 1);
    mbar_init(pt_ready, AT_BWD_CW);
    mbar_init(dkv_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == AT_BWD_W_MMA) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_ST = tmem_base, tmem_dPT = tmem_base + AT_M, tmem_dV = tmem_base + 2 * AT_M,
                 tmem_dK = tmem_base + 2 * AT_M + HD;

  // key tile and query tiles share the 128-row grid: the query tiles of an item start at its key tile
  auto item_range = [&](int item, int& b, int& kvh, int& j0, int& n_qt) {
    const int jt = item / BKV, bk = item - jt * BKV;
    b = bk / p.KV;
    kvh = bk - b * p.KV;
    j0 = jt * AT_N;
    int i_hi = p.T;
    if (p.window > 0) i_hi = min(p.T, j0 + AT_N - 1 + p.window);
    n_qt = (i_hi - j0 + AT_M - 1) / AT_M;
  };

  if (warp == AT_BWD_W_TMA) {
    if (lane == 0) {
      uint32_t g_it = 0, item_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_it) {
        int b, kvh, j0, n_qt;
        item_range(item, b, kvh, j0, n_qt);
        const int row_base = b * p.T;
        // K and V of the previous item have been read (committed after its last S^T / dP^T)
        if (!at_wait(kv_empty, (item_it & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) break;
        mbar_arrive_expect_tx(kv_full, 2 * TILE);
        load_tile<HD>(&tmK, kv_full, sK, kvh * HD, row_base + j0);
        load_tile<HD>(&tmV, kv_full, sV, kvh * HD, row_base + j0);
        const int n_it = group * n_qt;
        for (int it = 0; it < n_it; ++it, ++g_it) {
          const int s = g_it % STAGES, ph = (g_it / STAGES) & 1;
          const int h = kvh * group + it / n_qt;
          const int i0 = j0 + (it % n_qt) * AT_M;
          if (!at_wait(&q_empty[s], ph ^ 1, p.status, ST_TIMEOUT_EMPTY, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&q_full[s], 2 * TILE);
          load_tile<HD>(&tmQ, &q_full[s], sQ + s * TILE, h * HD, row_base + i0);
          load_tile<HD>(&tmDO, &q_full[s], sDO + s * TILE, h * HD, row_base + i0);
        }
      }
    }
    __syncwarp();
  } else if (warp == AT_BWD_W_MMA) {
    if (lane == 0) {
      constexpr int fmt = OperandFmt<T>::value;
      const uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, AT_M, AT_N);
      const uint32_t idesc_d = make_idesc_f16(fmt, 0, 1, AT_M, HD);
      uint32_t g_it = 0, item_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_it) {
        int b, kvh, j0, n_qt;
        item_range(item, b, kvh, j0, n_qt);
        if (!at_wait(kv_full, item_it & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) break;
        const int n_it = group * n_qt;
        for (int it = 0; it < n_it; ++it, ++g_it) {
          const int s = g_it % STAGES, ph = (g_it / STAGES) & 1;
          if (!at_wait(&q_full[s], ph, p.status, ST_TIMEOUT_FULL, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_kmajor_kmajor<HD>(tmem_ST, smem_u32(sK), smem_u32(sQ + s * TILE), idesc_s, false);
          mma_kmajor_kmajor<HD>(tmem_dPT, smem_u32(sV), smem_u32(sDO + s * TILE), idesc_s, false);
          umma_commit(st_full);
          if (it == n_it - 1) umma_commit(kv_empty);
          if (!at_wait(pt_ready, g_it & 1u, p.status, ST_TIMEOUT_TMEM_EMPTY, abort_flag)) { ok = false; break; }
          tc_fence_after();
          // the first dV / dK of an item overwrite the accumulators: the compute warps have read the previous item's
          // before they arrived on pt_ready for this iteration
          mma_kmajor_mnmajor<AT_M>(tmem_dV, smem_u32(sPT), smem_u32(sDO + s * TILE), idesc_d, it > 0);
          mma_kmajor_mnmajor<AT_M>(tmem_dK, smem_u32(sDST), smem_u32(sQ + s * TILE), idesc_d, it > 0);
          umma_commit(&q_empty[s]);
        }
        if (ok) umma_commit(dkv_full);
      }
    }
    __syncwarp();
  } else {
    const int cq = warp >> 2;                  // 32-column (query) chunk of this warp
    const int r = (warp & 3) * 32 + lane;      // key row of this thread (its TMEM lane)
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const float sc = p.scale;
    const float sc2 = sc * 1.4426950408889634f;
    constexpr float LOG2E = 1.4426950408889634f;
    uint32_t g_it = 0, item_it = 0;
    bool ok = true;
    // Per-query statistics of an iteration (log-sum-exp in log2 units, delta, first visible key), fetched by the four
    // cq == 0 warps (thread r = column r) one iteration ahead, the next item's first iteration included: the loads
    // of iteration n + 1 are in flight while iteration n is computed.
    float n_lse = INFINITY, n_dl = 0.f;
    int n_lo = 0x7fffffff;
    auto fetch_stats = [&](int b, int h, int i0) {
      const int i = i0 + r;
      const bool in = i < p.T;
      const long long row = (long long)b * p.T + i;
      n_lse = in ? p.lse[row * p.H + h] * LOG2E : INFINITY;
      n_dl = in ? p.delta[row * p.H + h] * sc : 0.f;       // delta times the scale: dS = P (dP * scale - that)
      int lo = 0;
      if (in && p.lo) lo = p.lo[row];
      if (in && p.window > 0) lo = max(lo, i - p.window + 1);
      n_lo = in ? lo : 0x7fffffff;
    };
    if (cq == 0 && (int)blockIdx.x < n_items) {
      int b, kvh, j0, n_qt;
      item_range(blockIdx.x, b, kvh, j0, n_qt);
      fetch_stats(b, kvh * group, j0);
    }
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++item_it) {
      int b, kvh, j0, n_qt;
      item_range(item, b, kvh, j0, n_qt);
      const long long row_base = (long long)b * p.T;
      const int j = j0 + r;
      const bool row_ok = j < p.T;
      const int n_it = group * n_qt;
      for (int it = 0; it < n_it; ++it, ++g_it) {
        const int i0 = j0 + (it % n_qt) * AT_M;
        const int bufi = g_it & 1;
        if (cq == 0) {
          sLse[bufi * AT_N + r] = n_lse;
          sDl[bufi * AT_N + r] = n_dl;
          sLo[bufi * AT_N + r] = n_lo;
          if (it + 1 < n_it) {
            fetch_stats(b, kvh * group + (it + 1) / n_qt, j0 + ((it + 1) % n_qt) * AT_M);
          } else if (item + (int)gridDim.x < n_items) {
            int b2, kvh2, j02, n_qt2;
            item_range(item + gridDim.x, b2, kvh2, j02, n_qt2);
            fetch_stats(b2, kvh2 * group, j02);
          }
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");   // all AT_BWD_CW * 32 compute threads
        // after a failed wait the loops keep running (without waiting or computing) so that every thread still
        // reaches the named barrier above in every iteration
        if (ok && !at_wait(st_full, g_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) ok = false;
        if (!ok) continue;
        tc_fence_after();
        const float* lse = sLse + bufi * AT_N;
        const float* dl = sDl + bufi * AT_N;
        const int* lo = sLo + bufi * AT_N;
        // every (key, query) pair of the tile visible: a query tile after the key tile, whole tiles, and the largest
        // `lo` of the tile (its last column: lo does not decrease along a sequence) at or before the first key
        const bool full = i0 > j0 && j0 + AT_N <= p.T && i0 + AT_M <= p.T && lo[AT_M - 1] <= j0;
        {
          const int c = cq;
          uint32_t rs[32], rp[32];
          tmem_ld_32x32(tmem_ST + lane_base + c * 32, rs);
          tmem_ld_32x32(tmem_dPT + lane_base + c * 32, rp);
          tmem_ld_wait();
          float pt[32], ds[32];
          if (full) {
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const int col = c * 32 + k;
              const float pr = exp2f(fmaf(__uint_as_float(rs[k]), sc2, -lse[col]));
              pt[k] = pr;
              ds[k] = pr * fmaf(__uint_as_float(rp[k]), sc, -dl[col]);
            }
          } else {
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const int col = c * 32 + k;
              const int i = i0 + col;
              const bool vis = row_ok && j <= i && j >= lo[col];
              const float pr = vis ? exp2f(fmaf(__uint_as_float(rs[k]), sc2, -lse[col])) : 0.f;
              pt[k] = pr;
              ds[k] = pr * fmaf(__uint_as_float(rp[k]), sc, -dl[col]);
            }
          }
          store_p_chunk<T>(sPT, r, c * 32, pt);
          store_p_chunk<T>(sDST, r, c * 32, ds);
        }
        tc_fence_before();
        fence_proxy_async();
        __syncwarp();                 // every lane's writes and fences, then one arrival for the warp
        if (lane == 0) mbar_arrive(pt_ready);
      }
      if (ok && !at_wait(dkv_full, item_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) ok = false;
      if (!ok) continue;
      tc_fence_after();
      T* dkp = reinterpret_cast<T*>(p.dk) + (row_base + j) * p.ld_dk + (long long)kvh * HD;
      T* dvp = reinterpret_cast<T*>(p.dv) + (row_base + j) * p.ld_dv + (long long)kvh * HD;
      if (cq < HD / 32) {
        const int c = cq;
        uint32_t rv[32], rk[32];
        tmem_ld_32x32(tmem_dV + lane_base + c * 32, rv);
        tmem_ld_32x32(tmem_dK + lane_base + c * 32, rk);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 qv, qk;
            qv.x = Cvt<T>::pack2(__uint_as_float(rv[8 * k + 0]), __uint_as_float(rv[8 * k + 1]));
            qv.y = Cvt<T>::pack2(__uint_as_float(rv[8 * k + 2]), __uint_as_float(rv[8 * k + 3]));
            qv.z = Cvt<T>::pack2(__uint_as_float(rv[8 * k + 4]), __uint_as_float(rv[8 * k + 5]));
            qv.w = Cvt<T>::pack2(__uint_as_float(rv[8 * k + 6]), __uint_as_float(rv[8 * k + 7]));
            qk.x = Cvt<T>::pack2(__uint_as_float(rk[8 * k + 0]), __uint_as_float(rk[8 * k + 1]));
            qk.y = Cvt<T>::pack2(__uint_as_float(rk[8 * k + 2]), __uint_as_float(rk[8 * k + 3]));
            qk.z = Cvt<T>::pack2(__uint_as_float(rk[8 * k + 4]), __uint_as_float(rk[8 * k + 5]));
            qk.w = Cvt<T>::pack2(__uint_as_float(rk[8 * k + 6]), __uint_as_float(rk[8 * k + 7]));
            reinterpret_cast<uint4*>(dvp + c * 32)[k] = qv;
            reinterpret_cast<uint4*>(dkp + c * 32)[k] = qk;
          }
        }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (*abort_flag) {
    for (int k = 0; k < 64; ++k) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == AT_BWD_W_MMA) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ============================================================================================ backward: dK, dV (head_dim 64)
// The same product in query steps of 64 instead of 128: S^T 64 + dP^T 64 + dV 64 + dK 64 = 256 tensor-memory columns
// and under 100 KB of shared memory, so two CTAs of 8 compute warps share an SM (see the dQ kernel above for why).
template <typename T>
__global__ void __launch_bounds__(AT_DQ64_THREADS, 2) attn_tc_bwd_dkv64_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                           const __grid_constant__ CUtensorMap tmK,
                                                                           const __grid_constant__ CUtensorMap tmV,
                                                                           const __grid_constant__ CUtensorMap tmDO,
                                                                           const AttnTcParams p) {
  constexpr int HD = 64, QN = 64, ST = 2;
  constexpr int W_TMA = AT_DQ64_CW, W_MMA = AT_DQ64_CW + 1;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr uint32_t TILE = AT_N * HD * 2;          // K, V: [128 x 64]; P^T, dS^T of a step: [128 keys x 64 queries]
  constexpr uint32_t QTILE = QN * HD * 2;           // Q, dO of a step: [64 x 64]
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_BAD_ARGUMENT);
    return;
  }
  uint8_t* sK = smem_raw;
  uint8_t* sV = sK + TILE;
  uint8_t* sPT = sV + TILE;
  uint8_t* sDST = sPT + TILE;
  uint8_t* sQ = sDST + TILE;                // ST
  uint8_t* sDO = sQ + ST * QTILE;           // ST
  float* sLse = reinterpret_cast<float*>(sDO + ST * QTILE);   // [2][64]
  float* sDl = sLse + 2 * QN;
  int* sLo = reinterpret_cast<int*>(sDl + 2 * QN);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sLo + 2 * QN);
  uint64_t* kv_full = bars;
  uint64_t* kv_empty = bars + 1;
  uint64_t* st_full = bars + 2;
  uint64_t* pt_ready = bars + 3;
  uint64_t* dkv_full = bars + 4;
  uint64_t* q_full = bars + 5;              // ST
  uint64_t* q_empty = bars + 5 + ST;        // ST
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5 + 2 * ST);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.H / p.KV;
  const int n_kt = (p.T + AT_N - 1) / AT_N, BKV = p.B * p.KV;
  const int n_items = n_kt * BKV;
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(kv_empty, 1);
    mbar_init(st_full, 1);
    mbar_init(pt_ready, AT_DQ64_CW);
    mbar_init(dkv_full, 1);
    for (int s = 0; s < ST; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == W_MMA) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_ST = tmem_base, tmem_dPT = tmem_base + QN, tmem_dV = tmem_base + 2 * QN, tmem_dK = tmem_base + 2 * QN + HD;

  // the query steps of an item start at its key tile: n_qs steps of 64 queries for each head of the group
  auto item_range = [&](int item, int& b, int& kvh, int& j0, int& n_qs) {
    const int jt = item / BKV, bk = item - jt * BKV;
    b = bk / p.KV;
    kvh = bk - b * p.KV;
    j0 = jt * AT_N;
    int i_hi = p.T;
    if (p.window > 0) i_hi = min(p.T, j0 + AT_N - 1 + p.window);
    n_qs = (i_hi - j0 + QN - 1) / QN;
  };

  if (warp == W_TMA) {
    if (lane == 0) {
      uint32_t g_it = 0, item_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_it) {
        int b, kvh, j0, n_qs;
        item_range(item, b, kvh, j0, n_qs);
        const int row_base = b * p.T;
        if (!at_wait(kv_empty, (item_it & 1u) ^ 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) break;
        mbar_arrive_expect_tx(kv_full, 2 * TILE);
        load_tile<HD>(&tmK, kv_full, sK, kvh * HD, row_base + j0);
        load_tile<HD>(&tmV, kv_full, sV, kvh * HD, row_base + j0);
        const int n_it = group * n_qs;
        for (int it = 0; it < n_it; ++it, ++g_it) {
          const int s = g_it % ST, ph = (g_it / ST) & 1;
          const int h = kvh * group + it / n_qs;
          const int i0 = j0 + (it % n_qs) * QN;
          if (!at_wait(&q_empty[s], ph ^ 1, p.status, ST_TIMEOUT_EMPTY, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&q_full[s], 2 * QTILE);
          tma_load_2d(&tmQ, &q_full[s], sQ + s * QTILE, h * HD, row_base + i0);
          tma_load_2d(&tmDO, &q_full[s], sDO + s * QTILE, h * HD, row_base + i0);
        }
      }
    }
    __syncwarp();
  } else if (warp == W_MMA) {
    if (lane == 0) {
      constexpr int fmt = OperandFmt<T>::value;
      const uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, AT_N, QN);
      const uint32_t idesc_d = make_idesc_f16(fmt, 0, 1, AT_N, HD);
      uint32_t g_it = 0, item_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_it) {
        int b, kvh, j0, n_qs;
        item_range(item, b, kvh, j0, n_qs);
        if (!at_wait(kv_full, item_it & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) break;
        const int n_it = group * n_qs;
        for (int it = 0; it < n_it; ++it, ++g_it) {
          const int s = g_it % ST, ph = (g_it / ST) & 1;
          if (!at_wait(&q_full[s], ph, p.status, ST_TIMEOUT_FULL, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_kmajor_kmajor<HD>(tmem_ST, smem_u32(sK), smem_u32(sQ + s * QTILE), idesc_s, false);
          mma_kmajor_kmajor<HD>(tmem_dPT, smem_u32(sV), smem_u32(sDO + s * QTILE), idesc_s, false);
          umma_commit(st_full);
          if (it == n_it - 1) umma_commit(kv_empty);
          if (!at_wait(pt_ready, g_it & 1u, p.status, ST_TIMEOUT_TMEM_EMPTY, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_kmajor_mnmajor<QN>(tmem_dV, smem_u32(sPT), smem_u32(sDO + s * QTILE), idesc_d, it > 0);
          mma_kmajor_mnmajor<QN>(tmem_dK, smem_u32(sDST), smem_u32(sQ + s * QTILE), idesc_d, it > 0);
          umma_commit(&q_empty[s]);
        }
        if (ok) umma_commit(dkv_full);
      }
    }
    __syncwarp();
  } else {
    const int cq = warp >> 2;                  // 32-column chunk: of the 64 queries of a step, of the 64 of dV / dK
    const int r = (warp & 3) * 32 + lane;      // key row of this thread (its TMEM lane)
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const float sc = p.scale;
    const float sc2 = sc * 1.4426950408889634f;
    constexpr float LOG2E = 1.4426950408889634f;
    uint32_t g_it = 0, item_it = 0;
    bool ok = true;
    // statistics of the next step's 64 queries, fetched one step ahead by the first 64 compute threads
    const bool stat_thread = threadIdx.x < QN;
    float n_lse = INFINITY, n_dl = 0.f;
    int n_lo = 0x7fffffff;
    auto fetch_stats = [&](int b, int h, int i0) {
      const int i = i0 + (int)threadIdx.x;
      const bool in = i < p.T;
      const long long row = (long long)b * p.T + i;
      n_lse = in ? p.lse[row * p.H + h] * LOG2E : INFINITY;
      n_dl = in ? p.delta[row * p.H + h] * sc : 0.f;       // delta times the scale: dS = P (dP * scale - that)
      int lo = 0;
      if (in && p.lo) lo = p.lo[row];
      if (in && p.window > 0) lo = max(lo, i - p.window + 1);
      n_lo = in ? lo : 0x7fffffff;
    };
    if (stat_thread && (int)blockIdx.x < n_items) {
      int b, kvh, j0, n_qs;
      item_range(blockIdx.x, b, kvh, j0, n_qs);
      fetch_stats(b, kvh * group, j0);
    }
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++item_it) {
      int b, kvh, j0, n_qs;
      item_range(item, b, kvh, j0, n_qs);
      const long long row_base = (long long)b * p.T;
      const int j = j0 + r;
      const bool row_ok = j < p.T;
      const int n_it = group * n_qs;
      for (int it = 0; it < n_it; ++it, ++g_it) {
        const int i0 = j0 + (it % n_qs) * QN;
        const int bufi = g_it & 1;
        if (stat_thread) {
          sLse[bufi * QN + threadIdx.x] = n_lse;
          sDl[bufi * QN + threadIdx.x] = n_dl;
          sLo[bufi * QN + threadIdx.x] = n_lo;
          if (it + 1 < n_it) {
            fetch_stats(b, kvh * group + (it + 1) / n_qs, j0 + ((it + 1) % n_qs) * QN);
          } else if (item + (int)gridDim.x < n_items) {
            int b2, kvh2, j02, n_qs2;
            item_range(item + gridDim.x, b2, kvh2, j02, n_qs2);
            fetch_stats(b2, kvh2 * group, j02);
          }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");   // all AT_DQ64_CW * 32 compute threads
        // after a failed wait the loops keep running (without waiting or computing) so that every thread still
        // reaches the named barrier above in every step
        if (ok && !at_wait(st_full, g_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) ok = false;
        if (!ok) continue;
        tc_fence_after();
        const float* lse = sLse + bufi * QN;
        const float* dl = sDl + bufi * QN;
        const int* lo = sLo + bufi * QN;
        // every (key, query) pair of the step visible: queries after the whole key tile, whole tiles, and the largest
        // `lo` of the step (its last query) at or before the first key
        const bool full = i0 >= j0 + AT_N && j0 + AT_N <= p.T && i0 + QN <= p.T && lo[QN - 1] <= j0;
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(tmem_ST + lane_base + cq * 32, rs);
        tmem_ld_32x32(tmem_dPT + lane_base + cq * 32, rp);
        tmem_ld_wait();
        float pt[32], ds[32];
        // the statistics of this warp's 32 queries come as 16-byte loads (every lane reads the same words), four
        // queries at a time
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) {
          const float4 a4 = reinterpret_cast<const float4*>(lse + cq * 32)[k4];
          const float4 d4 = reinterpret_cast<const float4*>(dl + cq * 32)[k4];
          const float lv[4] = {a4.x, a4.y, a4.z, a4.w};
          const float dv[4] = {d4.x, d4.y, d4.z, d4.w};
          if (full) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int k = 4 * k4 + e;
              const float pr = exp2f(fmaf(__uint_as_float(rs[k]), sc2, -lv[e]));
              pt[k] = pr;
              ds[k] = pr * fmaf(__uint_as_float(rp[k]), sc, -dv[e]);
            }
          } else {
            const int4 l4 = reinterpret_cast<const int4*>(lo + cq * 32)[k4];
            const int lov[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int k = 4 * k4 + e;
              const int i = i0 + cq * 32 + k;
              const bool vis = row_ok && j <= i && j >= lov[e];
              const float pr = vis ? exp2f(fmaf(__uint_as_float(rs[k]), sc2, -lv[e])) : 0.f;
              pt[k] = pr;
              ds[k] = pr * fmaf(__uint_as_float(rp[k]), sc, -dv[e]);
            }
          }
        }
        store_p_chunk<T>(sPT, r, cq * 32, pt);
        store_p_chunk<T>(sDST, r, cq * 32, ds);
        tc_fence_before();
        fence_proxy_async();
        __syncwarp();                 // every lane's writes and fences, then one arrival for the warp
        if (lane == 0) mbar_arrive(pt_ready);
      }
      if (ok && !at_wait(dkv_full, item_it & 1u, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) ok = false;
      if (!ok) continue;
      tc_fence_after();
      T* dkp = reinterpret_cast<T*>(p.dk) + (row_base + j) * p.ld_dk + (long long)kvh * HD;
      T* dvp = reinterpret_cast<T*>(p.dv) + (row_base + j) * p.ld_dv + (long long)kvh * HD;
      uint32_t rv[32], rk[32];
      tmem_ld_32x32(tmem_dV + lane_base + cq * 32, rv);
      tmem_ld_32x32(tmem_dK + lane_base + cq * 32, rk);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint4 qv, qk;
          qv.x = Cvt<T>::pack2(__uint_as_float(rv[8 * k + 0]), __uint_as_float(rv[8 * k + 1]));
          qv.y = Cvt<T>::pack2(__uint_as_float(rv[8 * k + 2]), __uint_as_float(rv[8 * k + 3]));
          qv.z = Cvt<T>::pack2(__uint_as_float(rv[8 * k + 4]), __uint_as_float(rv[8 * k + 5]));
          qv.w = Cvt<T>::pack2(__uint_as_float(rv[8 * k + 6]), __uint_as_float(rv[8 * k + 7]));
          qk.x = Cvt<T>::pack2(__uint_as_float(rk[8 * k + 0]), __uint_as_float(rk[8 * k + 1]));
          qk.y = Cvt<T>::pack2(__uint_as_float(rk[8 * k + 2]), __uint_as_float(rk[8 * k + 3]));
          qk.z = Cvt<T>::pack2(__uint_as_float(rk[8 * k + 4]), __uint_as_float(rk[8 * k + 5]));
          qk.w = Cvt<T>::pack2(__uint_as_float(rk[8 * k + 6]), __uint_as_float(rk[8 * k + 7]));
          reinterpret_cast<uint4*>(dvp + cq * 32)[k] = qv;
          reinterpret_cast<uint4*>(dkp + cq * 32)[k] = qk;
        }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (*abort_flag) {
    for (int k = 0; k < 64; ++k) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == W_MMA) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// lo[i] = first position of the run of equal segment ids that contains i (per sequence).  Rows with a negative id see
// every earlier key (lo = 0) as long as no non-negative id has come before them in the sequence; after one they count
// as a run of their own.  That keeps lo non-decreasing along a sequence, which the tensor-core kernels rely on (the
// first row of a tile has its smallest lo, the last one its largest).
// One block of 1024 threads per sequence: running maximum of the run-start positions (chunked inclusive scan).
__global__ void __launch_bounds__(1024) attn_seg_lo_kernel(const int* __restrict__ seg, int* __restrict__ lo, int B, int T) {
  __shared__ int s_warp[32], s_flag[32];
  __shared__ int s_carry, s_carry_f;
  const long long base = (long long)blockIdx.x * T;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) { s_carry = 0; s_carry_f = 0; }
  __syncthreads();
  for (int c0 = 0; c0 < T; c0 += 1024) {
    const int i = c0 + threadIdx.x;
    int s = 0, v = 0, f = 0;                 // f: a non-negative id at or before i
    if (i < T) {
      s = seg[base + i];
      if (i == 0 || seg[base + i - 1] != s) v = i;
      f = s >= 0 ? 1 : 0;
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, v, o);
      const int nf = __shfl_up_sync(0xffffffffu, f, o);
      if (lane >= o) { v = max(v, n); f = max(f, nf); }
    }
    if (lane == 31) { s_warp[warp] = v; s_flag[warp] = f; }
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane], wf = s_flag[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, w, o);
        const int nf = __shfl_up_sync(0xffffffffu, wf, o);
        if (lane >= o) { w = max(w, n); wf = max(wf, nf); }
      }
      s_warp[lane] = w;
      s_flag[lane] = wf;
    }
    __syncthreads();
    if (warp > 0) { v = max(v, s_warp[warp - 1]); f = max(f, s_flag[warp - 1]); }
    v = max(v, s_carry);
    f = max(f, s_carry_f);
    if (i < T) lo[base + i] = (s < 0 && !f) ? 0 : v;
    __syncthreads();
    if (threadIdx.x == 1023) { s_carry = v; s_carry_f = f; }
    __syncthreads();
  }
}

template <typename T, int HD>
int launch_tc_fwd(const gb_attn_args* a, int* lo, int* status, cudaStream_t st) {
  CUtensorMap tq, tk, tv;
  const long long rows = (long long)a->B * a->T;
  if (gb_make_tmap_2d_16b(&tq, a->q, rows, (uint64_t)a->H * HD, a->ld_q, AT_M, 64, a->is_bf16)) return -20;
  if (gb_make_tmap_2d_16b(&tk, a->k, rows, (uint64_t)a->KV * HD, a->ld_k, AT_N, 64, a->is_bf16)) return -21;
  if (gb_make_tmap_2d_16b(&tv, a->v, rows, (uint64_t)a->KV * HD, a->ld_v, AT_N, 64, a->is_bf16)) return -22;
  if (!(a->scale > 0.f)) return -1;            // the row maximum is taken on raw scores
  AttnTcParams p{};
  p.B = a->B; p.T = a->T; p.H = a->H; p.KV = a->KV; p.window = a->window; p.scale = a->scale;
  p.lo = lo; p.o = a->o; p.ld_o = a->ld_o; p.lse = a->lse; p.status = status;
  constexpr size_t smem = (size_t)AT_M * HD * 2 * 5 + AT_M * AT_N * 2 + 128 + (HD == 64 ? 0 : 1024);
  auto kern = attn_tc_fwd_kernel<T, HD>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -10;
    // the largest shared-memory carve-out, so that two 112 KB CTAs fit one SM
    (void)cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    attr = true;
  }
  // persistent: as many CTAs as fit the device at once (two per SM at head_dim 64), each walking its share of the items
  static int resident = 0;
  if (!resident) {
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return -10;
    // two 112 KB CTAs share an SM at head_dim 64 (the carve-out preference above); the occupancy query does not see
    // that preference, so the count is stated here
    per_sm = HD == 64 ? 2 : 1;
    resident = sms * per_sm;
  }
  const long long n_items = (long long)((a->T + AT_M - 1) / AT_M) * a->B * a->H;
  if (n_items > 0x7fffffffll - resident) return -1;
  const unsigned grid = (unsigned)std::min<long long>(n_items, resident);
  kern<<<grid, AT_THREADS, smem, st>>>(tq, tk, tv, p);
  return gb_launch_rc();
}

template <typename T>
__global__ void attn_tc_delta_kernel(const T* __restrict__ d_o, long long ld_do, const T* __restrict__ o, long long ld_o,
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

// The same with HD/8 lanes per (token, head) and one 16-byte load of each operand per lane: 256/HD rows per warp.
template <typename T, int HD>
__global__ void __launch_bounds__(256) attn_tc_delta_vec_kernel(const T* __restrict__ d_o, long long ld_do,
                                                                const T* __restrict__ o, long long ld_o,
                                                                float* __restrict__ delta, long long n_tok, int H) {
  constexpr int LPI = HD / 8, IPW = 32 / LPI;
  const int lane = threadIdx.x & 31, sub = lane / LPI, j = lane % LPI;
  const long long item = (blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5)) * IPW + sub;
  const bool live = item < n_tok * H;
  float s = 0.f;
  if (live) {
    const long long t = item / H;
    const int h = (int)(item - t * H);
    const uint4 qa = *reinterpret_cast<const uint4*>(d_o + t * ld_do + (long long)h * HD + 8 * j);
    const uint4 qb = *reinterpret_cast<const uint4*>(o + t * ld_o + (long long)h * HD + 8 * j);
    const float2 a0 = Cvt<T>::unpack2(qa.x), a1 = Cvt<T>::unpack2(qa.y), a2 = Cvt<T>::unpack2(qa.z), a3 = Cvt<T>::unpack2(qa.w);
    const float2 b0 = Cvt<T>::unpack2(qb.x), b1 = Cvt<T>::unpack2(qb.y), b2 = Cvt<T>::unpack2(qb.z), b3 = Cvt<T>::unpack2(qb.w);
    s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
  }
#pragma unroll
  for (int off = LPI / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (live && j == 0) delta[item] = s;
}

template <typename T, int HD>
int launch_tc_bwd(const gb_attn_args* a, int* lo, int* status, cudaStream_t st) {
  constexpr int STAGES = HD == 64 ? 2 : 1;
  CUtensorMap tq, tk, tv, tdo;
  const long long rows = (long long)a->B * a->T;
  if (gb_make_tmap_2d_16b(&tq, a->q, rows, (uint64_t)a->H * HD, a->ld_q, AT_M, 64, a->is_bf16)) return -20;
  if (gb_make_tmap_2d_16b(&tk, a->k, rows, (uint64_t)a->KV * HD, a->ld_k, AT_N, 64, a->is_bf16)) return -21;
  if (gb_make_tmap_2d_16b(&tv, a->v, rows, (uint64_t)a->KV * HD, a->ld_v, AT_N, 64, a->is_bf16)) return -22;
  if (gb_make_tmap_2d_16b(&tdo, a->d_o, rows, (uint64_t)a->H * HD, a->ld_do, AT_M, 64, a->is_bf16)) return -23;
  if (a->ld_do % 8 == 0 && a->ld_o % 8 == 0 && (((uintptr_t)a->d_o | (uintptr_t)a->o) & 15) == 0) {
    constexpr int per_block = 8 * (256 / HD);
    attn_tc_delta_vec_kernel<T, HD><<<(unsigned)((rows * a->H + per_block - 1) / per_block), 256, 0, st>>>(
        reinterpret_cast<const T*>(a->d_o), a->ld_do, reinterpret_cast<const T*>(a->o), a->ld_o, a->delta, rows, a->H);
  } else {
    attn_tc_delta_kernel<T><<<(unsigned)((rows * a->H + 7) / 8), 256, 0, st>>>(
        reinterpret_cast<const T*>(a->d_o), a->ld_do, reinterpret_cast<const T*>(a->o), a->ld_o, a->delta, rows, a->H, HD);
  }
  AttnTcParams p{};
  p.B = a->B; p.T = a->T; p.H = a->H; p.KV = a->KV; p.window = a->window; p.scale = a->scale;
  p.lo = lo; p.lse = a->lse; p.delta = a->delta; p.status = status;
  p.dq = a->dq; p.ld_dq = a->ld_dq; p.dk = a->dk; p.ld_dk = a->ld_dk; p.dv = a->dv; p.ld_dv = a->ld_dv;
  constexpr size_t TILE = (size_t)AT_M * HD * 2;
  constexpr size_t smem_q = TILE * (2 + 2 * STAGES) + AT_M * AT_N * 2 + 128 + 1024;
  constexpr size_t smem_kv = TILE * (2 + 2 * STAGES) + 2 * AT_M * AT_N * 2 + 6 * AT_N * 4 + 128 + 1024;
  auto kq = attn_tc_bwd_dq_kernel<T, HD, STAGES>;
  auto kkv = attn_tc_bwd_dkv_kernel<T, HD, STAGES>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q) != cudaSuccess) return -10;
    if (cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv) != cudaSuccess) return -10;
    attr = true;
  }
  // persistent: one CTA per SM (each holds all 512 tensor-memory columns), walking its share of the items
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        sms < 1) {
      sms = 0;
      return -10;
    }
  }
  const long long tiles = (a->T + AT_M - 1) / AT_M;
  const long long items_q = tiles * a->B * a->H, items_kv = tiles * a->B * a->KV;
  if (items_q > 0x7fffffffll - sms) return -1;
  if constexpr (HD == 64) {
    // key steps of 64, two CTAs per SM
    CUtensorMap tk64, tv64;
    if (gb_make_tmap_2d_16b(&tk64, a->k, rows, (uint64_t)a->KV * HD, a->ld_k, 64, 64, a->is_bf16)) return -21;
    if (gb_make_tmap_2d_16b(&tv64, a->v, rows, (uint64_t)a->KV * HD, a->ld_v, 64, 64, a->is_bf16)) return -22;
    auto kq64 = attn_tc_bwd_dq64_kernel<T>;
    constexpr size_t smem_q64 = TILE * 3 + (size_t)64 * HD * 2 * 2 * AT_DQ64_STAGES + 128;
    static bool attr64 = false;
    if (!attr64) {
      if (cudaFuncSetAttribute(kq64, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q64) != cudaSuccess) return -10;
      (void)cudaFuncSetAttribute(kq64, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      attr64 = true;
    }
    kq64<<<(unsigned)std::min<long long>(items_q, 2ll * sms), AT_DQ64_THREADS, smem_q64, st>>>(tq, tk64, tv64, tdo, p);
  } else {
    kq<<<(unsigned)std::min<long long>(items_q, sms), AT_BWD_THREADS, smem_q, st>>>(tq, tk, tv, tdo, p);
  }
  if constexpr (HD == 64) {
    // query steps of 64, two CTAs per SM
    CUtensorMap tq64, tdo64;
    if (gb_make_tmap_2d_16b(&tq64, a->q, rows, (uint64_t)a->H * HD, a->ld_q, 64, 64, a->is_bf16)) return -20;
    if (gb_make_tmap_2d_16b(&tdo64, a->d_o, rows, (uint64_t)a->H * HD, a->ld_do, 64, 64, a->is_bf16)) return -23;
    auto kkv64 = attn_tc_bwd_dkv64_kernel<T>;
    constexpr size_t smem_kv64 = TILE * 4 + (size_t)64 * HD * 2 * 2 * 2 + 6 * 64 * 4 + 128;
    static bool attr_kv64 = false;
    if (!attr_kv64) {
      if (cudaFuncSetAttribute(kkv64, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv64) != cudaSuccess) return -10;
      (void)cudaFuncSetAttribute(kkv64, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      attr_kv64 = true;
    }
    kkv64<<<(unsigned)std::min<long long>(items_kv, 2ll * sms), AT_DQ64_THREADS, smem_kv64, st>>>(tq64, tk, tv, tdo64, p);
  } else {
    kkv<<<(unsigned)std::min<long long>(items_kv, sms), AT_BWD_THREADS, smem_kv, st>>>(tq, tk, tv, tdo, p);
  }
  return gb_launch_rc();
}

}  // namespace gb

using namespace gb;

extern "C" int gb_attn_tc_bwd(const gb_attn_args* a, int* lo_scratch, int lo_ready, int* status, cudaStream_t st) {
  if (!a || !status || a->B <= 0 || a->T <= 0 || a->H % a->KV) return -1;
  if (a->hd != 64 && a->hd != 128) return -2;
  if (!a->d_o || !a->delta || !a->lse || !a->dq || !a->dk || !a->dv || !a->o) return -1;
  if ((a->seg || lo_ready) && !lo_scratch) return -1;
  int* lo = nullptr;
  if (lo_ready) {
    lo = lo_scratch;                 // filled earlier by gb_attn_seg_lo for the same segment ids
  } else if (a->seg) {
    attn_seg_lo_kernel<<<a->B, 1024, 0, st>>>(a->seg, lo_scratch, a->B, a->T);
    lo = lo_scratch;
  }
  if (a->is_bf16) return a->hd == 64 ? launch_tc_bwd<__nv_bfloat16, 64>(a, lo, status, st) : launch_tc_bwd<__nv_bfloat16, 128>(a, lo, status, st);
  return a->hd == 64 ? launch_tc_bwd<__half, 64>(a, lo, status, st) : launch_tc_bwd<__half, 128>(a, lo, status, st);
}

// Tensor-core attention forward.  `lo_scratch` ([B*T] int32) is needed when a->seg is given: segment ids must form
// contiguous runs inside each sequence (packed documents).  Supports head_dim 64 and 128; other sizes: gb_attn_fwd.
// lo[i] = start of the run of equal segment ids containing i; compute once per batch and pass lo_ready = 1 below.
extern "C" int gb_attn_seg_lo(const int* seg, int* lo, int B, int T, cudaStream_t st) {
  if (!seg || !lo || B <= 0 || T <= 0) return -1;
  attn_seg_lo_kernel<<<B, 1024, 0, st>>>(seg, lo, B, T);
  return gb_launch_rc();
}

extern "C" int gb_attn_tc_fwd(const gb_attn_args* a, int* lo_scratch, int lo_ready, int* status, cudaStream_t st) {
  if (!a || !status || a->B <= 0 || a->T <= 0 || a->H % a->KV) return -1;
  if (a->hd != 64 && a->hd != 128) return -2;
  if ((a->seg || lo_ready) && !lo_scratch) return -1;
  int* lo = nullptr;
  if (lo_ready) {
    lo = lo_scratch;                 // filled earlier by gb_attn_seg_lo for the same segment ids
  } else if (a->seg) {
    attn_seg_lo_kernel<<<a->B, 1024, 0, st>>>(a->seg, lo_scratch, a->B, a->T);
    lo = lo_scratch;
  }
  if (a->is_bf16) return a->hd == 64 ? launch_tc_fwd<__nv_bfloat16, 64>(a, lo, status, st) : launch_tc_fwd<__nv_bfloat16, 128>(a, lo, status, st);
  return a->hd == 64 ? launch_tc_fwd<__half, 64>(a, lo, status, st) : launch_tc_fwd<__half, 128>(a, lo, status, st);
}
