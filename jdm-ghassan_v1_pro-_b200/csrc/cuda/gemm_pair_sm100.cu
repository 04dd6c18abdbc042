// Two-SM GEMM for sm_100a: a cluster of two CTAs computes one 256 x 256 output tile with
// tcgen05.mma.cta_group::2.  Each CTA stages 128 rows of A and 128 rows (output columns) of B per 64-deep
// k-block, so a k-block costs each SM 32 KB of shared-memory traffic where the one-CTA 128 x 256 tile costs 48 KB;
// each CTA keeps its 128 x 256 half of the accumulator in its own tensor memory (two buffers, 512 columns) and
// drains it through shared memory with TMA stores: an epilogue warp converts 32 rows x 128 bytes, writes them into
// a 128-byte-swizzled 4 KB slot and one lane issues the bulk store, so no warp waits on a global store and every
// store is a full 128-byte line.  fp32 accumulation into an existing matrix (weight gradients) is a TMA reduce-add;
// the SwiGLU backward epilogue also fetches the saved gate/up block with TMA ahead of the accumulator.
//
// Nothing here is a multicast load: both CTAs issue their own cp.async.bulk.tensor loads (cta_group::2 form, bytes
// counted on the barrier of CTA 0, which issues the MMAs).  The two signals that go to both CTAs are tcgen05.commit
// arrivals.  All waits are bounded and end in a status code, as in the one-CTA kernel (gemm_sm100.cu), which stays
// the path for small problems, per-tile destinations and unaligned outputs.
//
// Same roles as there: warps 0-7 epilogue (two per TMEM lane quarter, each a 128-column half), warp 8 TMA producer,
// warp 9 MMA issuer (CTA 0 only).  Replaces the reference's cuBLAS call sites (cuda/kernels.cu:97-325) and the
// per-expert GEMM loops (cuda/moe.cu:678-970) for every shape with enough 256 x 256 tiles to fill the GPU.
#include "sm100_common.cuh"
#include "gb_api.h"

namespace gb {
namespace pr {

static constexpr int HM = 128;        // A rows per CTA  (pair tile: 256)
static constexpr int HN = 128;        // B rows per CTA  (pair tile: 256 output columns)
static constexpr int TM = 256, TN = 256;
static constexpr int BK = 64, UMMA_K = 16;
static constexpr int THREADS = 320, W_TMA = 8, W_MMA = 9, EPI_WARPS = 8;
static constexpr uint32_t A_BYTES = HM * BK * 2, B_BYTES = HN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
static constexpr uint32_t SLOT_BYTES = 4096;   // 32 rows x 128 bytes
static constexpr uint32_t TMEM_COLS = 512;
static constexpr uint32_t BAR_BYTES = 512;

enum { EPI_STORE = 0, EPI_SWIGLU_FWD = 1, EPI_SWIGLU_BWD = 2 };

struct Params {
  int M, N, K;
  int a_mn, b_mn, fmt;
  int mode;                    // 0 dense, 1 expert-sorted rows, 2 grouped over the reduction dim
  const int* tile_expert;      // mode 1: expert of each 128-row tile (tiles 2i and 2i+1 must agree)
  const int* num_m_tiles;      // mode 1: live 128-row tiles (device scalar)
  const int* seg_offsets;      // mode 2
  int groups;
  int b_group_rows;
  const float* addend;         // fp32 out only: out = acc + addend (a different matrix than out)
  int ld_add;
  int reduce;                  // fp32 out only: out += acc through TMA reduce-add
  int has_aux_out;             // SwiGLU forward: also store the interleaved gate/up pre-activations
  int a_mn3, b_mn3;            // the MN-major operand's map is the chunked 3-D view: one load per k-block
  int* status;
};

struct Tile {
  int m0, n0, b_row_off, k_begin, k_end, g;
};

__device__ __forceinline__ Tile decode(const Params& p, int tile, int tiles_m, int tiles_n) {
  Tile t;
  t.b_row_off = 0;
  t.k_begin = 0;
  t.k_end = p.K;
  t.g = 0;
  if (p.mode == 2) {
    // groups from the last to the first: the always-on expert is the last group and the longest reduction
    const int per = tiles_m * tiles_n;
    const int gi = tile / per, r = tile - gi * per;
    t.g = p.groups - 1 - gi;
    t.m0 = (r % tiles_m) * TM;
    t.n0 = (r / tiles_m) * TN;
    t.k_begin = p.seg_offsets[t.g];
    t.k_end = p.seg_offsets[t.g + 1];
  } else {
    const int tm = tile / tiles_n, tn = tile - tm * tiles_n;   // column tiles of one row block are neighbours
    t.m0 = tm * TM;
    t.n0 = tn * TN;
    if (p.mode == 1) t.b_row_off = p.tile_expert[2 * tm] * p.b_group_rows;
  }
  return t;
}

// Bounded wait shared by all roles of a CTA: gives up when another role has given up or after ~2 s.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, int* status, int code, volatile int* abort_flag) {
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 2048; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > 4000000000LL) {
      atomicCAS(status, 0, code);
      *abort_flag = 1;
      return false;
    }
  }
}

// 16-byte piece j of this lane's 128-byte row inside a swizzled slot (the layout TMA expects for SWIZZLE_128B)
__device__ __forceinline__ uint4* slot_piece(uint8_t* slot, int lane, int j) {
  return reinterpret_cast<uint4*>(slot + lane * 128 + ((j ^ (lane & 7)) << 4));
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.f + __expf(-g)); }

template <int EPI, int STAGES, int SLOTS, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmO, const __grid_constant__ CUtensorMap tmX, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* slots = smem + STAGES * STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(slots + EPI_WARPS * SLOTS * SLOT_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* aux_bar = tempty_bar + 2;               // [EPI_WARPS][2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux_bar + 2 * EPI_WARPS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = the CTA that issues the MMAs

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 2 * EPI_WARPS); }
    for (int i = 0; i < 2 * EPI_WARPS; ++i) mbar_init(&aux_bar[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == W_MMA) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == W_TMA && lane == 0) {
    tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmO);
    if (EPI != EPI_STORE) tma_prefetch_desc(&tmX);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();        // both CTAs' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.mode == 1) ? (*p.num_m_tiles + 1) / 2 : (p.M + TM - 1) / TM;
  const int tiles_n = (p.N + TN - 1) / TN;
  const int total_tiles = tiles_m * tiles_n * (p.mode == 2 ? p.groups : 1);
  const int pair_id = (int)cluster_id_x(), n_pairs = (int)cluster_nctaid_x();

  if (warp == W_TMA) {
    // ------------------------------------------------------------- TMA producer (one per CTA, for its own halves)
    if (lane == 0) {
      const uint32_t full0 = mapa_shared(smem_u32(&full_bar[0]), 0);   // the full barriers that count are CTA 0's
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair_id; tile < total_tiles && ok; tile += n_pairs) {
        const Tile t = decode(p, tile, tiles_m, tiles_n);
        const int am = t.m0 + (int)rank * HM, bn = t.n0 + (int)rank * HN;
        for (int k = t.k_begin; k < t.k_end; k += BK, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!wait_bar(&empty_bar[s], ph ^ 1, p.status, ST_TIMEOUT_EMPTY, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * STAGE_BYTES);   // both CTAs' bytes
          const uint32_t fb = full0 + s * 8;
          if (!p.a_mn) {
            tma_load_2d_pair(&tmA, fb, sa, k, am);
          } else if (p.a_mn3) {
            tma_load_3d_pair(&tmA, fb, sa, 0, k, am >> 6);
          } else {
#pragma unroll
            for (int c = 0; c < HM / 64; ++c) tma_load_2d_pair(&tmA, fb, sa + c * (64 * 128), am + c * 64, k);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(&tmB, fb, sb, k, t.b_row_off + bn);
          } else if (p.b_mn3) {
            tma_load_3d_pair(&tmB, fb, sb, 0, t.b_row_off + k, bn >> 6);
          } else {
#pragma unroll
            for (int c = 0; c < HN / 64; ++c) tma_load_2d_pair(&tmB, fb, sb + c * (64 * 128), bn + c * 64, t.b_row_off + k);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == W_MMA) {
    // ------------------------------------------------------------- MMA issuer (CTA 0 only)
    if (rank == 0 && lane == 0) {
      const uint32_t idesc = make_idesc_f16(p.fmt, p.a_mn, p.b_mn, TM, TN);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int tile = pair_id; tile < total_tiles && ok; tile += n_pairs) {
        const Tile t = decode(p, tile, tiles_m, tiles_n);
        if (t.k_end <= t.k_begin) continue;
        const uint32_t ab = acc_it & 1, aph = (acc_it >> 1) & 1;
        if (!wait_bar(&tempty_bar[ab], aph ^ 1, p.status, ST_TIMEOUT_TMEM_EMPTY, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * TN;
        bool first = true;
        for (int k = t.k_begin; k < t.k_end; k += BK, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!wait_bar(&full_bar[s], ph, p.status, ST_TIMEOUT_FULL, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          // same operand layouts as the one-CTA kernel with 128-row A and B tiles; the other CTA's halves sit at
          // the same shared-memory offsets
          const uint64_t da = p.a_mn ? make_smem_desc_sw128(sa, 64 * 128, 1024) : make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t db = p.b_mn ? make_smem_desc_sw128(sb, 64 * 128, 1024) : make_smem_desc_sw128(sb, 16, 1024);
          const uint64_t a_step = p.a_mn ? (2048 >> 4) : (32 >> 4);
          const uint64_t b_step = p.b_mn ? (2048 >> 4) : (32 >> 4);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            umma_f16_pair(d_tmem, da + kk * a_step, db + kk * b_step, idesc, first ? 0u : 1u);
            first = false;
          }
          umma_commit_pair(&empty_bar[s], 3);     // frees this stage in both CTAs
        }
        if (ok) umma_commit_pair(&tfull_bar[ab], 3);
        ++acc_it;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------- epilogue (warps 0-7 of both CTAs)
    const int quarter = warp & 3, half = warp >> 2;
    uint8_t* my_slots = slots + warp * (SLOTS * SLOT_BYTES);
    uint64_t* my_aux = aux_bar + 2 * warp;
    const uint32_t tempty0 = mapa_shared(smem_u32(&tempty_bar[0]), 0);
    uint32_t acc_it = 0, n_slot = 0;
    uint32_t aux_cnt[2] = {0, 0};     // completed phases of this warp's two load barriers
    bool ok = true;
    // next free slot; the SLOTS-1 most recent stores may still be reading theirs
    auto acquire = [&]() -> uint8_t* {
      if (lane == 0) bulk_wait_read<SLOTS - 1>();
      __syncwarp();
      uint8_t* s = my_slots + (n_slot % SLOTS) * SLOT_BYTES;
      ++n_slot;
      return s;
    };
    for (int tile = pair_id; tile < total_tiles && ok; tile += n_pairs) {
      const Tile t = decode(p, tile, tiles_m, tiles_n);
      const bool empty_k = (t.k_end <= t.k_begin);
      const int row_q = t.m0 + (int)rank * HM + quarter * 32;   // first of this warp's 32 rows
      const int colh = t.n0 + half * 128;                       // first of this warp's 128 accumulator columns
      const bool rows_live = row_q < p.M;

      if constexpr (EPI == EPI_SWIGLU_BWD) {
        // fetch the saved [64 gate | 64 up] blocks of both 64-column halves before the accumulator is waited for
        if (lane == 0) {
          bulk_wait_read<0>();          // the previous tile's stores have left the slots
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            const int j = colh + blk * 64;
            if (rows_live && j < p.N) {
              const int gcol = (j >> 6) * 128;
              mbar_arrive_expect_tx(&my_aux[blk], 2 * SLOT_BYTES);
              tma_load_3d(&tmX, &my_aux[blk], my_slots + (2 * blk) * SLOT_BYTES, gcol, row_q, 0);
              tma_load_3d(&tmX, &my_aux[blk], my_slots + (2 * blk + 1) * SLOT_BYTES, gcol + 64, row_q, 0);
            }
          }
        }
        __syncwarp();
      }

      uint32_t ab = 0;
      if (!empty_k) {
        ab = acc_it & 1;
        const uint32_t aph = (acc_it >> 1) & 1;
        if (!wait_bar(&tfull_bar[ab], aph, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) { ok = false; break; }
        tc_fence_after();
      }
      const uint32_t taddr = tmem_base + ab * TN + half * 128 + (uint32_t(quarter * 32) << 16);

      if constexpr (EPI == EPI_STORE && sizeof(OutT) == 2) {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {               // 64-column chunks
          uint32_t r0[32], r1[32];
          if (!empty_k) {
            tmem_ld_32x32(taddr + c * 64, r0);
            tmem_ld_32x32(taddr + c * 64 + 32, r1);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) { r0[i] = 0; r1[i] = 0; }
          }
          uint8_t* slot = acquire();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 q;
            q.x = Cvt<OutT>::pack2(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
            q.y = Cvt<OutT>::pack2(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
            q.z = Cvt<OutT>::pack2(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
            q.w = Cvt<OutT>::pack2(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
            *slot_piece(slot, lane, j) = q;
            q.x = Cvt<OutT>::pack2(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
            q.y = Cvt<OutT>::pack2(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
            q.z = Cvt<OutT>::pack2(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
            q.w = Cvt<OutT>::pack2(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
            *slot_piece(slot, lane, j + 4) = q;
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            const int col = colh + c * 64;
            if (rows_live && col < p.N) tma_store_3d(&tmO, slot, col, row_q, t.g);
            bulk_commit();
          }
        }
      } else if constexpr (EPI == EPI_STORE) {
        // fp32 output, 32-column chunks: plain store, store of acc + addend, or reduce-add into the matrix
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          const int col = colh + c * 32;
          uint32_t r[32];
          if (!empty_k) {
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0;
          }
          if (empty_k && p.reduce) continue;        // nothing to add (warp-uniform)
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (p.addend) {
            const int row = row_q + lane;
            if (row < p.M && col < p.N) {
              const float* arow = p.addend + (long long)row * p.ld_add + col;
              if (p.N - col >= 32 && (reinterpret_cast<uintptr_t>(arow) & 15) == 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float4 f = __ldg(reinterpret_cast<const float4*>(arow) + i);
                  v[4 * i] += f.x; v[4 * i + 1] += f.y; v[4 * i + 2] += f.z; v[4 * i + 3] += f.w;
                }
              } else {
                for (int i = 0; i < 32; ++i)
                  if (col + i < p.N) v[i] += arow[i];
              }
            }
          }
          uint8_t* slot = acquire();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 q;
            q.x = __float_as_uint(v[4 * j]); q.y = __float_as_uint(v[4 * j + 1]);
            q.z = __float_as_uint(v[4 * j + 2]); q.w = __float_as_uint(v[4 * j + 3]);
            *slot_piece(slot, lane, j) = q;
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            if (rows_live && col < p.N) {
              if (p.reduce) tma_reduce_add_3d(&tmO, slot, col, row_q, t.g);
              else tma_store_3d(&tmO, slot, col, row_q, t.g);
            }
            bulk_commit();
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU_FWD) {
        // this warp's 128 accumulator columns are one [64 gate | 64 up] block: 64 activation columns
        uint32_t act[32];                           // silu(g) * u, packed pairs, 64 columns
        uint8_t* sg = nullptr;
        uint8_t* su = nullptr;
        if (p.has_aux_out) { sg = acquire(); su = acquire(); }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(taddr + h2 * 32, rg);
          tmem_ld_32x32(taddr + 64 + h2 * 32, ru);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float g[8], u[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { g[i] = __uint_as_float(rg[8 * j + i]); u[i] = __uint_as_float(ru[8 * j + i]); }
            if (p.has_aux_out) {
              uint4 q;
              q.x = Cvt<OutT>::pack2(g[0], g[1]); q.y = Cvt<OutT>::pack2(g[2], g[3]);
              q.z = Cvt<OutT>::pack2(g[4], g[5]); q.w = Cvt<OutT>::pack2(g[6], g[7]);
              *slot_piece(sg, lane, h2 * 4 + j) = q;
              q.x = Cvt<OutT>::pack2(u[0], u[1]); q.y = Cvt<OutT>::pack2(u[2], u[3]);
              q.z = Cvt<OutT>::pack2(u[4], u[5]); q.w = Cvt<OutT>::pack2(u[6], u[7]);
              *slot_piece(su, lane, h2 * 4 + j) = q;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
              act[(h2 * 4 + j) * 4 + i] = Cvt<OutT>::pack2(silu_f(g[2 * i]) * u[2 * i], silu_f(g[2 * i + 1]) * u[2 * i + 1]);
          }
        }
        const bool live = rows_live && (colh + 64) < p.N;   // the up half bounds the block
        if (p.has_aux_out) {
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            if (live) tma_store_3d(&tmX, sg, colh, row_q, 0);
            bulk_commit();
            if (live) tma_store_3d(&tmX, su, colh + 64, row_q, 0);
            bulk_commit();
          }
        }
        uint8_t* sa = acquire();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *slot_piece(sa, lane, j) = make_uint4(act[4 * j], act[4 * j + 1], act[4 * j + 2], act[4 * j + 3]);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          if (live) tma_store_3d(&tmO, sa, colh >> 1, row_q, 0);
          bulk_commit();
        }
      } else {
        // EPI_SWIGLU_BWD: acc = d(act)[row, j]; (g, u) arrive by TMA in the slots and are overwritten with (dg, du)
#pragma unroll 1
        for (int blk = 0; blk < 2; ++blk) {
          const int j0 = colh + blk * 64;
          const bool live = rows_live && j0 < p.N;      // warp-uniform
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + blk * 64, r0);
          tmem_ld_32x32(taddr + blk * 64 + 32, r1);
          tmem_ld_wait();
          if (!live) continue;
          if (!wait_bar(&my_aux[blk], aux_cnt[blk] & 1, p.status, ST_TIMEOUT_AUX, abort_flag)) { ok = false; break; }
          ++aux_cnt[blk];
          uint8_t* sg = my_slots + (2 * blk) * SLOT_BYTES;
          uint8_t* su = sg + SLOT_BYTES;
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const uint4 qg = *slot_piece(sg, lane, jj), qu = *slot_piece(su, lane, jj);
            const uint32_t gw[4] = {qg.x, qg.y, qg.z, qg.w}, uw[4] = {qu.x, qu.y, qu.z, qu.w};
            uint32_t dgw[4], duw[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 g2 = Cvt<OutT>::unpack2(gw[i]), u2 = Cvt<OutT>::unpack2(uw[i]);
              const int e = jj * 8 + 2 * i;
              const float da0 = __uint_as_float(e < 32 ? r0[e & 31] : r1[e & 31]);
              const float da1 = __uint_as_float(e < 32 ? r0[(e + 1) & 31] : r1[(e + 1) & 31]);
              const float s0 = 1.f / (1.f + __expf(-g2.x)), s1 = 1.f / (1.f + __expf(-g2.y));
              duw[i] = Cvt<OutT>::pack2(da0 * g2.x * s0, da1 * g2.y * s1);
              dgw[i] = Cvt<OutT>::pack2(da0 * u2.x * (s0 * (1.f + g2.x * (1.f - s0))),
                                        da1 * u2.y * (s1 * (1.f + g2.y * (1.f - s1))));
            }
            *slot_piece(sg, lane, jj) = make_uint4(dgw[0], dgw[1], dgw[2], dgw[3]);
            *slot_piece(su, lane, jj) = make_uint4(duw[0], duw[1], duw[2], duw[3]);
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            const int gcol = (j0 >> 6) * 128;
            tma_store_3d(&tmO, sg, gcol, row_q, 0);
            tma_store_3d(&tmO, su, gcol + 64, row_q, 0);
            bulk_commit();
          }
        }
        if (!ok) break;
      }

      if (!empty_k) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty0 + ab * 8);
        ++acc_it;
      }
    }
    if (lane == 0) bulk_wait<0>();      // every store has left shared memory and is complete
    __syncwarp();
  }

  __syncthreads();
  cluster_sync_all();       // neither CTA leaves while the other may still touch its shared or tensor memory
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);   // copies still in flight get time to land
    __syncthreads();
  }
  if (warp == W_MMA) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <int STAGES, int SLOTS>
constexpr size_t smem_bytes() {
  return size_t(STAGES) * STAGE_BYTES + size_t(EPI_WARPS) * SLOTS * SLOT_BYTES + BAR_BYTES + 1024;
}

}  // namespace pr
}  // namespace gb

// =============================================================================== host side
int gb_make_tmap_3d_box128(CUtensorMap* out, const void* base, int dtype, uint64_t cols, uint64_t rows, uint64_t groups,
                           uint64_t ld, uint64_t group_stride, uint32_t box_rows) {
  gb_encode_tiled_fn enc = gb_get_encode_tiled();
  if (!enc) return -1;
  const uint64_t es = dtype == 2 ? 4 : 2;
  if (groups < 1) groups = 1;
  if (groups == 1) group_stride = ld * rows;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * es) & 15) || ((group_stride * es) & 15)) return -2;
  cuuint64_t dims[3] = {cols, rows, groups};
  cuuint64_t strides[2] = {ld * es, group_stride * es};
  cuuint32_t box[3] = {(cuuint32_t)(128 / es), box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = dtype == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

int gb_make_tmap_mn_chunks(CUtensorMap* out, const void* base, uint64_t k_rows, uint64_t mn, uint64_t ld, uint32_t box_k,
                           uint32_t chunks, int is_bf16) {
  gb_encode_tiled_fn enc = gb_get_encode_tiled();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15) || (mn & 63)) return -2;
  cuuint64_t dims[3] = {64, k_rows, mn / 64};
  cuuint64_t strides[2] = {ld * 2, 128};
  cuuint32_t box[3] = {64, box_k, chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

namespace {

template <int EPI, int STAGES, int SLOTS, typename OutT>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const CUtensorMap& tx,
                const gb::pr::Params& p, int max_tiles, cudaStream_t st) {
  auto kern = gb::pr::gemm_pair_kernel<EPI, STAGES, SLOTS, OutT>;
  constexpr size_t smem = gb::pr::smem_bytes<STAGES, SLOTS>();
  static_assert(smem <= 232448, "shared memory of the pair kernel exceeds 227 KB");
  static int max_pairs = 0;        // clusters of two that the device holds at once
  if (!max_pairs) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -10;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(gb::pr::THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      int dev = 0, sms = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      n = sms > 1 ? sms / 2 : 1;
    }
    max_pairs = n;
  }
  int pairs = max_tiles < max_pairs ? max_tiles : max_pairs;
  if (pairs < 1) pairs = 1;
  kern<<<2 * pairs, gb::pr::THREADS, smem, st>>>(ta, tb, to, tx, p);
  return gb_launch_rc();
}

}  // namespace

// Two-CTA path of gb_gemm (args->pair != 0).  Returns -20 .. -29 when the problem does not fit this kernel; the
// caller (ops/gemm.py: pair_ok) is expected to ask only for what does.
extern "C" int gb_gemm_pair(const gb_gemm_args* a, cudaStream_t st) {
  namespace pr = gb::pr;
  if (!a || a->M <= 0 || a->N <= 0 || a->K < 0 || !a->status) return -1;
  if (a->mode != 2 && a->K <= 0) return -1;
  if (a->tile_out) return -20;
  const int ot = a->out_dtype;
  if (a->addend && ot != 2) return -21;
  pr::Params p{};
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.a_mn = a->a_mn_major; p.b_mn = a->b_mn_major; p.fmt = a->is_bf16;
  p.mode = a->mode;
  p.tile_expert = a->tile_expert; p.num_m_tiles = a->num_m_tiles; p.seg_offsets = a->seg_offsets;
  p.groups = a->groups > 0 ? a->groups : 1;
  p.b_group_rows = a->b_group_rows;
  p.status = a->status;
  if (a->mode == 1 && (!a->tile_expert || !a->num_m_tiles)) return -1;
  if (a->mode == 2 && !a->seg_offsets) return -1;
  const int groups = a->mode == 2 ? p.groups : 1;
  if (a->addend) {
    if (a->addend == a->out && a->ld_add == a->ldo) p.reduce = 1;
    else if (a->mode == 2) return -22;     // a separate addend is only read in the dense mode
    else { p.addend = a->addend; p.ld_add = a->ld_add; }
  }

  CUtensorMap ta, tb, to, tx;
  int rc;
  // An MN-major operand is fetched with one chunked 3-D load per k-block (measured 4-10 % faster on the weight
  // gradients than two 2-D loads); a matrix whose width is not a multiple of 64 keeps the 2-D boxes.
  const bool chunked = true;
  if (!a->a_mn_major) rc = gb_make_tmap_2d_16b(&ta, a->A, a->a_rows, a->a_cols, a->lda, pr::HM, pr::BK, a->is_bf16);
  else if (chunked && a->a_cols % 64 == 0) {
    rc = gb_make_tmap_mn_chunks(&ta, a->A, a->a_rows, a->a_cols, a->lda, pr::BK, pr::HM / 64, a->is_bf16);
    p.a_mn3 = 1;
  } else rc = gb_make_tmap_2d_16b(&ta, a->A, a->a_rows, a->a_cols, a->lda, pr::BK, 64, a->is_bf16);
  if (rc) return rc - 100;
  if (!a->b_mn_major) rc = gb_make_tmap_2d_16b(&tb, a->B, a->b_rows, a->b_cols, a->ldb, pr::HN, pr::BK, a->is_bf16);
  else if (chunked && a->b_cols % 64 == 0) {
    rc = gb_make_tmap_mn_chunks(&tb, a->B, a->b_rows, a->b_cols, a->ldb, pr::BK, pr::HN / 64, a->is_bf16);
    p.b_mn3 = 1;
  } else rc = gb_make_tmap_2d_16b(&tb, a->B, a->b_rows, a->b_cols, a->ldb, pr::BK, 64, a->is_bf16);
  if (rc) return rc - 200;

  const int tiles_m = (a->M + pr::TM - 1) / pr::TM, tiles_n = (a->N + pr::TN - 1) / pr::TN;
  const int max_tiles = tiles_m * tiles_n * groups;

  switch (a->epilogue) {
    case pr::EPI_STORE: {
      rc = gb_make_tmap_3d_box128(&to, a->out, ot, a->N, a->M, groups, a->ldo, a->out_group_stride, 32);
      if (rc) return rc - 300;
      tx = to;
      if (ot == 2) return launch_pair<pr::EPI_STORE, 5, 2, float>(ta, tb, to, tx, p, max_tiles, st);
      if (ot == 1) return launch_pair<pr::EPI_STORE, 5, 2, __nv_bfloat16>(ta, tb, to, tx, p, max_tiles, st);
      return launch_pair<pr::EPI_STORE, 5, 2, __half>(ta, tb, to, tx, p, max_tiles, st);
    }
    case pr::EPI_SWIGLU_FWD: {
      if (a->N % 128 || ot == 2 || a->mode == 2) return -23;
      rc = gb_make_tmap_3d_box128(&to, a->out, ot, a->N / 2, a->M, 1, a->ldo, 0, 32);
      if (rc) return rc - 300;
      tx = to;
      if (a->aux_out) {
        rc = gb_make_tmap_3d_box128(&tx, a->aux_out, ot, a->N, a->M, 1, a->ld_aux, 0, 32);
        if (rc) return rc - 400;
        p.has_aux_out = 1;
      }
      if (ot == 1) return launch_pair<pr::EPI_SWIGLU_FWD, 4, 3, __nv_bfloat16>(ta, tb, to, tx, p, max_tiles, st);
      return launch_pair<pr::EPI_SWIGLU_FWD, 4, 3, __half>(ta, tb, to, tx, p, max_tiles, st);
    }
    case pr::EPI_SWIGLU_BWD: {
      if (a->N % 64 || ot == 2 || a->mode == 2 || !a->aux_in) return -24;
      rc = gb_make_tmap_3d_box128(&to, a->out, ot, 2LL * a->N, a->M, 1, a->ldo, 0, 32);
      if (rc) return rc - 300;
      rc = gb_make_tmap_3d_box128(&tx, a->aux_in, ot, 2LL * a->N, a->M, 1, a->ld_aux, 0, 32);
      if (rc) return rc - 400;
      if (ot == 1) return launch_pair<pr::EPI_SWIGLU_BWD, 3, 4, __nv_bfloat16>(ta, tb, to, tx, p, max_tiles, st);
      return launch_pair<pr::EPI_SWIGLU_BWD, 3, 4, __half>(ta, tb, to, tx, p, max_tiles, st);
    }
  }
  return -1;
}
