// Persistent warp-specialised GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma
// with the accumulator in tensor memory (double-buffered so the epilogue of tile i overlaps the
// main loop of tile i+1) -> tcgen05.ld epilogue with fused cast / residual add / SwiGLU.
//
// One kernel serves every matrix product of the model:
//   dense            C[M,N]  = A[M,K] * B[N,K]^T                 (forward linears, lm-head)
//   operand majors   A and B may each be K-major (reduction dim contiguous) or MN-major, which covers
//                    dgrad (B = W stored [N_red, K_out]) and wgrad (both operands row-major over tokens)
//   grouped-M        rows are expert-sorted, every 128-row tile belongs to one expert (device-side map)
//   grouped-K        one output per expert, reduction runs over that expert's (padded) row range
// It replaces the reference's cuBLAS GemmEx call sites and per-expert GEMM loops
// (cuda/kernels.cu:97-325, cuda/moe.cu:678-970 in the reference tree).
#include "sm100_common.cuh"
#include "gb_api.h"

namespace gb {

static constexpr int BM = 128;
static constexpr int BK = 64;       // 64 x 2 B = one 128-byte swizzle row
static constexpr int UMMA_K = 16;
static constexpr int GEMM_THREADS = 320;  // warps 0-7 epilogue (two per TMEM lane quarter), warp 8 TMA producer, warp 9 MMA issuer
static constexpr int W_TMA = 8, W_MMA = 9, EPI_THREADS = 256;

struct GemmParams {
  int M, N, K;
  int a_mn_major, b_mn_major, fmt;
  int mode;                   // 0 dense, 1 grouped-M, 2 grouped-K
  const int* tile_expert;     // mode 1: expert of each 128-row tile
  const int* num_m_tiles;     // mode 1: device scalar, number of live 128-row tiles
  const int* seg_offsets;     // mode 2: [groups+1] padded row offsets (multiples of 128)
  int groups;
  int b_group_rows;           // rows per group in the stored B matrix (mode 1)
  void* out; int ldo; long long out_group_stride;
  const float* addend; int ld_add;
  void* aux_out;              // SwiGLU fwd: interleaved gate/up copy (may be null)
  const void* aux_in;         // SwiGLU bwd: saved interleaved gate/up
  int ld_aux;
  const long long* tile_out;  // mode 1, plain store: address of row 0 of each 128-row tile's output (may be a peer GPU's memory)
  int* status;
};

enum { EPI_STORE = 0, EPI_SWIGLU_FWD = 1, EPI_SWIGLU_BWD = 2,
       EPI_STORE_TILED = 3 };   // EPI_STORE with per-tile destinations (16-bit output), chosen by the launcher

__device__ __forceinline__ bool wait_or_flag(uint64_t* bar, uint32_t parity, int* status, int code, volatile int* abort_flag) {
  long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 2048; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag) return false;
    if (clock64() - t0 > 4000000000LL) {  // ~2 s at 1.9 GHz
      atomicCAS(status, 0, code);
      *abort_flag = 1;
      return false;
    }
  }
}

struct TileInfo {
  int a_row0;      // first row of the A tile (logical m)
  int n0;          // first logical output column
  int b_row_off;   // stored-row offset applied to B (expert selection)
  int k_begin, k_end;
  long long out_off;
  int tm;          // index of the 128-row tile (modes 0 and 1)
  bool valid;
};

template <int BN>
__device__ __forceinline__ TileInfo decode_tile(const GemmParams& p, int tile, int tiles_m, int tiles_n) {
  TileInfo t;
  t.valid = true;
  t.b_row_off = 0;
  t.out_off = 0;
  t.k_begin = 0;
  t.k_end = p.K;
  t.tm = 0;
  if (p.mode == 2) {
    int per = tiles_m * tiles_n;
    int g = tile / per;
    int r = tile - g * per;
    t.a_row0 = (r % tiles_m) * BM;
    t.n0 = (r / tiles_m) * BN;
    t.k_begin = p.seg_offsets[g];
    t.k_end = p.seg_offsets[g + 1];
    t.out_off = (long long)g * p.out_group_stride;
  } else {
    // column tiles of one row block are neighbours in the schedule: the CTAs that run at the same time share the
    // A rows (fetched from DRAM once, then L2 hits), and B -- one expert's weights, a few MB -- stays in L2 anyway
    int tm = tile / tiles_n;
    int tn = tile - tm * tiles_n;
    t.a_row0 = tm * BM;
    t.n0 = tn * BN;
    t.tm = tm;
    if (p.mode == 1) {
      int e = p.tile_expert[tm];
      t.b_row_off = e * p.b_group_rows;
    }
  }
  return t;
}

template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* dst, const float (&v)[32], int ncols_valid) {
  if (ncols_valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 q;
        q.x = Cvt<OutT>::pack2(v[8 * i + 0], v[8 * i + 1]);
        q.y = Cvt<OutT>::pack2(v[8 * i + 2], v[8 * i + 3]);
        q.z = Cvt<OutT>::pack2(v[8 * i + 4], v[8 * i + 5]);
        q.w = Cvt<OutT>::pack2(v[8 * i + 6], v[8 * i + 7]);
        reinterpret_cast<uint4*>(dst)[i] = q;
      }
    }
  } else {
    for (int i = 0; i < 32; ++i)
      if (i < ncols_valid) dst[i] = Cvt<OutT>::from_f(v[i]);
  }
}

template <typename T>
__device__ __forceinline__ void load_row32(const T* src, float (&v)[32], int ncols_valid) {
  if (ncols_valid >= 32 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 f = reinterpret_cast<const float4*>(src)[i];
        v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 q = reinterpret_cast<const uint4*>(src)[i];
        float2 a = Cvt<T>::unpack2(q.x), b = Cvt<T>::unpack2(q.y), c = Cvt<T>::unpack2(q.z), d = Cvt<T>::unpack2(q.w);
        v[8 * i + 0] = a.x; v[8 * i + 1] = a.y; v[8 * i + 2] = b.x; v[8 * i + 3] = b.y;
        v[8 * i + 4] = c.x; v[8 * i + 5] = c.y; v[8 * i + 6] = d.x; v[8 * i + 7] = d.y;
      }
    }
  } else {
    for (int i = 0; i < 32; ++i) v[i] = (i < ncols_valid) ? Cvt<T>::to_f(src[i]) : 0.f;
  }
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.f + __expf(-g)); }

template <int BN, int STAGES, int EPI, typename OutT, typename InT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: [stages][A 16 KB][B BN*128 B] then barriers
  constexpr uint32_t A_BYTES = BM * BK * 2;
  constexpr uint32_t B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // 2 KB per epilogue warp: a 32 x 32 block of 16-bit results is turned from "one row per lane" into "four lanes per
  // row" before it goes to a per-tile destination (another GPU's memory likes 64-byte pieces, not 16-byte ones)
  uint8_t* stage = smem + STAGES * STAGE_BYTES + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], EPI_THREADS); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == W_MMA) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == W_TMA && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int tiles_m = (p.mode == 1) ? *p.num_m_tiles : (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int total_tiles = tiles_m * tiles_n * (p.mode == 2 ? p.groups : 1);

  if (warp == W_TMA) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        TileInfo t = decode_tile<BN>(p, tile, tiles_m, tiles_n);
        for (int k = t.k_begin; k < t.k_end; k += BK, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!wait_or_flag(&empty_bar[s], ph ^ 1, p.status, ST_TIMEOUT_EMPTY, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
          if (!p.a_mn_major) {
            tma_load_2d(&tmA, &full_bar[s], sa, k, t.a_row0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(&tmA, &full_bar[s], sa + c * (64 * 128), t.a_row0 + c * 64, k);
          }
          if (!p.b_mn_major) {
            tma_load_2d(&tmB, &full_bar[s], sb, k, t.b_row_off + t.n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(&tmB, &full_bar[s], sb + c * (64 * 128), t.n0 + c * 64, t.b_row_off + k);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == W_MMA) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(p.fmt, p.a_mn_major, p.b_mn_major, BM, BN);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        TileInfo t = decode_tile<BN>(p, tile, tiles_m, tiles_n);
        if (t.k_end <= t.k_begin) continue;
        const uint32_t ab = acc_it & 1, aph = (acc_it >> 1) & 1;
        if (!wait_or_flag(&tempty_bar[ab], aph ^ 1, p.status, ST_TIMEOUT_TMEM_EMPTY, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * BN;
        bool first = true;
        for (int k = t.k_begin; k < t.k_end; k += BK, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!wait_or_flag(&full_bar[s], ph, p.status, ST_TIMEOUT_FULL, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          // K-major: rows of 128 B, 8-row groups 1024 B apart; k16 step = 32 B inside the swizzle row.
          // MN-major: 64-element chunks (8 KB apart), 8 k-rows = 1024 B; k16 step = 16 rows = 2048 B.
          const uint64_t da = p.a_mn_major ? make_smem_desc_sw128(sa, 64 * 128, 1024) : make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t db = p.b_mn_major ? make_smem_desc_sw128(sb, 64 * 128, 1024) : make_smem_desc_sw128(sb, 16, 1024);
          const uint64_t a_step = p.a_mn_major ? (2048 >> 4) : (32 >> 4);
          const uint64_t b_step = p.b_mn_major ? (2048 >> 4) : (32 >> 4);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            umma_f16(d_tmem, da + kk * a_step, db + kk * b_step, idesc, first ? 0u : 1u);
            first = false;
          }
          umma_commit(&empty_bar[s]);  // smem stage is free once these MMAs retire
        }
        if (ok) umma_commit(&tfull_bar[ab]);
        ++acc_it;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------- epilogue (warps 0-7)
    // A warp reads the 32 TMEM lanes of its quarter (warp % 4); warps q and q+4 share a quarter and split the
    // tile's columns in halves, so two warps drain each row group.  One row per thread.
    uint32_t acc_it = 0;
    bool ok = true;
    const int quarter = warp & 3, half = warp >> 2;
    const int r_in_tile = quarter * 32 + lane;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      TileInfo t = decode_tile<BN>(p, tile, tiles_m, tiles_n);
      const bool empty_k = (t.k_end <= t.k_begin);
      uint32_t ab = 0;
      if (!empty_k) {
        ab = acc_it & 1;
        const uint32_t aph = (acc_it >> 1) & 1;
        if (!wait_or_flag(&tfull_bar[ab], aph, p.status, ST_TIMEOUT_TMEM_FULL, abort_flag)) { ok = false; break; }
        tc_fence_after();
      }
      const int row = t.a_row0 + r_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t taddr0 = tmem_base + ab * BN + (uint32_t(quarter * 32) << 16);
      if constexpr (EPI == EPI_STORE || EPI == EPI_STORE_TILED) {
        // per-tile destinations: the rows of this tile go to wherever the table says (expert-parallel combine
        // writes them straight into the buffer of the GPU that owns the tokens)
        OutT* orow = p.tile_out ? reinterpret_cast<OutT*>(p.tile_out[t.tm]) + (long long)r_in_tile * p.ldo
                                : reinterpret_cast<OutT*>(p.out) + t.out_off + (long long)row * p.ldo;
        const float* arow = p.addend ? p.addend + t.out_off + (long long)row * p.ld_add : nullptr;
        constexpr int CH = BN / 64;            // 32-column chunks per half
#pragma unroll 1
        for (int c0 = half * CH; c0 < (half + 1) * CH; c0 += 2) {
          constexpr int NB = CH >= 2 ? 2 : 1;   // chunks loaded per wait
          uint32_t r[NB][32];
          if (!empty_k) {
#pragma unroll
            for (int b = 0; b < NB; ++b) tmem_ld_32x32(taddr0 + (c0 + b) * 32, r[b]);
            tmem_ld_wait();
          }
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = empty_k ? 0.f : __uint_as_float(r[b][i]);
            const int col = t.n0 + (c0 + b) * 32;
            const int nvalid = p.N - col;
            if constexpr (EPI == EPI_STORE_TILED && sizeof(OutT) == 2) {
              if (nvalid >= 32) {                               // warp-uniform: col and N are
                uint4* ws = reinterpret_cast<uint4*>(stage + warp * 2048);
                __syncwarp();
#pragma unroll
                for (int pp = 0; pp < 4; ++pp) {
                  uint4 q;
                  q.x = Cvt<OutT>::pack2(v[8 * pp + 0], v[8 * pp + 1]);
                  q.y = Cvt<OutT>::pack2(v[8 * pp + 2], v[8 * pp + 3]);
                  q.z = Cvt<OutT>::pack2(v[8 * pp + 4], v[8 * pp + 5]);
                  q.w = Cvt<OutT>::pack2(v[8 * pp + 6], v[8 * pp + 7]);
                  ws[lane * 4 + (pp ^ ((lane >> 1) & 3))] = q;      // swizzled: quarter-warps hit eight bank groups
                }
                __syncwarp();
                OutT* tbase = reinterpret_cast<OutT*>(p.tile_out[t.tm]);
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                  const int rr = it * 8 + (lane >> 2), part = lane & 3;
                  const uint4 q = ws[rr * 4 + (part ^ ((rr >> 1) & 3))];
                  const int grow = quarter * 32 + rr;
                  if (t.a_row0 + grow < p.M)
                    *reinterpret_cast<uint4*>(tbase + (long long)grow * p.ldo + col + part * 8) = q;
                }
                continue;
              }
            }
            if (row_ok && nvalid > 0) {
              if (arow) {
                float a[32];
                load_row32<float>(arow + col, a, nvalid);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] += a[i];
              }
              store_row32<OutT>(orow + col, v, nvalid);
            }
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU_FWD) {
        // every 128 tile columns hold [64 gate_j | 64 up_j] for 64 consecutive j; a pair = 32 gate columns and the
        // matching 32 up columns.  BN/64 pairs per tile, split between the two column halves.
        static_assert(EPI != EPI_SWIGLU_FWD || BN % 128 == 0, "SwiGLU forward epilogue needs BN % 128 == 0");
        constexpr int PAIRS_PER_HALF = BN / 128;
        OutT* act_row = reinterpret_cast<OutT*>(p.out) + (long long)row * p.ldo;
        OutT* gu_row = p.aux_out ? reinterpret_cast<OutT*>(p.aux_out) + (long long)row * p.ld_aux : nullptr;
#pragma unroll 1
        for (int pp = half * PAIRS_PER_HALF; pp < (half + 1) * PAIRS_PER_HALF; ++pp) {
          const int gcol = (pp >> 1) * 128 + (pp & 1) * 32;   // gate columns inside the tile; up = gcol + 64
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(taddr0 + gcol, rg);
          tmem_ld_32x32(taddr0 + gcol + 64, ru);
          tmem_ld_wait();
          float g[32], u[32], a[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            g[i] = __uint_as_float(rg[i]);
            u[i] = __uint_as_float(ru[i]);
            a[i] = silu_f(g[i]) * u[i];
          }
          const int nvalid = p.N - (t.n0 + gcol + 64);  // columns of the up half bound both halves
          if (row_ok && nvalid > 0) {
            if (gu_row) {
              store_row32<OutT>(gu_row + t.n0 + gcol, g, nvalid);
              store_row32<OutT>(gu_row + t.n0 + gcol + 64, u, nvalid);
            }
            store_row32<OutT>(act_row + (t.n0 >> 1) + (pp >> 1) * 64 + (pp & 1) * 32, a, nvalid);
          }
        }
      } else {
        // EPI_SWIGLU_BWD: acc = d(act)[row, j]; consumes saved interleaved (g,u), emits interleaved (dg,du)
        const InT* gu = reinterpret_cast<const InT*>(p.aux_in) + (long long)row * p.ld_aux;
        OutT* dgu = reinterpret_cast<OutT*>(p.out) + (long long)row * p.ldo;
#pragma unroll 1
        for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr0 + c * 32, r);
          tmem_ld_wait();
          const int j = t.n0 + c * 32;
          const int nvalid = p.N - j;
          if (row_ok && nvalid > 0) {
            const int base = (j >> 6) * 128 + (j & 63);
            float g[32], u[32], dg[32], du[32];
            load_row32<InT>(gu + base, g, nvalid);
            load_row32<InT>(gu + base + 64, u, nvalid);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float da = __uint_as_float(r[i]);
              const float sg = 1.f / (1.f + __expf(-g[i]));
              const float sl = g[i] * sg;
              du[i] = da * sl;
              dg[i] = da * u[i] * (sg * (1.f + g[i] * (1.f - sg)));
            }
            store_row32<OutT>(dgu + base, dg, nvalid);
            store_row32<OutT>(dgu + base + 64, du, nvalid);
          }
        }
      }
      if (!empty_k) {
        tc_fence_before();
        mbar_arrive(&tempty_bar[ab]);
        ++acc_it;
      }
    }
  }

  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight time to land before shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == W_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int STAGES>
constexpr size_t gemm_smem_bytes() {
  return size_t(STAGES) * (BM * BK * 2 + BN * BK * 2) + 256 /* barriers */ + 8 * 2048 /* epilogue staging */ + 1024;
}

}  // namespace gb

// =============================================================================== host side
gb_encode_tiled_fn gb_get_encode_tiled() {
  static gb_encode_tiled_fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<gb_encode_tiled_fn>(p);
  }
  return fn;
}

int gb_make_tmap_2d_16b(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                        uint32_t box_rows, uint32_t box_cols, int is_bf16) {
  gb_encode_tiled_fn enc = gb_get_encode_tiled();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   box_cols * 2 == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

namespace {

int g_num_sms = 0;
int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int BN, int STAGES, int EPI, typename OutT, typename InT>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const gb::GemmParams& p, int max_tiles, cudaStream_t st) {
  auto kern = gb::gemm_tcgen05_kernel<BN, STAGES, EPI, OutT, InT>;
  constexpr size_t smem = gb::gemm_smem_bytes<BN, STAGES>();
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return -10;
    attr_set = true;
  }
  int grid = max_tiles < num_sms() ? max_tiles : num_sms();
  if (grid < 1) grid = 1;
  kern<<<grid, gb::GEMM_THREADS, smem, st>>>(ta, tb, p);
  return gb_launch_rc();
}

template <int EPI, typename OutT, typename InT>
int dispatch_bn(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const gb::GemmParams& p, int max_tiles, cudaStream_t st) {
  if constexpr (EPI == gb::EPI_SWIGLU_FWD) {
    if (bn == 256) return launch_gemm<256, 4, EPI, OutT, InT>(ta, tb, p, max_tiles, st);
    return launch_gemm<128, 6, EPI, OutT, InT>(ta, tb, p, max_tiles, st);
  } else {
    if (bn == 64) return launch_gemm<64, 8, EPI, OutT, InT>(ta, tb, p, max_tiles, st);
    if (bn == 256) return launch_gemm<256, 4, EPI, OutT, InT>(ta, tb, p, max_tiles, st);
    return launch_gemm<128, 6, EPI, OutT, InT>(ta, tb, p, max_tiles, st);
  }
}

}  // namespace

// Public launcher.  All pointers are device pointers; see gb_api.h for the argument contract.
extern "C" int gb_gemm(const gb_gemm_args* a, cudaStream_t st) {
  if (!a || a->M <= 0 || a->N <= 0 || a->K < 0) return -1;
  if (a->pair) return gb_gemm_pair(a, st);
  const int bn = a->block_n ? a->block_n : 128;
  if (bn != 64 && bn != 128 && bn != 256) return -1;
  gb::GemmParams p{};
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.a_mn_major = a->a_mn_major; p.b_mn_major = a->b_mn_major; p.fmt = a->is_bf16;
  p.mode = a->mode;
  p.tile_expert = a->tile_expert; p.num_m_tiles = a->num_m_tiles; p.seg_offsets = a->seg_offsets;
  p.groups = a->groups > 0 ? a->groups : 1;
  p.b_group_rows = a->b_group_rows;
  p.out = a->out; p.ldo = a->ldo; p.out_group_stride = a->out_group_stride;
  p.addend = a->addend; p.ld_add = a->ld_add;
  p.aux_out = a->aux_out; p.aux_in = a->aux_in; p.ld_aux = a->ld_aux;
  p.tile_out = (a->mode == 1 && a->epilogue == gb::EPI_STORE && !a->addend) ? a->tile_out : nullptr;
  if (a->tile_out && !p.tile_out) return -1;
  p.status = a->status;
  if (!p.status) return -1;

  // Tensor maps over the stored matrices.
  CUtensorMap ta, tb;
  int rc;
  if (!a->a_mn_major) rc = gb_make_tmap_2d_16b(&ta, a->A, a->a_rows, a->a_cols, a->lda, gb::BM, gb::BK, a->is_bf16);
  else rc = gb_make_tmap_2d_16b(&ta, a->A, a->a_rows, a->a_cols, a->lda, gb::BK, 64, a->is_bf16);
  if (rc) return rc - 100;
  if (!a->b_mn_major) rc = gb_make_tmap_2d_16b(&tb, a->B, a->b_rows, a->b_cols, a->ldb, bn, gb::BK, a->is_bf16);
  else rc = gb_make_tmap_2d_16b(&tb, a->B, a->b_rows, a->b_cols, a->ldb, gb::BK, 64, a->is_bf16);
  if (rc) return rc - 200;

  const int tiles_n = (a->N + bn - 1) / bn;
  int tiles_m = (a->M + gb::BM - 1) / gb::BM;
  int max_tiles = tiles_m * tiles_n * (a->mode == 2 ? p.groups : 1);

  const int ot = a->out_dtype;  // 0 fp16, 1 bf16, 2 fp32
  switch (a->epilogue) {
    case gb::EPI_STORE:
      if (p.tile_out) {   // expert-parallel combine: its own instantiation, so the plain store keeps its registers
        if (ot == 2) return -1;
        if (ot == 1) return dispatch_bn<gb::EPI_STORE_TILED, __nv_bfloat16, __nv_bfloat16>(bn, ta, tb, p, max_tiles, st);
        return dispatch_bn<gb::EPI_STORE_TILED, __half, __half>(bn, ta, tb, p, max_tiles, st);
      }
      if (ot == 2) return dispatch_bn<gb::EPI_STORE, float, __half>(bn, ta, tb, p, max_tiles, st);
      if (ot == 1) return dispatch_bn<gb::EPI_STORE, __nv_bfloat16, __nv_bfloat16>(bn, ta, tb, p, max_tiles, st);
      return dispatch_bn<gb::EPI_STORE, __half, __half>(bn, ta, tb, p, max_tiles, st);
    case gb::EPI_SWIGLU_FWD:
      if (ot == 1) return dispatch_bn<gb::EPI_SWIGLU_FWD, __nv_bfloat16, __nv_bfloat16>(bn == 256 ? 256 : 128, ta, tb, p, max_tiles, st);
      if (ot == 0) return dispatch_bn<gb::EPI_SWIGLU_FWD, __half, __half>(bn == 256 ? 256 : 128, ta, tb, p, max_tiles, st);
      return -1;
    case gb::EPI_SWIGLU_BWD:
      if (ot == 1) return dispatch_bn<gb::EPI_SWIGLU_BWD, __nv_bfloat16, __nv_bfloat16>(bn, ta, tb, p, max_tiles, st);
      if (ot == 0) return dispatch_bn<gb::EPI_SWIGLU_BWD, __half, __half>(bn, ta, tb, p, max_tiles, st);
      return -1;
  }
  return -1;
}
