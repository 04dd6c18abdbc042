// Gradient exchange over NVSwitch peer memory fused with the optimizer: see gb_comm.h for the protocol.
//
// Reproducibility: every element is reduced by exactly one rank, which adds the ranks' contributions in rank order;
// the sum of squares uses a fixed grid and a fixed tree; every rank folds the ranks' partial norms in rank order.
// The result therefore does not depend on timing, and all ranks compute the same clip factor and skip decision
// without a further exchange.
//
// Waiting: a rank waits for a peer in two places (the barrier and the mailbox).  Both spins are bounded; when the
// bound is hit the kernel records ST_TIMEOUT_PEER in the status word and returns without touching weights.
#include "sm100_common.cuh"
#include "gb_comm.h"

namespace gb {

constexpr int CTL_BARRIER = 0;       // word offset of the barrier flags
constexpr int CTL_MAILFLAG = 64;     // word offset of the mailbox flags
constexpr int CTL_MAIL_BYTES = 1024; // byte offset of the mailbox payload
constexpr long long SPIN_LIMIT = 40LL * 1000 * 1000;   // x ~50 ns: about two seconds

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// true when the flag reached `epoch` before the spin limit
__device__ __forceinline__ bool wait_flag(const unsigned int* flag, unsigned int epoch, bool no_wait) {
  for (long long it = 0; it < SPIN_LIMIT; ++it) {
    if ((int)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if (no_wait) return false;
    __nanosleep(40);
  }
  return false;
}

__global__ void sync_barrier_kernel(unsigned int* const* __restrict__ peer_ctl, int rank, int world, unsigned int epoch,
                                    int* __restrict__ status) {
  const int p = threadIdx.x;
  if (p < world) {
    __threadfence_system();
    st_release_sys(peer_ctl[p] + CTL_BARRIER + rank, epoch);
    if (!wait_flag(peer_ctl[rank] + CTL_BARRIER + p, epoch, false)) atomicExch(status, ST_TIMEOUT_PEER);
  }
  __syncthreads();
}

// Same barrier with the epoch kept in device memory: a CUDA graph that contains it can be replayed.
__global__ void sync_barrier_auto_kernel(unsigned int* const* __restrict__ peer_ctl, int rank, int world,
                                         unsigned int* __restrict__ counter, long long spin_limit,
                                         int* __restrict__ status) {
  __shared__ unsigned int s_epoch;
  if (threadIdx.x == 0) s_epoch = ++(*counter);
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const int p = threadIdx.x;
  if (p < world) {
    __threadfence_system();
    st_release_sys(peer_ctl[p] + CTL_BARRIER + rank, epoch);
    const unsigned int* flag = peer_ctl[rank] + CTL_BARRIER + p;
    bool ok = false;
    for (long long it = 0; it < spin_limit; ++it) {
      if ((int)(ld_acquire_sys(flag) - epoch) >= 0) { ok = true; break; }
      __nanosleep(40);
    }
    if (!ok) atomicExch(status, ST_TIMEOUT_PEER);
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------- NVSwitch multicast
// One load that the switch answers with the sum over all ranks' copies, and one store that the switch delivers to all
// of them.  Only with a multicast address (the symmetric buffer bound to a multicast object); never in a test where a
// rank leaves.
__device__ __forceinline__ float4 mc_ld_reduce_f32x4(const float* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_16B(void* p, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// ---------------------------------------------------------------------------------------------- reduce-scatter
template <int W>
__device__ __forceinline__ float4 sum_peers(float* const* __restrict__ g, long long i, int world) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const int n = W > 0 ? W : world;
#pragma unroll
  for (int r = 0; r < n; ++r) {   // rank order: the sum does not depend on who computes it or when
    const float4 x = *reinterpret_cast<const float4*>(g[r] + i);
    acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
  }
  return acc;
}

template <int W>
__global__ void __launch_bounds__(256) sync_reduce_kernel(gb_sync_args a) {
  __shared__ double red[256];
  __shared__ float* gp[GB_MAX_RANKS];
  __shared__ bool last;
  if (threadIdx.x < a.world) gp[threadIdx.x] = a.peer_grad[threadIdx.x];
  __syncthreads();
  const long long lo = (long long)a.rank * a.shard;
  const long long hi = min(a.total, lo + a.shard);
  float* mine = gp[a.rank];
  double sq = 0.0;
  // U independent 16-byte loads per peer and thread in flight: NVLink latency is several microseconds
  constexpr int U = W == 0 ? 1 : (W >= 8 ? 2 : 4);
  const long long tile = 256LL * 4 * U;
  const long long stride = (long long)gridDim.x * tile;
  for (long long base = lo + (long long)blockIdx.x * tile; base < hi; base += stride) {
    float4 s[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = base + ((long long)u * 256 + threadIdx.x) * 4;
      s[u] = i >= hi ? make_float4(0.f, 0.f, 0.f, 0.f)
                     : (a.mc_grad ? mc_ld_reduce_f32x4(a.mc_grad + i) : sum_peers<W>(gp, i, a.world));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = base + ((long long)u * 256 + threadIdx.x) * 4;
      if (i < hi) {
        *reinterpret_cast<float4*>(mine + i) = s[u];   // own shard of the own buffer: no peer reads this range
        sq += (double)s[u].x * s[u].x + (double)s[u].y * s[u].y + (double)s[u].z * s[u].z + (double)s[u].w * s[u].w;
      }
    }
  }
  red[threadIdx.x] = sq;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    a.partial[blockIdx.x] = red[0];
    __threadfence();
    last = atomicAdd(a.ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  double acc = 0.0;
  for (int i = threadIdx.x; i < (int)gridDim.x; i += 256) acc += *((volatile double*)&a.partial[i]);
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  // post {sum of squares of my shard, my token count} into every rank's mailbox (my own included)
  if (threadIdx.x < a.world) {
    unsigned int* ctl = a.peer_ctl[threadIdx.x];
    volatile double* mail = reinterpret_cast<volatile double*>(reinterpret_cast<char*>(ctl) + CTL_MAIL_BYTES) + 2 * a.rank;
    mail[0] = red[0];
    mail[1] = a.ntok_local;
    __threadfence_system();
    st_release_sys(ctl + CTL_MAILFLAG + a.rank, a.epoch);
  }
  if (threadIdx.x == 0) *a.ticket = 0;
}

// ---------------------------------------------------------------------------------------------- update + all-gather
template <typename T, int KIND>
__global__ void __launch_bounds__(256) sync_update_kernel(gb_sync_args a) {
  __shared__ float s_scale;
  __shared__ int s_ok;
  __shared__ float* mp[GB_MAX_RANKS];
  __shared__ T* wp[GB_MAX_RANKS];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < a.world) {
    mp[threadIdx.x] = a.peer_master[threadIdx.x];
    wp[threadIdx.x] = reinterpret_cast<T*>(a.peer_w16[threadIdx.x]);
    if (!wait_flag(a.peer_ctl[a.rank] + CTL_MAILFLAG + threadIdx.x, a.epoch, a.no_wait != 0)) s_ok = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float scale = 0.f, gnorm = 0.f;
    double ntok = 0.0;
    if (s_ok) {
      const volatile double* mail = reinterpret_cast<const volatile double*>(
          reinterpret_cast<const char*>(a.peer_ctl[a.rank]) + CTL_MAIL_BYTES);
      double sq = 0.0;
      for (int r = 0; r < a.world; ++r) {   // rank order on every rank: identical clip factor everywhere
        sq += mail[2 * r];
        ntok += mail[2 * r + 1];
      }
      if (ntok > 0.0) {
        const float gs = 1.0f / ((float)ntok * a.loss_scale);
        const double gn = sqrt(sq) * (double)gs;
        float clip_scale = 1.0f;
        if (a.clip > 0.0f && gn > (double)a.clip) clip_scale = (float)((double)a.clip / (gn + 1e-6));
        scale = isfinite(gn) ? gs * clip_scale : 0.f;
        gnorm = (float)gn;
      }
    } else {
      atomicExch(a.status, ST_TIMEOUT_PEER);
    }
    s_scale = scale;
    if (blockIdx.x == 0) {
      a.out[0] = scale;
      a.out[1] = gnorm;
      a.out[2] = (float)ntok;
      a.out[3] = s_ok ? 0.f : 1.f;
    }
  }
  __syncthreads();
  const float scale = s_scale;
  if (scale == 0.f) return;   // skipped step (overflow, nothing supervised, or a peer that never answered)
  if (KIND == 2) return;      // norm and skip decision only: the optimizer runs elsewhere (Muon)
  const float lr = a.hyper[0], bc1 = a.hyper[1], bc2 = a.hyper[2];
  const long long lo = (long long)a.rank * a.shard;
  const long long hi = min(a.total, lo + a.shard);
  float* w = mp[a.rank];
  const float* g = a.peer_grad[a.rank];
  const long long stride = (long long)gridDim.x * 256 * 8;
  for (long long i = lo + ((long long)blockIdx.x * 256 + threadIdx.x) * 8; i < hi; i += stride) {
    float wv[8], gv[8], mv[8], vv[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 x = *reinterpret_cast<const float4*>(w + i + 4 * h), y = *reinterpret_cast<const float4*>(g + i + 4 * h),
                   z = *reinterpret_cast<const float4*>(a.m + i + 4 * h);
      wv[4 * h] = x.x; wv[4 * h + 1] = x.y; wv[4 * h + 2] = x.z; wv[4 * h + 3] = x.w;
      gv[4 * h] = y.x; gv[4 * h + 1] = y.y; gv[4 * h + 2] = y.z; gv[4 * h + 3] = y.w;
      mv[4 * h] = z.x; mv[4 * h + 1] = z.y; mv[4 * h + 2] = z.z; mv[4 * h + 3] = z.w;
      if (KIND == 0) {
        const float4 q = *reinterpret_cast<const float4*>(a.v + i + 4 * h);
        vv[4 * h] = q.x; vv[4 * h + 1] = q.y; vv[4 * h + 2] = q.z; vv[4 * h + 3] = q.w;
      }
    }
    const float wd = i >= a.decay_start ? a.wd : 0.f;   // segments are 64-aligned: 8 neighbours share the region
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gi = gv[k] * scale;
      if (KIND == 0) {
        const float mi = a.beta1 * mv[k] + (1.0f - a.beta1) * gi;
        const float vi = a.beta2 * vv[k] + (1.0f - a.beta2) * gi * gi;
        mv[k] = mi;
        vv[k] = vi;
        float upd = (mi / bc1) / (sqrtf(vi / bc2) + a.eps);
        if (wd != 0.0f) upd += wd * wv[k];
        wv[k] -= lr * upd;
      } else {
        const float c = a.beta1 * mv[k] + (1.0f - a.beta1) * gi;
        float upd = (c > 0.0f) ? 1.0f : ((c < 0.0f) ? -1.0f : 0.0f);
        if (wd != 0.0f) upd += wd * wv[k];
        wv[k] -= lr * upd;
        mv[k] = a.beta2 * mv[k] + (1.0f - a.beta2) * gi;
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      *reinterpret_cast<float4*>(a.m + i + 4 * h) = make_float4(mv[4 * h], mv[4 * h + 1], mv[4 * h + 2], mv[4 * h + 3]);
      if (KIND == 0)
        *reinterpret_cast<float4*>(a.v + i + 4 * h) = make_float4(vv[4 * h], vv[4 * h + 1], vv[4 * h + 2], vv[4 * h + 3]);
    }
    uint4 q16;
    q16.x = Cvt<T>::pack2(wv[0], wv[1]);
    q16.y = Cvt<T>::pack2(wv[2], wv[3]);
    q16.z = Cvt<T>::pack2(wv[4], wv[5]);
    q16.w = Cvt<T>::pack2(wv[6], wv[7]);
    if (a.mc_w16) {                       // one store per 16 bytes, delivered to every rank (this one included)
      mc_st_16B(reinterpret_cast<T*>(a.mc_w16) + i, make_float4(__uint_as_float(q16.x), __uint_as_float(q16.y),
                                                                   __uint_as_float(q16.z), __uint_as_float(q16.w)));
      if (i < a.f32_end && a.mc_master) {
        mc_st_16B(a.mc_master + i, make_float4(wv[0], wv[1], wv[2], wv[3]));
        mc_st_16B(a.mc_master + i + 4, make_float4(wv[4], wv[5], wv[6], wv[7]));
      } else {
        *reinterpret_cast<float4*>(w + i) = make_float4(wv[0], wv[1], wv[2], wv[3]);
        *reinterpret_cast<float4*>(w + i + 4) = make_float4(wv[4], wv[5], wv[6], wv[7]);
      }
      continue;
    }
    if (a.local_only) {                   // peers fetch the new values themselves afterwards (gb_sync_gather)
      *reinterpret_cast<uint4*>(wp[a.rank] + i) = q16;
      *reinterpret_cast<float4*>(w + i) = make_float4(wv[0], wv[1], wv[2], wv[3]);
      *reinterpret_cast<float4*>(w + i + 4) = make_float4(wv[4], wv[5], wv[6], wv[7]);
      continue;
    }
    const bool also_f32 = i < a.f32_end;
    for (int r = 0; r < a.world; ++r) {   // all-gather: the new values go straight into every rank's buffers
      *reinterpret_cast<uint4*>(wp[r] + i) = q16;
      if (also_f32 || r == a.rank) {
        *reinterpret_cast<float4*>(mp[r] + i) = make_float4(wv[0], wv[1], wv[2], wv[3]);
        *reinterpret_cast<float4*>(mp[r] + i + 4) = make_float4(wv[4], wv[5], wv[6], wv[7]);
      }
    }
  }
}

// All-gather by peer loads: every rank copies the other ranks' shards of a flat buffer into its own copy.  Bytes
// [r * shard_bytes, (r + 1) * shard_bytes) clipped to limit_bytes come from rank r.  A thread keeps U 16-byte loads in
// flight; consecutive blocks take consecutive pieces of one peer's shard, and the peer index is the outer loop, rotated
// by the rank so that at any moment the ranks read from different peers.
template <int U>
__global__ void __launch_bounds__(256) sync_gather_kernel(const unsigned char* const* __restrict__ peer,
                                                          unsigned char* __restrict__ local, long long shard_bytes,
                                                          long long limit_bytes, int rank, int world) {
  const long long tile = 256LL * 16 * U;
  for (int k = 1; k < world; ++k) {
    const int r = (rank + k) % world;
    const long long lo = (long long)r * shard_bytes;
    const long long hi = min(limit_bytes, lo + shard_bytes);
    const unsigned char* src = peer[r];
    for (long long base = lo + (long long)blockIdx.x * tile; base < hi; base += (long long)gridDim.x * tile) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = base + ((long long)u * 256 + threadIdx.x) * 16;
        if (i < hi) v[u] = *reinterpret_cast<const uint4*>(src + i);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = base + ((long long)u * 256 + threadIdx.x) * 16;
        if (i < hi) *reinterpret_cast<uint4*>(local + i) = v[u];
      }
    }
  }
}

__global__ void sync_small_allreduce_kernel(const float* const* __restrict__ src, float* __restrict__ dst, int n, int world) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0.f;
  for (int r = 0; r < world; ++r) acc += src[r][i];
  dst[i] = acc;
}

}  // namespace gb

using namespace gb;

extern "C" int gb_sync_barrier(unsigned int* const* peer_ctl, int rank, int world, unsigned int epoch, int* status,
                               cudaStream_t st) {
  if (!peer_ctl || !status || world < 1 || world > GB_MAX_RANKS || rank < 0 || rank >= world) return -1;
  sync_barrier_kernel<<<1, 32, 0, st>>>(peer_ctl, rank, world, epoch, status);
  return gb_launch_rc();
}

extern "C" int gb_sync_barrier_auto(unsigned int* const* peer_ctl, int rank, int world, unsigned int* counter,
                                    long long spin_limit, int* status, cudaStream_t st) {
  if (!peer_ctl || !status || !counter || world < 1 || world > GB_MAX_RANKS || rank < 0 || rank >= world) return -1;
  if (spin_limit <= 0) spin_limit = SPIN_LIMIT;
  sync_barrier_auto_kernel<<<1, 32, 0, st>>>(peer_ctl, rank, world, counter, spin_limit, status);
  return gb_launch_rc();
}

static int check_sync_args(const gb_sync_args* a) {
  if (!a || a->world < 1 || a->world > GB_MAX_RANKS || a->rank < 0 || a->rank >= a->world) return -1;
  if (!a->peer_grad || !a->peer_master || !a->peer_w16 || !a->peer_ctl || !a->partial || !a->ticket || !a->out ||
      !a->status)
    return -1;
  if (a->kind != 2 && (!a->m || !a->hyper)) return -1;
  if (a->kind == 0 && !a->v) return -1;
  if (a->shard <= 0 || a->shard % 64 || a->total % 8 || a->decay_start % 8 || a->f32_end % 8) return -2;
  return 0;
}

extern "C" int gb_sync_reduce(const gb_sync_args* a, cudaStream_t st) {
  if (int rc = check_sync_args(a)) return rc;
  switch (a->world) {
    case 1: sync_reduce_kernel<1><<<GB_SYNC_BLOCKS, 256, 0, st>>>(*a); break;
    case 2: sync_reduce_kernel<2><<<GB_SYNC_BLOCKS, 256, 0, st>>>(*a); break;
    case 4: sync_reduce_kernel<4><<<GB_SYNC_BLOCKS, 256, 0, st>>>(*a); break;
    case 8: sync_reduce_kernel<8><<<GB_SYNC_BLOCKS, 256, 0, st>>>(*a); break;
    default: sync_reduce_kernel<0><<<GB_SYNC_BLOCKS, 256, 0, st>>>(*a); break;
  }
  return gb_launch_rc();
}

extern "C" int gb_sync_update(const gb_sync_args* a, cudaStream_t st) {
  if (int rc = check_sync_args(a)) return rc;
  const int blocks = 148 * 4;
  if (a->kind == 2) {       // wait for the mailboxes, fold the norm, publish {scale, gnorm, tokens}: no update
    sync_update_kernel<__half, 2><<<1, 256, 0, st>>>(*a);
    return gb_launch_rc();
  }
  if (a->is_bf16) {
    if (a->kind == 0) sync_update_kernel<__nv_bfloat16, 0><<<blocks, 256, 0, st>>>(*a);
    else sync_update_kernel<__nv_bfloat16, 1><<<blocks, 256, 0, st>>>(*a);
  } else {
    if (a->kind == 0) sync_update_kernel<__half, 0><<<blocks, 256, 0, st>>>(*a);
    else sync_update_kernel<__half, 1><<<blocks, 256, 0, st>>>(*a);
  }
  return gb_launch_rc();
}

extern "C" int gb_sync_gather(const void* const* peer, void* local, long long shard_bytes, long long limit_bytes, int rank,
                              int world, cudaStream_t st) {
  if (!peer || !local || world < 1 || world > GB_MAX_RANKS || rank < 0 || rank >= world) return -1;
  if (shard_bytes <= 0 || (shard_bytes & 15) || (limit_bytes & 15) || (reinterpret_cast<uintptr_t>(local) & 15)) return -2;
  if (world == 1 || limit_bytes <= 0) return 0;
  sync_gather_kernel<4><<<GB_SYNC_BLOCKS, 256, 0, st>>>(reinterpret_cast<const unsigned char* const*>(peer),
                                                        reinterpret_cast<unsigned char*>(local), shard_bytes, limit_bytes,
                                                        rank, world);
  return gb_launch_rc();
}

extern "C" int gb_sync_small_allreduce(const float* const* peer_src, float* dst, int n, int world, cudaStream_t st) {
  if (!peer_src || !dst || n < 0 || world < 1 || world > GB_MAX_RANKS) return -1;
  if (n == 0) return 0;
  sync_small_allreduce_kernel<<<(n + 255) / 256, 256, 0, st>>>(peer_src, dst, n, world);
  return gb_launch_rc();
}
