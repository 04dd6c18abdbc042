// Expert parallelism over peer memory: planning of the received layout and the dispatch pull (see gb_ep.h).
#include "gb_ep.h"
#include "gb_comm.h"
#include "sm100_common.cuh"

namespace gb {

// One block.  Thread 0 walks (own expert, source rank) in order and lays the blocks out back to back; the shared
// expert's rows (group `ne`) follow, taken from this rank only.  Then all threads fill the per-tile tables.
__global__ void __launch_bounds__(256) ep_plan_kernel(gb_ep_plan_args a) {
  __shared__ int s_desc[GB_EP_MAX_DESC][4];
  __shared__ int s_desc_expert[GB_EP_MAX_DESC];
  __shared__ int s_ndesc;
  __shared__ int s_seg[GB_MAX_RANKS][GB_EP_MAX_EXPERTS + 2];
  const int ne1 = a.ne + (a.has_shared ? 1 : 0);
  const int per = a.ne / a.world;
  // all offsets of all ranks at once: a peer load costs microseconds, so they must not be issued one after another
  for (int i = threadIdx.x; i < a.world * (ne1 + 1); i += blockDim.x) {
    const int s = i / (ne1 + 1), e = i - s * (ne1 + 1);
    s_seg[s][e] = __ldcg(a.peer_seg[s] + e);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int nd = 0, row = 0, bad = 0;
    for (int e = 0; e < ne1; ++e) {
      a.out.recv_seg[e] = row;
      const bool shared = e == a.ne;
      if (!shared && e / per != a.rank) continue;
      for (int s = 0; s < a.world; ++s) {
        if (shared && s != a.rank) continue;
        const int lo = s_seg[s][e], hi = s_seg[s][e + 1];
        const int n = hi - lo;
        if (n <= 0) continue;
        if ((n & 127) || (lo & 127) || nd >= GB_EP_MAX_DESC || row + n > a.max_rows) { bad = 1; break; }
        s_desc[nd][0] = s; s_desc[nd][1] = lo; s_desc[nd][2] = row; s_desc[nd][3] = n;
        s_desc_expert[nd] = e;
        ++nd;
        row += n;
      }
      if (bad) break;
    }
    if (bad) {              // leave an empty, consistent plan behind and report
      nd = 0; row = 0;
      for (int e = 0; e <= ne1; ++e) a.out.recv_seg[e] = 0;
      atomicCAS(a.status, 0, ST_EP_OVERFLOW);
    } else {
      a.out.recv_seg[ne1] = row;
    }
    s_ndesc = nd;
    *a.out.num_desc = nd;
    *a.out.num_tiles = row >> 7;
  }
  __syncthreads();
  const int nd = s_ndesc;
  for (int i = threadIdx.x; i < nd * 4; i += blockDim.x) a.out.desc[i] = s_desc[i >> 2][i & 3];
  for (int i = 0; i < nd; ++i) {
    const int src = s_desc[i][0], src_row = s_desc[i][1], dst_row = s_desc[i][2], n = s_desc[i][3];
    const int t0 = dst_row >> 7, nt = n >> 7;
    for (int j = threadIdx.x; j < nt; j += blockDim.x) {
      a.out.tile_expert[t0 + j] = s_desc_expert[i];
      const long long r = (long long)src_row + 128LL * j;
      a.out.tile_out_a[t0 + j] = a.base_a[src] + r * a.row_bytes_a;
      a.out.tile_out_b[t0 + j] = a.base_b[src] + r * a.row_bytes_b;
    }
  }
}

// Each warp moves whole rows; four rows are in flight per warp so that the link latency is covered.
__global__ void __launch_bounds__(256) ep_pull_kernel(const void* const* __restrict__ peer_src, void* __restrict__ dst,
                                                      long long row_bytes, const int* __restrict__ desc,
                                                      const int* __restrict__ num_desc) {
  __shared__ int s_desc[GB_EP_MAX_DESC][4];
  const int nd = min(*num_desc, GB_EP_MAX_DESC);
  for (int i = threadIdx.x; i < nd * 4; i += blockDim.x) s_desc[i >> 2][i & 3] = desc[i];
  __syncthreads();
  if (nd == 0) return;
  const int total = s_desc[nd - 1][2] + s_desc[nd - 1][3];
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int vec_per_row = int(row_bytes >> 4);
  constexpr int R = 4;
  for (int r0 = warp * R; r0 < total; r0 += nwarps * R) {
    const uint4* src[R];
    uint4* out[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int r = r0 + k;
      src[k] = nullptr; out[k] = nullptr;
      if (r < total) {
        int i = 0;
        while (i + 1 < nd && s_desc[i + 1][2] <= r) ++i;
        const char* base = static_cast<const char*>(peer_src[s_desc[i][0]]);
        src[k] = reinterpret_cast<const uint4*>(base + (long long)(s_desc[i][1] + (r - s_desc[i][2])) * row_bytes);
        out[k] = reinterpret_cast<uint4*>(static_cast<char*>(dst) + (long long)r * row_bytes);
      }
    }
    for (int v = lane; v < vec_per_row; v += 32) {
      uint4 q[R];
#pragma unroll
      for (int k = 0; k < R; ++k)
        if (src[k]) q[k] = __ldcg(src[k] + v);      // L2 only: the same peer addresses carry new rows every layer
#pragma unroll
      for (int k = 0; k < R; ++k)
        if (src[k]) out[k][v] = q[k];
    }
  }
}

}  // namespace gb

extern "C" int gb_ep_plan(const gb_ep_plan_args* a, cudaStream_t st) {
  if (!a || a->world < 1 || a->world > GB_MAX_RANKS || a->rank < 0 || a->rank >= a->world) return -1;
  if (a->ne < a->world || a->ne % a->world || a->ne > GB_EP_MAX_EXPERTS) return -2;
  if ((a->ne / a->world) * a->world + 1 > GB_EP_MAX_DESC) return -2;
  if (a->max_rows <= 0 || (a->max_rows & 127)) return -2;
  if (!a->peer_seg || !a->base_a || !a->base_b || !a->status || !a->out.recv_seg || !a->out.tile_expert ||
      !a->out.num_tiles || !a->out.desc || !a->out.num_desc || !a->out.tile_out_a || !a->out.tile_out_b)
    return -1;
  gb::ep_plan_kernel<<<1, 256, 0, st>>>(*a);
  return gb_launch_rc();
}

extern "C" int gb_ep_pull(const void* const* peer_src, void* dst, long long row_bytes, const int* desc,
                          const int* num_desc, int max_rows, cudaStream_t st) {
  if (!peer_src || !dst || !desc || !num_desc || row_bytes <= 0 || (row_bytes & 15) || max_rows <= 0) return -1;
  if (reinterpret_cast<uintptr_t>(dst) & 15) return -2;
  int blocks = (max_rows + 31) / 32;            // 8 warps x 4 rows per block and trip
  if (blocks > 592) blocks = 592;
  if (blocks < 1) blocks = 1;
  gb::ep_pull_kernel<<<blocks, 256, 0, st>>>(peer_src, dst, row_bytes, desc, num_desc);
  return gb_launch_rc();
}
