// Expert parallelism over peer memory (ep.cu).
//
// Every rank routes its own tokens and leaves the rows grouped by expert (each group padded to 128 rows, pads zero)
// in a symmetric buffer, with the group offsets beside it.  The rank that owns expert e then
//   1. plans: reads every rank's offsets and lays the rows of its experts out as [expert][source rank] blocks,
//   2. pulls those blocks with peer loads (the dispatch half of the all-to-all),
//   3. runs the grouped tcgen05 GEMMs on them, and
//   4. lets the last GEMM's epilogue store each 128-row tile straight into the source rank's buffer (the combine
//      half of the all-to-all is part of the GEMM: gb_gemm's per-tile destination table).
// The reference replicates all experts and loops over them on one GPU (cuda/moe.cu:734-751); it has no expert
// parallelism.  Barriers between the phases are gb_sync_barrier on a control block of this subsystem.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GB_EP_MAX_DESC 160          // (experts per rank x ranks) + 1 copy descriptors at most
#define GB_EP_MAX_EXPERTS 128       // routed experts (global)

// Plan of one layer on one rank (device memory, written by gb_ep_plan, read by gb_ep_pull and the GEMM launches).
typedef struct gb_ep_plan_buffers {
  int* recv_seg;          // [ne1 + 1] padded row offsets of the received layout, by expert (non-owned experts: empty)
  int* tile_expert;       // [max_tiles] expert of each received 128-row tile
  int* num_tiles;         // [1]
  int* desc;              // [GB_EP_MAX_DESC][4] {source rank, source row, destination row, rows}
  int* num_desc;          // [1]
  long long* tile_out_a;  // [max_tiles] address, in the source rank's buffer A, of the rows tile j came from
  long long* tile_out_b;  // [max_tiles] same for buffer B
} gb_ep_plan_buffers;

typedef struct gb_ep_plan_args {
  int rank, world;
  int ne;                 // routed experts (global); owner of expert e = e / (ne / world)
  int has_shared;         // 1: group ne holds every local token for the shared expert (never leaves its rank)
  int max_rows;           // capacity of the received layout (multiple of 128); more rows = status ST_EP_OVERFLOW
  const int* const* peer_seg;   // [world] every rank's [ne1 + 1] offsets (symmetric memory)
  const long long* base_a;      // [world] byte address of every rank's buffer A (forward: expert outputs)
  const long long* base_b;      // [world] byte address of every rank's buffer B (backward: input gradients)
  long long row_bytes_a, row_bytes_b;
  gb_ep_plan_buffers out;
  int* status;
} gb_ep_plan_args;

int gb_ep_plan(const gb_ep_plan_args* a, cudaStream_t st);

// dst[desc.dst_row + i] = peer_src[desc.src][desc.src_row + i] for every descriptor; rows of `row_bytes` bytes
// (multiple of 16, both sides 16-byte aligned).
int gb_ep_pull(const void* const* peer_src, void* dst, long long row_bytes, const int* desc, const int* num_desc,
               int max_rows, cudaStream_t st);

#ifdef __cplusplus
}
#endif
