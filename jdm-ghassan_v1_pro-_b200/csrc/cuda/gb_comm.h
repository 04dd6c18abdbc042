// Peer-memory collectives fused with the optimizer (comm.cu).  All buffers named "peer" are arrays of `world`
// device pointers, one per rank, obtained from symmetric memory; entry r of a rank's own array is its local buffer.
// Peers are read with plain loads and written with plain stores; no TMA, no multicast.
//
// One gradient exchange = gb_sync_barrier, gb_sync_reduce, gb_sync_update (local_only), gb_sync_barrier, gb_sync_gather
// of the 16-bit weights (and of the fp32 part that kernels read in fp32) on the same stream of every rank; the barrier
// that opens the next exchange keeps a rank from overwriting its shard while a peer still reads it.
// It replaces the reference's per-parameter ncclAllReduce + host-side norm + per-tensor optimizer launches
// (training/trainer.cpp:1835-1876, 1476-1536) by: reduce-scatter through peer loads in rank order, Sum g^2 of the owned
// shard, a mailbox exchange of {Sum g^2, token count}, on each owner the unscale / clip / inf-check / optimizer update
// of its shard, and an all-gather of the new 16-bit weights by peer loads.  With kind = 2 (Muon) the update is left
// out and the ranks gather the reduced fp32 gradient instead.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Control block of one rank (symmetric memory, GB_CTL_WORDS 32-bit words, zero-initialised once):
//   words [0, 64)        barrier flags, slot = sender rank
//   words [64, 128)      mailbox flags, slot = sender rank
//   bytes [1024, 2048)   mailbox payload: 2 doubles per sender {sum of squares of its shard, its token count}
#define GB_CTL_WORDS 1024
#define GB_MAX_RANKS 16
#define GB_SYNC_BLOCKS 592          // grid of the reduce kernel: fixed, so the partial-sum tree never changes

typedef struct gb_sync_args {
  int rank, world;
  long long shard;                  // elements owned per rank (multiple of 64); rank r owns [r*shard, (r+1)*shard)
  long long total;                  // elements that exist (owned ranges are clipped to it)
  long long decay_start;            // elements at or beyond this index take weight decay
  long long f32_end;                // elements below this index are consumed in fp32: new values also go to peers' masters
  float* const* peer_grad;          // fp32 gradients of every rank (this rank's shard is reduced in place)
  float* const* peer_master;        // fp32 master weights of every rank
  void* const* peer_w16;            // 16-bit shadows of every rank
  unsigned int* const* peer_ctl;    // control blocks
  float* m; float* v;               // local moments, indexed like the flat buffers (only the own shard is touched)
  int kind;                         // 0 AdamW, 1 Lion, 2 none: gb_sync_update only folds the norm and publishes `out`
  float beta1, beta2, eps, wd;
  const float* hyper;               // device {lr, bc1, bc2}
  float loss_scale, clip;
  double ntok_local;                // supervised tokens of this rank in this step
  unsigned int epoch;               // strictly increasing per exchange, same on every rank
  double* partial;                  // local scratch, GB_SYNC_BLOCKS doubles
  unsigned int* ticket;             // local scratch, 1 word, zero before the first call
  float* out;                       // local [4]: grad_scale*clip (0 = skipped), gnorm, global token count, unused
  int* status;                      // device status word (ST_TIMEOUT_PEER on a wait that ran out)
  int is_bf16;
  int no_wait;                      // 1: all ranks' kernels run back to back on one device (tests): never spin
  int local_only;                   // 1: gb_sync_update writes the new values of the own shard locally only; the ranks
                                    //    then fetch each other's shards with gb_sync_gather (peer loads ran 1.8x faster
                                    //    than peer stores on NVSwitch here)
  // NVSwitch multicast addresses of the same three buffers (NULL: not used).  With mc_grad the reduce-scatter is one
  // multimem.ld_reduce per 16 bytes (the switch adds the ranks' values); with mc_w16 / mc_master the new values of
  // the own shard go to every rank with one multimem.st each and no gather follows.
  float* mc_grad; float* mc_master; void* mc_w16;
} gb_sync_args;

// All ranks have reached this point, and their earlier writes are visible to peer loads issued after it.
int gb_sync_barrier(unsigned int* const* peer_ctl, int rank, int world, unsigned int epoch, int* status, cudaStream_t st);
// The same, with the epoch read from and advanced in `counter` (device memory, starts at 0, one per control block and
// rank): usable inside a captured CUDA graph.  `spin_limit` polls of about 50 ns bound the wait (0 = about 2 s).
int gb_sync_barrier_auto(unsigned int* const* peer_ctl, int rank, int world, unsigned int* counter, long long spin_limit,
                         int* status, cudaStream_t st);
int gb_sync_reduce(const gb_sync_args* a, cudaStream_t st);
int gb_sync_update(const gb_sync_args* a, cudaStream_t st);
// All-gather by peer loads of a flat buffer that every rank holds a copy of: bytes [r*shard_bytes, (r+1)*shard_bytes)
// below limit_bytes are copied from rank r's buffer (peer[r]) into `local`, for every r != rank.  Call between two
// barriers: after the owners have written, and before anyone overwrites its shard again.
int gb_sync_gather(const void* const* peer, void* local, long long shard_bytes, long long limit_bytes, int rank, int world,
                   cudaStream_t st);
// dst[i] = sum over ranks (in rank order) of peer_src[r][i]: replicated small tensors (routing counts).
int gb_sync_small_allreduce(const float* const* peer_src, float* dst, int n, int world, cudaStream_t st);

#ifdef __cplusplus
}
#endif
