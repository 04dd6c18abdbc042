// C ABI of the sm_100a kernel library (_gb200_cuda.so).  Every function takes raw device
// pointers plus the CUDA stream to launch on and returns 0 on success (negative = rejected
// arguments or a launch error).  Kernels that wait on barriers or peers report timeouts through a
// device-side status word instead of trapping; the host reads it after synchronising.
// "16-bit" tensors are fp16 when is_bf16 == 0 and bf16 otherwise.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ----------------------------------------------------------------------------- GEMM (gemm_sm100.cu)
// C[M,N] (+)= A[M,K] * B[N,K]^T with 16-bit operands and fp32 accumulation on tcgen05.
typedef struct gb_gemm_args {
  const void* A;            // stored matrix holding the A operand
  const void* B;            // stored matrix holding the B operand
  int M, N, K;              // logical problem; per group in grouped modes
  long long a_rows, a_cols, lda;   // stored A: [a_rows, a_cols], row stride lda (elements)
  long long b_rows, b_cols, ldb;   // stored B
  int a_mn_major;           // 0: stored [M,K] (K contiguous); 1: stored [K,M]
  int b_mn_major;           // 0: stored [N,K]; 1: stored [K,N]
  int is_bf16;              // operand type: 0 fp16, 1 bf16
  int out_dtype;            // 0 fp16, 1 bf16, 2 fp32
  int epilogue;             // 0 store (+ optional fp32 addend), 1 SwiGLU forward, 2 SwiGLU backward
  int block_n;              // 64 / 128 / 256 (0 = 128)
  int mode;                 // 0 dense, 1 grouped over rows (tile map), 2 grouped over the reduction dim
  const int* tile_expert;   // mode 1
  const int* num_m_tiles;   // mode 1 (device scalar)
  const int* seg_offsets;   // mode 2
  int groups;               // mode 2
  int b_group_rows;         // mode 1: stored-B rows per group
  void* out; int ldo; long long out_group_stride;
  const float* addend; int ld_add;   // out = acc + addend (fp32), may alias out when out is fp32
  void* aux_out; const void* aux_in; int ld_aux;
  int* status;              // device status word
  const long long* tile_out;  // mode 1 + plain store, no addend: device table with the address of output row 0 of every
                              // 128-row tile (overrides out); destinations may be another GPU's mapped memory
  int pair;                   // 1: two-CTA 256 x 256 tiles (gemm_pair_sm100.cu).  Needs a 16-byte aligned output whose
                              // row pitch is a multiple of 16 bytes, no tile_out, an addend only with fp32 output, and
                              // in mode 1 expert segments padded to GB_MOE_PAD rows; block_n is ignored
} gb_gemm_args;
int gb_gemm(const gb_gemm_args* args, cudaStream_t stream);
int gb_gemm_pair(const gb_gemm_args* args, cudaStream_t stream);   // what gb_gemm calls when args->pair != 0
// Expert segments of the sorted MoE buffers start at multiples of this many rows (two 128-row tiles: one pair tile).
#define GB_MOE_PAD 256

// ----------------------------------------------------------------------------- elementwise.cu
int gb_embed_fwd(const int* ids, const float* table, float* out, int n_tok, int d, int vocab, cudaStream_t st);
int gb_embed_bwd(const int* ids, const float* dx, float* dtable, int n_tok, int d, int vocab, cudaStream_t st);
int gb_embed_bwd_sorted(const int* sorted_ids, const long long* order, const float* dx, float* dtable, int n_tok,
                        int d, int vocab, cudaStream_t st);
int gb_rmsnorm_fwd(const float* x, const float* w, void* y16, float* rrms, int rows, int d, float eps, int is_bf16,
                   cudaStream_t st);
int gb_rmsnorm_bwd_blocks(int rows);
int gb_rmsnorm_bwd(const void* g16, const float* x, const float* w, const float* rrms, const float* dres, float* dx_out,
                   void* dx16, float* part, float* dw, int rows, int d, int is_bf16, cudaStream_t st);
int gb_qk_rope_blocks(int n_items);
int gb_qk_norm_rope_fwd(const void* qkv, int ld_in, void* out, int ld_out, const float* qw, const float* kw,
                        const float* cos_sin, const int* pos, int n_tok, int H, int KV, int hd, float eps, int rope_type,
                        int is_bf16, cudaStream_t st);
int gb_qk_norm_rope_bwd(const void* dout, int ld_dout, const void* qkv, int ld_in, void* dqkv, int ld_dqkv,
                        const float* qw, const float* kw, const float* cos_sin, const int* pos, float* part, float* dqw,
                        float* dkw, int n_tok, int H, int KV, int hd, float eps, int rope_type, int is_bf16,
                        cudaStream_t st);
int gb_cast_f32_to_16(const float* src, void* dst, long long n, int is_bf16, cudaStream_t st);
// out16[i] = sum over splits of part[s*n + i]: second stage of a split-K GEMM (gb_gemm mode 2 with equal K ranges)
int gb_splitk_reduce(const float* part, int splits, long long n, void* out16, int is_bf16, cudaStream_t st);
int gb_splitk_accumulate(const float* part, int splits, long long n, float* out, cudaStream_t st);

// ----------------------------------------------------------------------------- attention
typedef struct gb_attn_args {
  const void* q; long long ld_q;     // [B*T, ld] 16-bit, head h at column h*hd
  const void* k; long long ld_k;
  const void* v; long long ld_v;
  void* o; long long ld_o;
  float* lse;                        // [B*T, H]
  const int* seg;                    // [B*T] segment ids or NULL: contiguous runs per sequence (packed documents); rows with a
                                     // negative id see every earlier key while no non-negative id has come before them
  int B, T, H, KV, hd, window, is_bf16;
  float scale;
  const void* d_o; long long ld_do;  // backward only
  float* delta;                      // [B*T, H] scratch
  void* dq; long long ld_dq;
  void* dk; long long ld_dk;
  void* dv; long long ld_dv;
} gb_attn_args;
int gb_attn_fwd(const gb_attn_args* a, cudaStream_t st);
int gb_attn_bwd(const gb_attn_args* a, cudaStream_t st);
// Tensor-core (tcgen05) versions for head_dim 64 / 128.  Segment ids must form contiguous runs per sequence;
// lo_scratch: [B*T] int32 (needed when a->seg != NULL); status: device status word.
int gb_attn_seg_lo(const int* seg, int* lo, int B, int T, cudaStream_t st);
// lo_ready != 0: lo_scratch already holds gb_attn_seg_lo output (a->seg is then ignored)
int gb_attn_tc_fwd(const gb_attn_args* a, int* lo_scratch, int lo_ready, int* status, cudaStream_t st);
// dq_acc: fp32 scratch [B*T, H*hd] is not needed: dQ accumulates in tensor memory.  delta is computed inside.
int gb_attn_tc_bwd(const gb_attn_args* a, int* lo_scratch, int lo_ready, int* status, cudaStream_t st);

// ----------------------------------------------------------------------------- moe.cu
typedef struct gb_moe_args {
  int n_tok, d, ne, top_k, shared;   // shared: 1 = an always-on expert with index ne takes every token
  int is_bf16;
  // router forward
  const void* x16;                   // [n_tok, d] normalised activations (16-bit)
  const float* router_w;             // [ne, d] fp32
  const float* bias;                 // [ne] selection bias or NULL
  float jitter; unsigned long long jitter_seed; int use_jitter;
  float* probs;                      // [n_tok, ne]
  int* idx;                          // [n_tok, top_k]
  float* w;                          // [n_tok, top_k] combine weights
  int* block_hist;                   // [n_blocks, ne+1] scratch (per 256-token block expert counts)
  // grouping
  int* seg_offsets;                  // [ne+2] padded (128) row offsets per expert (shared expert last)
  int* tile_expert;                  // [max_tiles]
  int* num_tiles;                    // [1]
  int* block_base;                   // [n_blocks, ne+1] first row of each block inside each expert segment
  int* slot_pos;                     // [n_tok, top_k+shared] row of each (token, slot) in the sorted buffer
  float* counts;                     // [ne] routed-slot counts accumulated (+=) for balancing, or NULL
  void* x_perm;                      // [cap, d] 16-bit expert-sorted copy of x16 (pad rows zeroed)
  int cap;                           // rows of the sorted buffers
  // combine
  const void* y_perm;                // [cap, d] expert outputs (unweighted)
  const float* resid;                // [n_tok, d] fp32 residual input
  float* out;                        // [n_tok, d] fp32: resid + shared + sum_k w_k y_k
  // backward
  const float* dout;                 // [n_tok, d] fp32 gradient of `out`
  void* dy_perm;                     // [cap, d] 16-bit: w_k * dout rows in sorted order (pad rows zeroed)
  float* gdot;                       // [n_tok, top_k] dout . y_k
  const void* dx_perm;               // [cap, d] 16-bit gradient w.r.t. sorted inputs
  float aux_coef;                    // coefficient of the aux-loss gradient on mean probs (0 = off)
  float* f_frac;                     // [ne] routed-slot share of this micro-batch (aux loss), or NULL
  float* d_router_w;                 // [ne, d] fp32, accumulated
  void* dx16;                        // [n_tok, d] 16-bit gradient w.r.t. x16 (all paths summed)
  float* aux_m;                      // [ne] mean router probability per expert (aux loss), or NULL
  float* part;                       // scratch: router-logit gradients [n_tok, ne]
  float* aux_acc;                    // [1] += ne * sum_e aux_m[e] * f[e] of this call (needs aux_m), or NULL
  const unsigned long long* dyn_seed;// device copy of jitter_seed (overrides it; lets a captured graph change seeds)
  const float* dyn_aux_coef;         // device copy of aux_coef (overrides it)
  float* part2;                      // scratch [GB_ROUTER_WGRAD_CHUNKS, ne, d] for the router weight gradient, or NULL
  // A pass that concatenates several micro-batches keeps the reference's per-micro-batch definitions when seg_tokens is
  // the micro-batch size (a multiple of the routing block, see gb_moe_seg_ok): f_frac and aux_m are then
  // [segments, ne], the jitter hash counts tokens inside a segment, dyn_aux_coef holds one coefficient per segment and
  // seg_weight (device, [segments], may be NULL = 1) weights each segment's balance loss in aux_acc.  0 = one segment.
  int seg_tokens;
  const float* seg_weight;
  int* status;                       // device status word for kernels with bounded waits (tensor-core router), or NULL
} gb_moe_args;
int gb_moe_seg_ok(int n_tok, int seg_tokens);   // 1 when seg_tokens is usable for a pass of n_tok tokens
#define GB_ROUTER_WGRAD_CHUNKS 256
int gb_moe_num_blocks(int n_tok);
int gb_moe_capacity(int n_tok, int ne, int top_k, int shared);
int gb_moe_route(const gb_moe_args* a, cudaStream_t st);          // router + top-k + histograms
int gb_moe_group(const gb_moe_args* a, cudaStream_t st);          // offsets, tile map, positions, sorted copy
int gb_moe_combine(const gb_moe_args* a, cudaStream_t st);        // out = resid + sum w_k y_k (+ shared)
int gb_moe_combine_bwd(const gb_moe_args* a, cudaStream_t st);    // dy_perm, gdot
int gb_moe_router_bwd(const gb_moe_args* a, cudaStream_t st);     // dx16 (un-permute sum + router path), d_router_w

// ----------------------------------------------------------------------------- ce.cu
// logits: [rows, V] 16-bit (in place: overwritten with d(logits) * grad_scale when write_grad != 0).
// acc[0] += sum of losses (double), acc[1] += number of supervised rows (as double); z-loss z*logZ^2.
// row_loss: scratch of `rows` floats.
// grad_scale_dev (optional, device): overrides grad_scale, so a captured graph can follow the loss scaler.
int gb_softmax_ce(void* logits, long long ld, const int* targets, int rows, int V, float z_loss, float grad_scale,
                  const float* grad_scale_dev, int write_grad, float* row_loss, double* acc, int is_bf16,
                  cudaStream_t st);

// ----------------------------------------------------------------------------- optim.cu
typedef struct gb_opt_args {
  float* w; const float* g; float* m; float* v;   // flat fp32 buffers (v NULL for Lion)
  void* w16;                                      // 16-bit shadow of w (or NULL)
  long long n;
  int kind;                                       // 0 AdamW, 1 Lion
  float beta1, beta2, eps, wd;
  const float* hyper;                             // device: {lr, bc1, bc2} of this step
  const float* scale_dev;                         // device scalar: grad_scale * clip_scale (0 => skip step)
  int is_bf16;
} gb_opt_args;
int gb_optimizer_step(const gb_opt_args* a, cudaStream_t st);
// partial[block] = sum g^2 (double) over 65536-element chunks of a flat range
int gb_sqnorm_blocks(long long n);
int gb_sqnorm_partial(const float* g, long long n, double* partial, cudaStream_t st);
// out[0] = grad_scale * clip factor (0 when the norm is not finite), out[1] = gnorm;
// grad_scale is read from grad_scale_dev[0] when that pointer is not NULL
int gb_finish_norm(const double* partial, int n_partial, const float* grad_scale_dev, float grad_scale, float clip,
                   float* out, cudaStream_t st);
int gb_fill_f32(float* p, float v, long long n, cudaStream_t st);

// ----------------------------------------------------------------------------- muon.cu
// Elementwise parts of Muon over "class" buffers: all matrices of one shape stacked as [n * rows_per_mat, C] fp32,
// rows_per_mat a multiple of 256 (pad rows zero).  row_src[r] = offset of class row r in the flat parameter / gradient
// buffers, -1 for a pad row.  scale_dev[0] = grad_scale * clip factor of the step; 0 makes every kernel a no-op.
int gb_muon_blocks(long long rows);                       // entries of `partial` that gb_muon_momentum fills
int gb_muon_momentum(float* m, const float* g, const long long* row_src, long long rows, int C, float beta1,
                     const float* scale_dev, double* partial, cudaStream_t st);
// Y = m / |m|_F per matrix, Y16 = bf16(Y), T = 1.5 Y; skip_flag[mat] = 1 when the norm is unusable
int gb_muon_normalize(const float* m, float* Y, float* T, void* Y16, const double* partial, long long rows,
                      int rows_per_mat, int C, const float* scale_dev, int* skip_flag, cudaStream_t st);
int gb_muon_gram_cast(const float* A, void* B16, long long n, const float* scale_dev, cudaStream_t st);   // bf16(-0.5 A)
int gb_muon_refresh(float* Y, float* T, void* Y16, long long rows, int rows_per_mat, int C, const float* scale_dev,
                    const int* skip_flag, cudaStream_t st);
// w <- (w - lr Y)(1 - lr wd) through row_src, plus the 16-bit shadow (w16 may be NULL); lr_dev[0] = learning rate
int gb_muon_apply(float* w, void* w16, int is_bf16, const float* Y, const long long* row_src, long long rows, int C,
                  const float* lr_dev, float wd, const float* scale_dev, cudaStream_t st);

#ifdef __cplusplus
}
#endif
