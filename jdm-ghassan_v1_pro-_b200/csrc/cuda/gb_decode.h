// Decode-time kernels: dequant-fused GEMV family, KV ring cache append, split-KV decode attention, device sampler.
// One decode step of the whole model is a fixed kernel sequence with every varying quantity (positions, cache
// lengths, selected experts, sampled tokens) in device memory, so it replays as one CUDA graph with no host
// round trip per token.  The reference's decode path (inference/generator.cpp, cuda/attention.cu:724-870,
// cuda/kernels.cu:876-1019) copies the token id to the device, launches ~15 kernels per layer with fp32
// activations and reads logits or candidates back every token.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Weight row formats: each of the N rows of a [N, K] matrix is stored on its own, blocks along K.
enum {
  GB_W_F16 = 0,        // 2 B / value
  GB_W_BF16 = 1,
  GB_W_GGML_Q8_0 = 2,  // 32 values: f16 scale + 32 x i8                       (34 B)   GGUF type 8
  GB_W_Q4_0 = 3,       // 32 values: f16 scale + 16 B, byte i = code[2i+1]<<4 | code[2i], v = (code-8)*s   (18 B)
  GB_W_Q8_64 = 4,      // 64 values: f32 scale + 64 x i8                       (68 B)   internal Q8_0
  GB_W_Q4_1 = 5        // 32 values: f16 scale, f16 min + 16 B, v = code*s + min (20 B)
};
long long gb_wfmt_row_bytes(int fmt, int K);   // -1 when K does not fit the block size

// out[b, n] = sum_k W[n, k] * x[b, k] (+ addend[b, n]);  x: [B, K] 16-bit, B <= 32;  out 16-bit or fp32.
int gb_gemv(const void* W, int fmt, int N, int K, const void* x16, int ldx, int B, void* out, int ldo, int out_f32,
            const float* addend, int ld_add, int is_bf16, cudaStream_t st);

// Mixture-of-experts decode.  slots = top_k (+1 when shared != 0: the shared expert has index ne and weight 1).
// act[b, slot, j] = silu(Wg_e[j,:] . x_b) * (Wu_e[j,:] . x_b),  e = idx[b, slot]
int gb_gemv_expert_swiglu(const void* Wg, const void* Wu, int fmt, int ne, int E, int d, const void* x16, int B,
                          const int* idx, int top_k, int shared, void* act16, int is_bf16, cudaStream_t st);
// out[b, :] = resid[b, :] + sum_slot w[b, slot] * (Wd_e . act[b, slot, :])
int gb_gemv_expert_down(const void* Wd, int fmt, int ne, int d, int E, const void* act16, int B, const int* idx,
                        const float* w, int top_k, int shared, const float* resid, float* out, int is_bf16,
                        cudaStream_t st);

// Router for B tokens (no jitter, no statistics): idx[b, k] experts, w[b, k] renormalised probabilities; `bias`
// (optional) is added to the probabilities for the selection only; ties go to the lowest index.
int gb_decode_route(const void* x16, const float* router_w, const float* bias, int B, int d, int ne, int top_k,
                    int* idx, float* w, int is_bf16, cudaStream_t st);

// Per-sequence decode state (device, one per batch row).
typedef struct gb_seq_state {
  int abs_pos;      // tokens seen so far = RoPE position of the next token
  int cache_len;    // slots in use (<= cap)
  int ring_start;   // next slot to overwrite, relative to `pinned`, once the cache is full
  int done;         // set by the sampler when a stop token was drawn
} gb_seq_state;

// Store the new token's K (after RoPE) and V: cache[b, slot, :] with slot = cache_len while there is room, else
// pinned + ring_start (the first `pinned` tokens are never evicted).  slot_pos[b, slot] = abs_pos.  Does not advance.
int gb_kv_append(const void* k16, long long ld_k, const void* v16, long long ld_v, void* cacheK, void* cacheV,
                 int* slot_pos, const gb_seq_state* state, int B, int cap, int pinned, int kv_dim, cudaStream_t st);
// out[b, h*hd:(h+1)*hd] = softmax(q_h . K^T * scale) V over the cached slots (the new token's slot included, so
// call after gb_kv_append).  window > 0 masks slots older than `window` positions.  scratch: B*H*splits*(hd+2) floats.
int gb_decode_attn(const void* q16, long long ld_q, const void* cacheK, const void* cacheV, const int* slot_pos,
                   const gb_seq_state* state, void* out16, long long ld_o, float* scratch, int splits, int B, int H,
                   int KV, int hd, int cap, int window, float scale, int is_bf16, cudaStream_t st);
// After the step: abs_pos++, cache_len / ring_start move on; pos_out[b] = new abs_pos (feeds RoPE of the next step).
int gb_decode_advance(gb_seq_state* state, int* pos_out, int B, int cap, int pinned, cudaStream_t st);

typedef struct gb_sample_args {
  const float* logits; long long ld;   // [B, V] fp32 (modified in place by the penalties)
  int B, V;
  float temperature; int top_k; float top_p, min_p;
  float rep_penalty, freq_penalty, presence_penalty; int rep_window;
  int greedy;
  const int* history; int hist_cap;    // [B, hist_cap] ring of previous tokens, hist_len[b] valid entries (oldest first)
  int* hist_len;
  const float* uniforms;               // draws in [0,1) from the host generator (same stream as a host sampler):
                                       // [B] when step == NULL, else a [log_cap, B] table indexed by step[0]
  int* out_tok;                        // [B] sampled token, also appended to the history
  gb_seq_state* state;                 // done flag set when the token is in stop[]
  const int* stop; int n_stop;
  int* tok_log; int log_cap; const int* step;   // tok_log[b, step[0]] = token (device-side transcript), may be NULL
} gb_sample_args;
int gb_sample(const gb_sample_args* a, cudaStream_t st);

// ---- fused forms of the token step (same numbers as the separate kernels; see decode.cu)
// out = W @ rmsnorm(x32) for fp32 rows x32 [B, K]; returns -2 when B*K*2 bytes do not fit the shared-memory budget.
int gb_gemv_norm(const void* W, int fmt, int N, int K, const float* x32, int ldx32, const float* norm_w, float eps, int B,
                 void* out, int ldo, int out_f32, int is_bf16, cudaStream_t st);
// Router of rmsnorm(x32) [B, d]: picks to idx_out / w_out [B, top_k].
int gb_route_norm(const float* x32, const float* norm_w, float eps, const float* router_w, const float* bias, int B, int d,
                  int ne, int top_k, int* idx_out, float* w_out, int is_bf16, cudaStream_t st);
// act = SwiGLU(gate, up) of the experts named by idx [B, top_k] (+ the shared one) applied to rmsnorm(x32).
// idx == NULL: dense feed-forward block.
int gb_swiglu_norm(const void* Wg, const void* Wu, int fmt, int ne, int E, int d, const float* x32, const float* norm_w, float eps,
                   const int* idx, int B, int top_k, int shared, void* act16, int is_bf16, cudaStream_t st);
// QK-norm + RoPE of the fused projection; q to q_out, k and v into the cache slot of the step (slot_pos updated).
int gb_qk_rope_append(const void* qkv, long long ld_in, void* q_out, long long ld_q, const float* qw, const float* kw,
                      const float* cos_sin, const int* pos, void* cacheK, void* cacheV, int* slot_pos,
                      const gb_seq_state* state, int B, int H, int KV, int hd, int cap, int pinned, float eps, int rope_type,
                      int is_bf16, cudaStream_t st);
// gb_decode_attn with the merge of the splits inside (ticket: B*KV ints, zero before the first call).
int gb_decode_attn_fused(const void* q16, long long ld_q, const void* cacheK, const void* cacheV, const int* slot_pos,
                         const gb_seq_state* state, void* out16, long long ld_o, float* scratch, int splits, int B, int H,
                         int KV, int hd, int cap, int window, float scale, int is_bf16, int* ticket, cudaStream_t st);

// ---- the whole token step of ONE sequence as one cooperative kernel (decode_mega.cu)
typedef struct gb_mega_layer {
  const float* attn_norm; const float* ffn_norm;
  const float* q_norm; const float* k_norm;      // NULL: no QK-norm
  const void* wqkv; const void* wo;              // stored rows, format `fmt`
  const float* router; const float* bias;        // NULL for a dense block / no balancing bias
  const void* wg; const void* wu; const void* wd;   // experts stacked, the shared one last
  void* cache_k; void* cache_v;                  // [cap, KV * hd] 16-bit
} gb_mega_layer;

typedef struct gb_mega_args {
  const gb_mega_layer* layers;                   // device array [n_layers]
  int n_layers, d, H, KV, hd, ne, top_k, shared, E, V;   // ne == 0: dense feed-forward of width E
  int fmt, head_fmt, is_bf16, rope_type;         // head_fmt: fmt, GB_W_F16 or GB_W_BF16
  float eps, scale;
  const float* emb; const int* cur_tok;          // fp32 embedding rows; the token to run
  const float* final_norm; const void* head; float* logits;   // logits: [V] fp32
  const float* cos_sin; int* pos;                // RoPE table [positions, hd]; pos[0] = position of the token
  gb_seq_state* state; int* slot_pos;            // advanced by the kernel at the end of the step
  int cap, pinned, window;
  float* xbuf;                                   // 2 * d floats
  void* qkv;                                     // (H + 2 KV) * hd 16-bit
  float* att_scratch; int max_splits;            // H * max_splits * (hd + 2) floats
  void* act;                                     // slots * E 16-bit
  int* r_idx; float* r_w;                        // router choice of the last layer (may be NULL)
  unsigned* sync;                                // 4 words, zero before the first launch, owned by the kernel afterwards
  int* status;                                   // set to 401 when a grid-wide wait ran out
  unsigned long long* prof;                      // NULL, or 16 * n_layers + 2 words: CTA 0's global-timer marks in
                                                 // nanoseconds (start; per layer both sides of each of the five
                                                 // barriers and six points inside the phases; end)
  int stage_bytes;                               // filled in by the launcher: shared-memory bytes per warp for staged rows
} gb_mega_args;
int gb_decode_mega_ok(const gb_mega_args* a);    // 0 when the shapes are covered, else a negative code
int gb_decode_mega_grid(void);                   // CTAs of the launch (one per SM)
int gb_decode_mega(const gb_mega_args* a, cudaStream_t st);

#ifdef __cplusplus
}
#endif
