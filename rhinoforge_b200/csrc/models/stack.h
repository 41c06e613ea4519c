// Transformer-stack runtime: one native object per model "subsystem" (causal
// decoder, vision tower, prefix LM, action expert) that owns the per-layer
// weight pointers, plans a static activation arena once, and enqueues the
// whole layer loop -- hand-written sm_100a kernels only -- on a CUDA stream so
// that a decode step or a denoise loop can be captured into one CUDA graph.
//
// This is the B200 counterpart of the reference's FusedModelBase subclasses
// (src/core/fused_model_base.h:466-1083, src/fused/rpu_qwen3_model.h:3040-3705):
// instead of one C++ class per family, a family is a StackConfig (norm kind,
// QK-norm, rope kind, GLU vs plain MLP, biases, gated residual, KV source).
#pragma once
#include <stdint.h>

#include "../rf_api.h"

#ifdef __cplusplus
extern "C" {
#endif

enum RfNormKind { RF_NORM_RMS = 0, RF_NORM_RMS_GEMMA = 1, RF_NORM_LAYERNORM = 2, RF_NORM_ADARMS = 3 };
enum RfMlpKind { RF_MLP_SWIGLU = 0, RF_MLP_GEGLU_TANH = 1, RF_MLP_GELU_TANH = 2, RF_MLP_GELU_ERF = 3, RF_MLP_SILU = 4 };

typedef struct RfStackConfig {
  int32_t layers, hidden;
  int32_t Hq, Hkv, hd;          // LOCAL (per rank) head counts; hd is the padded head dim
  int32_t inter;                // LOCAL intermediate size
  int32_t rot_dim;              // 0: no rope
  int32_t norm_kind, mlp_kind;
  float eps;
  int32_t qk_norm, rope_before_norm;
  int32_t gated_residual;       // adaRMS: hidden += gate * sublayer(x)
  int32_t sandwich_norm;        // extra norm on each sublayer output (Gemma-3/4 style)
  int32_t paged_kv;             // 1: K/V go to the paged pool; 0: attention reads K/V from the qkv buffer
  int32_t causal, window;
  float attn_scale;             // <= 0: 1/sqrt(true_hd) with true_hd below
  int32_t true_hd;              // unpadded head dim (for the softmax scale)
  int32_t dtype;                // 0 fp16, 1 bf16
  int32_t max_tokens;           // rows the arena is planned for
  int32_t max_seqs;
  int32_t vocab_local;          // lm_head rows on this rank (0: no head)
  int32_t vocab_offset;         // first vocab id of this rank's shard
  int32_t tp_world, tp_rank;
  int32_t weights_int8;         // linear weights are int8 + per-channel scale
  int32_t decode_gemv_max_m;    // use the CUDA-core GEMV for token counts up to this (0: never)
  int32_t attn_gate;            // q_proj also yields a per-channel output gate: attn *= sigmoid(gate)
  // Gated-DeltaNet layers (LOCAL head counts); gdn_Hv == 0: the stack has none
  int32_t gdn_Hk, gdn_Hv, gdn_Dk, gdn_Dv, gdn_conv_k;
  int32_t weights_packed;       // every linear weight (and the lm_head) is in the tile-major layout of RfGemm.w_packed
  // Sparse MoE MLP in the dense-einsum form (moe_experts == 0: dense MLP).  `inter` is then the LOCAL width of the
  // whole expert bank, moe_experts * moe_expert_inter plus the always-on shared expert's columns behind it: w_up /
  // w_down hold every expert side by side, the router picks moe_top_k experts per token and the routing weight
  // (zero for an expert that was not picked) scales that expert's column block between the two GEMMs.
  int32_t moe_experts, moe_top_k, moe_expert_inter;
  int32_t moe_score_fn;         // 0 sigmoid (+ selection-only bias), 1 softmax
  int32_t moe_norm_topk;        // picked weights are normalised to sum 1 before the routed scale
  float moe_routed_scale;
  // weights_int8 with weights_bits == 4: every quantised linear weight is the tile-major int4 image of RfGemm.w_bits
  // (weights_group = 0: the layer's s* pointers are per-channel scale vectors; 32 / 64 / 128: the scales sit inside
  // the image and a non-null s* pointer only marks the weight as quantised)
  int32_t weights_bits, weights_group;
  // 1: the norm weights of the two pre-norms are already multiplied into the columns of wqkv and w_up (plain RMSNorm or
  // the (1 + w) form, one GPU, dense MLP).  The stack then treats norm1_w / norm2_w as all-ones: with at most 256
  // tokens the residual GEMMs (o_proj, down_proj) emit per-token sums of squares and the next projection scales its
  // result by the reciprocal RMS, so no RMSNorm kernel runs between them; with more tokens a weight-free RMSNorm runs.
  int32_t norm_folded;
  // 1: every GEMM of the stack runs on the tcgen05 kernels.  Decoder engines set it so that the tokens of a tensor-
  // parallel run and of a one-GPU run come from one kernel family (the row-parallel GEMMs with a collective in them
  // always do); the action heads leave it 0 and take the latency-bound kernel for their few-row shapes.
  int32_t gemm_streaming_only;
} RfStackConfig;

typedef struct RfLayerWeights {
  const void* norm1_w; const void* norm1_b;
  const void* wqkv; const void* bqkv; const void* sqkv;
  const void* q_norm_w; const void* k_norm_w;
  const void* wo; const void* bo; const void* so;
  const void* norm2_w; const void* norm2_b;
  const void* w_up; const void* b_up; const void* s_up;       // [2*inter, H] for GLU kinds, [inter, H] otherwise
  const void* w_down; const void* b_down; const void* s_down;
  const void* post_attn_norm_w; const void* post_mlp_norm_w;   // sandwich norms
  void* k_pool; void* v_pool;                                  // this layer's KV pages
  // mixer == 1: Gated-DeltaNet layer.  wqkv is then the fused input projection
  // [q | k | v | z | b (padded to 8) | a (padded to 8)] and wo the output projection.
  int64_t mixer;
  const void* gdn_conv_w;        // [conv_dim, K]
  const float* gdn_A_log; const float* gdn_dt_bias;            // [Hv] fp32
  const void* gdn_norm_w;        // [Dv]
  void* gdn_conv_state;          // [slots, K-1, conv_dim]
  float* gdn_rec_state;          // [slots, Hv, Dk, Dv] fp32
  const void* moe_router_w;      // [experts, hidden]; null: this layer's MLP is dense
  const float* moe_router_bias;  // [experts] fp32 selection bias (optional)
} RfLayerWeights;

typedef struct RfStackComm {
  void* const* recv;       // device array [world] -> peers' receive buffers
  uint32_t* const* flags;  // device array [world] -> peers' flag arrays
  uint32_t* state;         // local [4]
  uint64_t recv_half_bytes;
  int32_t flag_count;
  int32_t cnt_base;        // first of `world` arrival counters in every rank's flag array (publish / consume all-reduce)
  // Symmetric activation buffers (optional; sym_rows == 0: none): every rank allocated [sym_rows, hidden] buffers for
  // the residual stream, the normalised rows, a side result and the row-parallel GEMM's partial at the same offsets
  // of its peer-mapped region.  *_tab are device arrays [world] of the ranks' bases, sym_* this rank's own bases.
  // With them a prefill-sized all-reduce runs as GEMM -> rf_ar_rows (reduce-scatter by peer loads, all-gather by peer
  // stores); the caller must then pass sym_hidden as RfStackForward.hidden.
  int32_t sym_rows;
  int32_t rows_flag_base;  // first of the 16 flags of rf_ar_rows in every rank's flag array
  void* sym_hidden; void* sym_xn; void* sym_tmp; void* sym_partial;
  void* const* hidden_tab; void* const* xn_tab; void* const* tmp_tab; void* const* partial_tab;
} RfStackComm;

typedef struct RfStackForward {
  void* hidden;                  // [tokens, hidden] residual stream, updated in place
  int32_t tokens;
  int32_t decode;                // 1: one token per sequence
  const int32_t* pos; int32_t pos_stride;
  const float* cos; const float* sin; const int8_t* axis_of_freq;
  const int32_t* seq_of_tok; const int32_t* cache_pos;
  int32_t num_seqs;
  const int32_t* q_start; const int32_t* q_len; const int32_t* kv_start; const int32_t* kv_len;
  int32_t max_q_len, max_kv_len;
  const int32_t* page_table; int32_t pt_stride; int64_t pool_pages;
  const uint8_t* mask; int64_t mask_ld, mask_seq_stride;
  const int32_t* seg_q; const int32_t* seg_k;
  const void* mod; int32_t rows_per_mod;   // adaRMS: [layers][2][tokens/rows_per_mod][3*hidden]
  int32_t layer_begin, layer_end;          // run layers [begin, end) (0,0 = all)
  // DeepStack: after layer i (< n_deepstack) add deepstack[i][j] to hidden row deepstack_rows[j]
  const void* const* deepstack; const int32_t* deepstack_rows; int32_t n_deepstack, n_deepstack_rows;
  // tap: copy hidden after layer tap_layers[i] into taps[i] (vision DeepStack features)
  void* const* taps; const int32_t* tap_layers; int32_t n_taps;
  // recurrent-state bookkeeping of Gated-DeltaNet layers: state slot of every sequence (null:
  // sequence index) and whether the sequence starts from an empty state (null: continue)
  const int32_t* state_slot; const int32_t* state_fresh;
  // Mixture-of-transformers routing by row: rows [0, twin_split) run through the layer's own weights, rows
  // [twin_split, tokens) through its twin set (rf_stack_set_twin_layer).  0: no routing.  The caller orders the rows
  // accordingly; positions, cache rows and the attention mask are per row, so the order is free.
  int32_t twin_split;
  int32_t reserved0;
} RfStackForward;

int64_t rf_stack_create(const RfStackConfig* cfg);
int rf_stack_destroy(int64_t h);
int rf_stack_set_layer(int64_t h, int32_t layer, const RfLayerWeights* w);
// Second weight set of a layer (mixture-of-transformers): the norms, q/k norms and the four projections of the rows
// routed to it (RfStackForward.twin_split); the KV pool and everything else stay the layer's own.  Dense attention
// layers on one GPU, weights in the same layout as the layer's own.
int rf_stack_set_twin_layer(int64_t h, int32_t layer, const RfLayerWeights* w);
// Final norm weights of the twin rows (rf_stack_final_norm_twin).
int rf_stack_set_twin_head(int64_t h, const void* final_norm_w);
int rf_stack_final_norm_twin(int64_t h, const void* hidden, void* out, int32_t rows, int32_t twin_split, rf_stream_t stream);
// Re-point one layer at another KV pool (binding a different cache object).
int rf_stack_set_kv(int64_t h, int32_t layer, void* k_pool, void* v_pool);
// Re-point a Gated-DeltaNet layer at other state tensors (binding a different cache object).
int rf_stack_set_state(int64_t h, int32_t layer, void* conv_state, float* rec_state);
int rf_stack_set_head(int64_t h, const void* final_norm_w, const void* final_norm_b, const void* w_lm,
                      const void* s_lm);
int rf_stack_set_comm(int64_t h, const RfStackComm* c);
// Bytes of activation arena / number of status words the handle needs; the
// caller allocates (zero-filled) device memory and binds it once.
uint64_t rf_stack_arena_bytes(int64_t h);
int rf_stack_bind_arena(int64_t h, void* base, uint64_t bytes);
int32_t* rf_stack_status_ptr(int64_t h);
int rf_stack_forward(int64_t h, const RfStackForward* f, rf_stream_t stream);
// final norm on `rows` selected rows (row_idx, or the first `rows` rows when null) of hidden,
// lm_head GEMM, arg-max -> out_ids (global vocab ids); logits_out optional [rows, vocab_local].
int rf_stack_head(int64_t h, const void* hidden, const int32_t* row_idx, int32_t rows, int32_t* out_ids,
                  float* out_vals, void* logits_out, rf_stream_t stream);
int rf_stack_final_norm(int64_t h, const void* hidden, void* out, int32_t rows, rf_stream_t stream);
// Device-resident decode bookkeeping inside the captured step: pos += 1, kv_len += 1,
// ids = out_ids (next step's input), hist[*step] = out_ids, *step += 1.  Any pointer may be null.
int rf_decode_advance(int32_t* pos, int32_t pos_stride, int32_t* kv_len, int32_t n, const int32_t* out_ids,
                      int32_t* ids, int32_t* hist, int32_t* step, int32_t hist_cap, rf_stream_t stream);

#ifdef __cplusplus
}
#endif
