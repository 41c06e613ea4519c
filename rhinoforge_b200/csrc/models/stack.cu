// Transformer-stack runtime (see stack.h).  Host-side C++ only: every device
// operation is one of the kernels in ../kernels, enqueued on the caller's stream.
#include "stack.h"

#include <stdlib.h>

#include <algorithm>
#include <memory>
#include <string>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../common/status.h"
#include "../runtime/handle_registry.h"

namespace rf {

struct Stack {
  RfStackConfig cfg;
  std::vector<RfLayerWeights> layers;
  std::vector<RfLayerWeights> twins;      // second weight set per layer (mixture-of-transformers); wqkv == null: none
  const void* twin_final_norm_w = nullptr;
  const void* final_norm_w = nullptr;
  const void* final_norm_b = nullptr;
  const void* w_lm = nullptr;
  const void* s_lm = nullptr;
  RfStackComm comm{};
  bool has_comm = false;
  // arena
  uint8_t* base = nullptr;
  uint64_t bytes = 0;
  uint64_t off_xn = 0, off_attn = 0, off_tmp = 0, off_wide = 0, off_conv = 0, off_head_xn = 0, off_logits = 0,
           off_argmax = 0, off_attn_ws = 0, off_wscratch = 0, off_moe = 0, off_sk_ws = 0, off_sk_flags = 0, off_ss = 0,
           off_status = 0, total = 0;
  uint64_t attn_ws_bytes = 0, argmax_bytes = 0, wscratch_bytes = 0, sk_ws_bytes = 0;
  int ss_ld = 0, ss_tiles = 0;
  static constexpr int kSkFlags = 1024;

  int qkv_dim() const { return (cfg.Hq + 2 * cfg.Hkv) * cfg.hd + (cfg.attn_gate ? cfg.Hq * cfg.hd : 0); }
  // Gated-DeltaNet geometry
  int gdn_key_dim() const { return cfg.gdn_Hk * cfg.gdn_Dk; }
  int gdn_value_dim() const { return cfg.gdn_Hv * cfg.gdn_Dv; }
  int gdn_conv_dim() const { return 2 * gdn_key_dim() + gdn_value_dim(); }
  int gdn_ba_pad() const { return (cfg.gdn_Hv + 7) / 8 * 8; }
  int gdn_in_dim() const { return cfg.gdn_Hv > 0 ? gdn_conv_dim() + gdn_value_dim() + 2 * gdn_ba_pad() : 0; }
  bool glu() const { return cfg.mlp_kind == RF_MLP_SWIGLU || cfg.mlp_kind == RF_MLP_GEGLU_TANH; }
  int moe_ld() const { return (cfg.moe_experts + 7) / 8 * 8; }   // row pitch of the router buffers

  void plan() {
    auto al = [](uint64_t v) { return (v + 1023) & ~uint64_t(1023); };
    const uint64_t T = (uint64_t)cfg.max_tokens, e = 2;
    uint64_t o = 0;
    off_xn = o; o += al(T * cfg.hidden * e);
    off_attn = o; o += al(T * std::max<uint64_t>(cfg.Hq * cfg.hd, gdn_value_dim()) * e);
    off_tmp = o; o += al(T * cfg.hidden * e);
    off_wide = o; o += al(T * std::max<uint64_t>(std::max(qkv_dim(), gdn_in_dim()), cfg.inter) * e);
    off_conv = o; o += al(T * (uint64_t)(cfg.gdn_Hv > 0 ? gdn_conv_dim() : 0) * e);
    off_head_xn = o; o += al((uint64_t)cfg.max_seqs * cfg.hidden * e);
    off_logits = o; o += al((uint64_t)cfg.max_seqs * std::max(cfg.vocab_local, 1) * e);
    argmax_bytes = rf_argmax_scratch_bytes(cfg.max_seqs, std::max(cfg.vocab_local, 1));
    off_argmax = o; o += al(argmax_bytes);
    attn_ws_bytes = cfg.paged_kv ? rf_attn_decode_scratch_bytes(cfg.max_seqs, cfg.Hq, cfg.hd) : 0;
    off_attn_ws = o; o += al(attn_ws_bytes);
    // W8A16 with prefill-sized token counts: room for the largest weight widened to 16 bits (tile-major image)
    wscratch_bytes = 0;
    if (cfg.weights_int8 && cfg.weights_bits != 4 && cfg.weights_packed && cfg.max_tokens > 256) {
      auto img = [](uint64_t rows, uint64_t K, uint64_t sections) {
        return sections * ((rows + 127) / 128) * 128 * ((K + 63) / 64) * 64 * 2;
      };
      const uint64_t H = (uint64_t)cfg.hidden, I = (uint64_t)cfg.inter;
      wscratch_bytes = std::max(std::max(img(qkv_dim(), H, 1), img(H, (uint64_t)cfg.Hq * cfg.hd, 1)),
                                std::max(glu() ? img(I, H, 2) : img(I, H, 1), img(H, I, 1)));
    }
    off_wscratch = o; o += al(wscratch_bytes);
    // MoE router: logits and dense routing weights [tokens, experts] (16-bit each), ids + weights of the picks
    off_moe = o;
    if (cfg.moe_experts > 0)
      o += al(T * (uint64_t)moe_ld() * e * 2) + al(T * (uint64_t)std::max(cfg.moe_top_k, 1) * 8);
    // persistent stream-K GEMM (at most 256 tokens): one fp32 partial slot (two accumulators of up to 256 token
    // columns x 128 features) and one flag per CTA; the flags start at zero and every launch leaves them at zero
    {
      const uint64_t bn = (uint64_t)((std::min(cfg.max_tokens, 256) + 15) / 16 * 16);
      sk_ws_bytes = (uint64_t)sm_count() * 2 /*CTAs per SM*/ * 2 /*accumulators*/ * bn * 128 * sizeof(float);
    }
    off_sk_ws = o; o += al(sk_ws_bytes);
    off_sk_flags = o; o += al(kSkFlags * sizeof(uint32_t));
    // folded RMSNorm: two buffers (after attention, after the MLP) of per-(128-column tile, token) sums of squares
    ss_ld = std::min(cfg.max_tokens, 256);
    ss_tiles = (cfg.hidden + 127) / 128;
    off_ss = o; o += al(cfg.norm_folded ? (uint64_t)2 * ss_tiles * ss_ld * sizeof(float) : 0);
    off_status = o; o += al(kStatusWords * sizeof(int32_t));
    total = o;
  }
  template <typename P = void> P* at(uint64_t off) const { return reinterpret_cast<P*>(base + off); }
  int32_t* status() const { return base ? at<int32_t>(off_status) : nullptr; }
};

static HandleRegistry<Stack>& registry() {
  static HandleRegistry<Stack> r;
  return r;
}

static int act_of(int mlp_kind) {
  switch (mlp_kind) {
    case RF_MLP_SWIGLU: return kActSiluMul;
    case RF_MLP_GEGLU_TANH: return kActGeluTanhMul;
    case RF_MLP_GELU_TANH: return kActGeluTanh;
    case RF_MLP_GELU_ERF: return kActGeluErf;
    case RF_MLP_SILU: return kActSilu;
  }
  return kActNone;
}

// Tensor-parallel all-reduce form for at most 256 tokens: "publish" (default) = the row-parallel GEMM pushes its
// partial rows and exits, rf_ar_consume waits, reduces, adds the residual and applies the next RMSNorm;
// RF_TP_AR=inkernel keeps wait + reduction inside the GEMM's epilogue (A/B timing).
static bool tp_publish_enabled() {
  static const bool v = [] { const char* e = getenv("RF_TP_AR"); return !(e && std::string(e) == "inkernel"); }();
  return v;
}

// Under tensor parallelism with prefill-sized rows the residual stream stays sharded by rows between the layers (each
// rank keeps the rows it reduces; only their RMSNorm is gathered).  RF_TP_SEQ_SHARD=0 gathers the stream itself too.
static bool tp_seq_shard_enabled() {
  static const bool v = [] { const char* e = getenv("RF_TP_SEQ_SHARD"); return !(e && e[0] == '0'); }();
  return v;
}

// L2 prefetch hint for the next linear() call on this thread (set by the layer loop right before the call, consumed
// by it): the weights of the linear layer that FOLLOWS, so that a weight-streaming GEMM hands HBM over to its
// successor without an idle gap.  RF_GEMM_L2_PREFETCH_MB caps the bytes asked for (0: off).
// Shortest prefill (longest new-token run of the launch) that takes the chunked Gated-DeltaNet kernel; RF_GDN_CHUNK_MIN
// overrides it (0 keeps every prefill on the recurrent kernel).
static int gdn_chunk_min() {
  static const int v = [] {
    const char* e = getenv("RF_GDN_CHUNK_MIN");
    const int n = e ? atoi(e) : 16;
    return n <= 0 ? (1 << 30) : n;
  }();
  return v;
}

static thread_local const void* t_pf_ptr = nullptr;
static thread_local uint64_t t_pf_bytes = 0;
static uint64_t prefetch_cap_bytes() {
  static const uint64_t v = [] {
    const char* e = getenv("RF_GEMM_L2_PREFETCH_MB");
    const long mb = e ? atol(e) : 0;
    return (uint64_t)(mb < 0 ? 0 : mb) << 20;
  }();
  return v;
}
static void hint_next_weights(const Stack& s, const void* w, const void* scale, int64_t rows, int64_t K, int sections,
                              int tokens) {
  t_pf_ptr = nullptr; t_pf_bytes = 0;
  if (!w || tokens > 256 || prefetch_cap_bytes() == 0) return;
  const bool quantised = s.cfg.weights_int8 && scale;
  const int eb = quantised ? 1 : 2;
  const uint64_t bytes = (quantised && s.cfg.weights_bits == 4) ? rf_pack_w4_bytes(rows, K, sections, s.cfg.weights_group)
                         : s.cfg.weights_packed            ? rf_pack_weight_bytes(rows, K, sections, eb)
                                                           : (uint64_t)rows * K * eb;
  t_pf_ptr = w;
  t_pf_bytes = bytes < prefetch_cap_bytes() ? bytes : prefetch_cap_bytes();
}

// Folded RMSNorm wiring of the next linear() call on this thread (set by the layer loop right before the call, consumed
// by it): the buffer it writes its per-tile sums of squares to, and / or the buffer whose sums give its row scale.
static thread_local float* t_ss_out = nullptr;
static thread_local const float* t_ss_in = nullptr;

// One linear layer: picks GEMV / tcgen05 GEMM / W8A16 and wires the fused all-reduce.  pub_ctas != null asks for
// the publish-and-exit form: *pub_ctas receives the CTA count the consumer must wait for, or 0 when the shape took
// the in-kernel form after all (more than 256 tokens), in which case `out` and `residual` were used as given.
static int linear(const Stack& s, const void* x, int64_t ldx, const void* w, const void* scale,
                  const void* bias, void* out, int64_t ldo, const void* residual, int64_t ldr, int M,
                  int N, int K, int act, int dual_offset, bool all_reduce, cudaStream_t st,
                  int* pub_ctas = nullptr) {
  RfGemm g = {};
  g.x = x; g.ldx = ldx; g.w = w; g.ldw = K; g.out = out; g.ldo = ldo;
  g.residual = residual; g.ldr = ldr; g.bias = bias; g.scale = scale;
  g.M = M; g.N = N; g.K = K; g.dtype = s.cfg.dtype; g.act = act; g.dual_offset = dual_offset;
  g.w_int8 = s.cfg.weights_int8 && scale != nullptr;
  g.w_packed = s.cfg.weights_packed;
  if (g.w_int8 && s.cfg.weights_bits == 4) {
    g.w_bits = 4; g.w_group = s.cfg.weights_group;
    if (g.w_group > 0) g.scale = nullptr;      // the group scales are part of the weight image
  }
  if (g.w_int8 && s.wscratch_bytes) {
    g.w_scratch = s.at(s.off_wscratch);
    g.w_scratch_bytes = s.wscratch_bytes;
  }
  g.status = s.status();
  g.force_swap = -1;
  g.streaming_only = s.cfg.gemm_streaming_only;
  g.prefetch = t_pf_ptr; g.prefetch_bytes = t_pf_bytes;
  t_pf_ptr = nullptr; t_pf_bytes = 0;
  if (t_ss_out || t_ss_in) {
    g.ss_out = t_ss_out; g.ss_in = t_ss_in;
    g.ss_ld = s.ss_ld; g.ss_tiles = s.ss_tiles; g.ss_dim = s.cfg.hidden; g.ss_eps = s.cfg.eps;
    t_ss_out = nullptr; t_ss_in = nullptr;
  }
  g.ws = s.at<float>(s.off_sk_ws); g.ws_bytes = s.sk_ws_bytes;
  g.sem = s.at<uint32_t>(s.off_sk_flags); g.sem_count = Stack::kSkFlags;
  const bool ar = all_reduce && s.cfg.tp_world > 1;
  if (ar) {
    if (!s.has_comm) return fail(RF_ERR_STATE, "tensor-parallel stack has no comm buffers bound");
    g.ar_world = s.cfg.tp_world; g.ar_rank = s.cfg.tp_rank;
    g.ar_recv = s.comm.recv; g.ar_flags = s.comm.flags; g.ar_state = s.comm.state;
    g.ar_recv_bytes = s.comm.recv_half_bytes; g.ar_flag_count = s.comm.flag_count;
    if (pub_ctas) {
      *pub_ctas = 0;
      if (M <= 256 && N % 8 == 0 && dual_offset == 0) {
        g.ar_publish = 1;
        g.ar_cnt_base = s.comm.cnt_base;
        const int ctas = rf_gemm_grid_ctas(&g);
        if (ctas < 0) return ctas;
        *pub_ctas = ctas;
      }
    }
  } else if (pub_ctas) {
    *pub_ctas = 0;
  }
  if (!ar && !g.w_packed && M <= 8 && (M <= s.cfg.decode_gemv_max_m) && K % (g.w_int8 ? 16 : 8) == 0) return rf_gemv(&g, st);
  if (g.w_int8) return rf_gemm_w8a16(&g, st);
  return rf_gemm(&g, st);
}

// Finish a published all-reduce: out = sum of the ranks' partial rows (+ residual), and when norm_w is given the
// RMSNorm of the finished rows into norm_out (the stack's plain or Gemma-style RMSNorm).
static int consume(const Stack& s, int pub_ctas, const void* residual, void* out, int M, const void* norm_w,
                   void* norm_out, cudaStream_t st) {
  RfArConsume a = {};
  a.M = M; a.N = s.cfg.hidden; a.world = s.cfg.tp_world; a.rank = s.cfg.tp_rank;
  a.ar_recv = s.comm.recv; a.ar_flags = s.comm.flags; a.ar_state = s.comm.state;
  a.ar_recv_bytes = s.comm.recv_half_bytes; a.ar_cnt_base = s.comm.cnt_base; a.pub_ctas = pub_ctas;
  a.residual = residual; a.ldr = s.cfg.hidden; a.out = out; a.ldo = s.cfg.hidden;
  if (norm_w) {
    a.norm_w = norm_w; a.norm_out = norm_out; a.ldn = s.cfg.hidden; a.eps = s.cfg.eps;
    a.norm_mode = s.cfg.norm_kind == RF_NORM_RMS_GEMMA ? 2 : 1;
  }
  a.status = s.status(); a.dtype = s.cfg.dtype;
  return rf_ar_consume(&a, st);
}

// Row-parallel projection + all-reduce (+ residual into `out` when residual != null).  With tensor parallelism and
// at most 256 tokens this is GEMM(publish) + consume, and the RMSNorm that follows in the layer (next_norm_w, result
// in next_xn) rides in the consumer: *normed tells the caller that next_xn is valid.
static int linear_ar(const Stack& s, const void* x, int64_t ldx, const void* w, const void* scale, const void* bias,
                     void* out, const void* residual, int M, int K, const void* next_norm_w, void* next_xn,
                     bool* normed, cudaStream_t st, bool rows_stay = false) {
  const int H = s.cfg.hidden;
  if (normed) *normed = false;
  if (s.cfg.tp_world > 1 && tp_publish_enabled() && M > 256 && s.comm.sym_rows >= M &&
      (out == s.comm.sym_hidden || out == s.comm.sym_tmp) && (!residual || residual == out)) {
    // Prefill-sized rows: the GEMM (persistent kernel, no collective in it) writes this rank's partial into its
    // symmetric buffer; rf_ar_rows reduces the rows this rank owns over NVLink, adds the residual, applies the
    // following RMSNorm and stores the finished rows into every rank's buffers.  Only rank 0 adds the bias.
    int rc = linear(s, x, ldx, w, scale, s.cfg.tp_rank == 0 ? bias : nullptr, s.comm.sym_partial, H, nullptr, 0, M, H, K,
                    kActNone, 0, false, st);
    if (rc) return rc;
    RfArRows a = {};
    a.M = M; a.N = H; a.world = s.cfg.tp_world; a.rank = s.cfg.tp_rank;
    a.partial_tab = s.comm.partial_tab;
    a.out_tab = out == s.comm.sym_hidden ? s.comm.hidden_tab : s.comm.tmp_tab;
    a.ar_flags = s.comm.flags; a.ar_state = s.comm.state; a.flag_base = s.comm.rows_flag_base;
    a.add_residual = residual ? 1 : 0;
    if (next_norm_w && next_xn == s.comm.sym_xn) {
      a.norm_tab = s.comm.xn_tab; a.norm_w = next_norm_w; a.eps = s.cfg.eps;
      a.norm_mode = s.cfg.norm_kind == RF_NORM_RMS_GEMMA ? 2 : 1;
      if (normed) *normed = true;
      // sequence-sharded residual stream: the next reader of these rows is the owner's own next reduction, so they
      // stay there and only their RMSNorm is gathered
      a.out_local = (rows_stay && residual && tp_seq_shard_enabled()) ? 1 : 0;
    }
    a.status = s.status(); a.dtype = s.cfg.dtype;
    return rf_ar_rows(&a, st);
  }
  if (s.cfg.tp_world > 1 && tp_publish_enabled()) {
    int ctas = 0;
    int rc = linear(s, x, ldx, w, scale, bias, out, H, residual, residual ? H : 0, M, H, K, kActNone, 0, true, st, &ctas);
    if (rc) return rc;
    if (ctas > 0) {
      rc = consume(s, ctas, residual, out, M, next_norm_w, next_xn, st);
      if (rc) return rc;
      if (normed && next_norm_w) *normed = true;
    }
    return RF_OK;
  }
  return linear(s, x, ldx, w, scale, bias, out, H, residual, residual ? H : 0, M, H, K, kActNone, 0, true, st);
}

static int norm(const Stack& s, const void* x, const void* w, const void* b, void* y, int rows,
                const void* mod, int rows_per_mod, cudaStream_t st) {
  const int H = s.cfg.hidden;
  switch (s.cfg.norm_kind) {
    case RF_NORM_LAYERNORM:
      return rf_layernorm(x, w, b, y, rows, H, H, H, s.cfg.eps, s.cfg.dtype, st);
    case RF_NORM_ADARMS:
      return rf_rmsnorm(x, nullptr, nullptr, y, nullptr, mod, rows_per_mod, rows, H, H, H, s.cfg.eps, 0,
                        s.cfg.dtype, st);
    case RF_NORM_RMS_GEMMA:
      return rf_rmsnorm(x, nullptr, w, y, nullptr, nullptr, 1, rows, H, H, H, s.cfg.eps, 1, s.cfg.dtype, st);
    default:
      return rf_rmsnorm(x, nullptr, w, y, nullptr, nullptr, 1, rows, H, H, H, s.cfg.eps, 0, s.cfg.dtype, st);
  }
}

// A projection of rows routed to two weight sets: rows [0, split) with (wA, sA, bA), rows [split, M) with (wB, sB, bB).
static int linear_twin(const Stack& s, const void* x, int64_t ldx, const void* wA, const void* sA, const void* bA,
                       const void* wB, const void* sB, const void* bB, void* out, int64_t ldo, const void* residual,
                       int64_t ldr, int M, int split, int N, int K, int act, int dual_offset, cudaStream_t st) {
  const size_t e = 2;
  int rc = RF_OK;
  if (split > 0) rc = linear(s, x, ldx, wA, sA, bA, out, ldo, residual, ldr, split, N, K, act, dual_offset, false, st);
  if (rc == RF_OK && split < M)
    rc = linear(s, (const uint8_t*)x + (size_t)split * ldx * e, ldx, wB, sB, bB, (uint8_t*)out + (size_t)split * ldo * e, ldo,
                residual ? (const uint8_t*)residual + (size_t)split * ldr * e : nullptr, ldr, M - split, N, K, act,
                dual_offset, false, st);
  return rc;
}

static int forward(Stack& s, const RfStackForward& f, cudaStream_t st) {
  const RfStackConfig& c = s.cfg;
  RF_REQUIRE(s.base != nullptr, "stack arena is not bound");
  RF_REQUIRE(f.hidden && f.tokens >= 0 && f.tokens <= c.max_tokens, "forward: %d tokens (max %d)", f.tokens, c.max_tokens);
  RF_REQUIRE(f.num_seqs > 0 && f.num_seqs <= c.max_seqs, "forward: %d sequences (max %d)", f.num_seqs, c.max_seqs);
  if (f.tokens == 0) return RF_OK;
  if (c.norm_kind == RF_NORM_ADARMS) RF_REQUIRE(f.mod && f.rows_per_mod > 0, "adaRMS stack needs mod");
  const int T = f.tokens, H = c.hidden, QD = s.qkv_dim(), AD = c.Hq * c.hd, I = c.inter;
  const int lb = f.layer_end > 0 ? f.layer_begin : 0, le = f.layer_end > 0 ? f.layer_end : c.layers;
  // under tensor parallelism with symmetric buffers the normalised rows and the side result live there, so that
  // the owner rank of a row can store them into every rank's copy
  const bool sym = s.has_comm && s.comm.sym_rows >= T && s.comm.sym_xn && s.comm.sym_tmp;
  void* xn = sym ? s.comm.sym_xn : s.at(s.off_xn);
  void* attn = s.at(s.off_attn);
  void* tmp = sym ? s.comm.sym_tmp : s.at(s.off_tmp);
  void* wide = s.at(s.off_wide);
  const size_t esz = 2;
  const int nmods = c.norm_kind == RF_NORM_ADARMS ? T / f.rows_per_mod : 0;
  const bool side = c.gated_residual || c.sandwich_norm;  // sublayer output goes to tmp first
  int rc;

  // A plain RMSNorm that follows an all-reduce can ride in the all-reduce's consumer (linear_ar)
  const bool norm_rides = !side && (c.norm_kind == RF_NORM_RMS || c.norm_kind == RF_NORM_RMS_GEMMA);
  bool have_xn = false;     // xn already holds this layer's first norm (written by the previous layer's consumer)
  // Norm weights folded into wqkv / w_up: the norm kernels (when they run) take no weight; with at most 256 tokens
  // they do not run at all between a residual GEMM and the next projection (sums of squares out, row scale in).
  const bool folded = c.norm_folded != 0;
  if (folded)
    RF_REQUIRE(norm_rides && c.tp_world == 1 && c.moe_experts == 0 && c.gdn_Hv == 0,
               "norm_folded needs a plain RMSNorm dense decoder on one GPU");
  const bool fuse_ss = folded && T <= 256;
  // mixture-of-transformers: rows [0, split) use the layers' own weights, rows [split, T) their twins
  const int split = f.twin_split;
  const bool twin = split > 0;
  if (twin) {
    RF_REQUIRE(split <= T && s.twins.size() == s.layers.size(), "twin_split %d needs twin weights on every layer (rows %d)", split, T);
    RF_REQUIRE(!folded && !side && c.tp_world == 1 && c.moe_experts == 0 && !f.decode && !f.mod,
               "twin routing runs on a plain pre-norm dense stack (prefill form, one GPU)");
  }
  float* ss_attn = s.at<float>(s.off_ss);                               // sums of squares of hidden after attention
  float* ss_mlp = ss_attn + (size_t)s.ss_tiles * s.ss_ld;               // ... after the MLP (the next layer's input)
  bool ss_ready = false;    // ss_mlp describes f.hidden as it is now

  for (int l = lb; l < le; ++l) {
    const RfLayerWeights& w = s.layers[l];
    const uint8_t* mod1 = f.mod ? (const uint8_t*)f.mod + ((size_t)(l * 2 + 0) * nmods) * 3 * H * esz : nullptr;
    const uint8_t* mod2 = f.mod ? (const uint8_t*)f.mod + ((size_t)(l * 2 + 1) * nmods) * 3 * H * esz : nullptr;
    // ---- token mixer: softmax attention or Gated-DeltaNet
    const bool qkv_from_hidden = fuse_ss && ss_ready;     // this layer's first norm is the QKV GEMM's row scale
    const RfLayerWeights* tw = twin ? &s.twins[l] : nullptr;
    if (twin) RF_REQUIRE(tw->wqkv && w.mixer == 0, "layer %d has no twin weights", l);
    const size_t hrow = (size_t)H * esz;
    if (twin) {
      rc = norm(s, f.hidden, w.norm1_w, w.norm1_b, xn, split, nullptr, 1, st);
      if (rc == RF_OK && split < T)
        rc = norm(s, (const uint8_t*)f.hidden + split * hrow, tw->norm1_w, tw->norm1_b, (uint8_t*)xn + split * hrow, T - split,
                  nullptr, 1, st);
      if (rc) return rc;
    } else if (!have_xn && !qkv_from_hidden) {
      rc = norm(s, f.hidden, folded ? nullptr : w.norm1_w, w.norm1_b, xn, T, mod1, f.rows_per_mod, st);
      if (rc) return rc;
    }
    have_xn = false;
    ss_ready = false;
    bool have_xn2 = false;  // xn holds the second norm (written by the attention all-reduce's consumer)
    const void* mix_out = attn;      // input of the output projection
    int mix_dim = AD;
    if (w.mixer == 1) {
      RF_REQUIRE(c.gdn_Hv > 0 && w.gdn_conv_w && w.gdn_conv_state && w.gdn_rec_state, "layer %d: GDN weights/state missing", l);
      const int CD = s.gdn_conv_dim(), VD = s.gdn_value_dim(), IN = s.gdn_in_dim(), BA = s.gdn_ba_pad();
      void* conv = s.at(s.off_conv);
      rc = linear(s, xn, H, w.wqkv, w.sqkv, nullptr, wide, IN, nullptr, 0, T, IN, H, kActNone, 0, false, st);
      if (rc) return rc;
      RfConv1d cv = {};
      cv.x = wide; cv.ldx = IN; cv.y = conv; cv.ldy = CD; cv.w = w.gdn_conv_w; cv.state = w.gdn_conv_state;
      cv.q_start = f.decode ? nullptr : f.q_start; cv.q_len = f.decode ? nullptr : f.q_len; cv.slot = f.state_slot;
      cv.num_seqs = f.num_seqs; cv.max_q_len = f.decode ? 1 : f.max_q_len; cv.C = CD; cv.K = c.gdn_conv_k; cv.silu = 1;
      cv.dtype = c.dtype;
      rc = rf_causal_conv1d(&cv, st);
      if (rc) return rc;
      RfGdn g = {};
      g.qkv = conv; g.ld = CD;
      g.b = (const uint8_t*)wide + (size_t)(CD + VD) * esz; g.a = (const uint8_t*)wide + (size_t)(CD + VD + BA) * esz;
      g.ld_ba = IN; g.out = attn; g.ldo = VD; g.state = w.gdn_rec_state; g.A_log = w.gdn_A_log; g.dt_bias = w.gdn_dt_bias;
      g.q_start = cv.q_start; g.q_len = cv.q_len; g.slot = f.state_slot; g.fresh = f.state_fresh;
      g.num_seqs = f.num_seqs; g.Hk = c.gdn_Hk; g.Hv = c.gdn_Hv; g.Dk = c.gdn_Dk; g.Dv = c.gdn_Dv; g.dtype = c.dtype;
      // prefill walks 64 tokens per step on the tensor cores; decode and very short inputs take the recurrent kernel
      rc = (!f.decode && f.max_q_len >= gdn_chunk_min()) ? rf_gdn_chunked(&g, st) : rf_gdn_recurrent(&g, st);
      if (rc) return rc;
      // gated RMSNorm over Dv: the conv buffer is free again and takes the result
      rc = rf_rmsnorm_gated(attn, VD, (const uint8_t*)wide + (size_t)CD * esz, IN, w.gdn_norm_w, conv, VD, T, c.gdn_Hv,
                            c.gdn_Dv, c.eps, c.dtype, st);
      if (rc) return rc;
      mix_out = conv;
      mix_dim = VD;
    } else {
    hint_next_weights(s, w.wo, w.so, H, AD, 1, T);
    if (qkv_from_hidden) t_ss_in = ss_mlp;
    if (twin)
      rc = linear_twin(s, xn, H, w.wqkv, w.sqkv, w.bqkv, tw->wqkv, tw->sqkv, tw->bqkv, wide, QD, nullptr, 0, T, split, QD, H,
                       kActNone, 0, st);
    else
      rc = linear(s, qkv_from_hidden ? f.hidden : xn, H, w.wqkv, w.sqkv, w.bqkv, wide, QD, nullptr, 0, T, QD, H, kActNone, 0,
                  false, st);
    if (rc) return rc;
    // twin q/k norm weights that differ from the layer's own: the per-head norm + rope + KV insert runs per row range
    const bool twin_qk = twin && c.qk_norm && tw->q_norm_w && (tw->q_norm_w != w.q_norm_w || tw->k_norm_w != w.k_norm_w);
    for (int part = 0; part < (twin_qk ? 2 : 1); ++part) {
      const int r0 = part == 0 ? 0 : split, rn = twin_qk ? (part == 0 ? split : T - split) : T;
      if (rn <= 0) continue;
      const RfLayerWeights& nw = part == 0 ? w : *tw;
      const int pstride = f.pos_stride > 0 ? f.pos_stride : 1;
      RfRopeKv a = {};
      a.qkv = (uint8_t*)wide + (size_t)r0 * QD * esz; a.ld = QD; a.tokens = rn; a.Hq = c.Hq; a.Hkv = c.Hkv; a.hd = c.hd;
      a.rot_dim = f.cos ? c.rot_dim : 0;
      a.q_norm_w = c.qk_norm ? nw.q_norm_w : nullptr;
      a.k_norm_w = c.qk_norm ? nw.k_norm_w : nullptr;
      a.eps = c.eps; a.norm_mode = c.norm_kind == RF_NORM_RMS_GEMMA ? 1 : 0;
      a.cos = f.cos; a.sin = f.sin; a.pos = f.pos ? f.pos + (size_t)r0 * pstride : nullptr; a.pos_stride = pstride;
      a.axis_of_freq = f.axis_of_freq;
      if (c.paged_kv) {
        a.k_pool = w.k_pool; a.v_pool = w.v_pool; a.page_table = f.page_table; a.pt_stride = f.pt_stride;
        a.seq_of_tok = f.seq_of_tok ? f.seq_of_tok + r0 : nullptr; a.cache_pos = f.cache_pos ? f.cache_pos + r0 : nullptr;
      } else {
        a.write_k_inplace = 1;
      }
      a.rope_before_norm = c.rope_before_norm; a.dtype = c.dtype;
      const bool needed = a.q_norm_w || a.rot_dim > 0 || c.paged_kv;
      if (needed) {
        RF_REQUIRE(f.pos != nullptr, "forward: positions are required");
        rc = rf_qk_norm_rope_kv(&a, st);
        if (rc) return rc;
      }
    }
    {
      RfAttn a = {};
      a.q = wide; a.ldq = QD; a.out = attn; a.ldo = AD; a.q_rows_total = T;
      a.num_seqs = f.num_seqs; a.Hq = c.Hq; a.Hkv = c.Hkv; a.hd = c.hd;
      a.kv_len = f.kv_len; a.max_kv_len = f.max_kv_len; a.max_q_len = f.max_q_len;
      a.scale = c.attn_scale > 0.f ? c.attn_scale : 1.0f / sqrtf((float)(c.true_hd > 0 ? c.true_hd : c.hd));
      a.status = s.status(); a.dtype = c.dtype;
      if (c.paged_kv) {
        a.k_pool = w.k_pool; a.v_pool = w.v_pool; a.pool_pages = f.pool_pages;
        a.page_table = f.page_table; a.pt_stride = f.pt_stride;
      } else {
        a.k = (const uint8_t*)wide + (size_t)c.Hq * c.hd * esz;
        a.v = (const uint8_t*)wide + (size_t)(c.Hq + c.Hkv) * c.hd * esz;
        a.ldk = QD; a.ldv = QD; a.kv_rows_total = T;
        a.kv_start = f.kv_start ? f.kv_start : f.q_start;
      }
      if (f.decode) {
        RF_REQUIRE(c.paged_kv, "decode needs a paged KV pool");
        RF_REQUIRE(c.window <= 0, "decode attention has no sliding-window form: a stack with window=%d would prefill "
                   "with the window and decode over the whole context", c.window);
        a.ws = s.at<float>(s.off_attn_ws); a.ws_bytes = s.attn_ws_bytes;
        rc = rf_attn_decode(&a, st);
      } else {
        a.q_start = f.q_start; a.q_len = f.q_len;
        a.causal = c.causal; a.window = c.window;
        a.mask = f.mask; a.mask_ld = f.mask_ld; a.mask_seq_stride = f.mask_seq_stride;
        a.seg_q = f.seg_q; a.seg_k = f.seg_k;
        rc = rf_attn_prefill(&a, st);
      }
      if (rc) return rc;
      if (c.attn_gate) {
        rc = rf_sigmoid_gate(attn, AD, (const uint8_t*)wide + (size_t)(c.Hq + 2 * c.Hkv) * c.hd * esz, QD, T, AD, c.dtype, st);
        if (rc) return rc;
      }
    }
    }
    // Gated residual with ONE modulation row for all tokens (a single sample's action rows): the gate is a
    // per-column vector, so hidden += gate * sublayer(x) is the GEMM's own epilogue (column scale, then the in-place
    // residual) and the separate gated-residual launch disappears.
    const bool fuse_gate = c.gated_residual && !c.sandwich_norm && f.rows_per_mod >= T && !c.weights_int8 &&
                           c.tp_world == 1 && f.mod != nullptr;
    hint_next_weights(s, w.w_up, w.s_up, s.glu() ? 2 * (int64_t)I : I, H, s.glu() ? 2 : 1, T);
    if (twin) {
      rc = linear_twin(s, mix_out, mix_dim, w.wo, w.so, w.bo, tw->wo, tw->so, tw->bo, f.hidden, H, f.hidden, H, T, split, H,
                       mix_dim, kActNone, 0, st);
      if (rc) return rc;
    } else if (!side) {
      if (fuse_ss) t_ss_out = ss_attn;
      rc = linear_ar(s, mix_out, mix_dim, w.wo, w.so, w.bo, f.hidden, f.hidden, T, mix_dim,
                     norm_rides ? w.norm2_w : nullptr, xn, &have_xn2, st, /*rows_stay=*/true);
      if (rc) return rc;
    } else if (fuse_gate && !w.bo) {
      rc = linear(s, mix_out, mix_dim, w.wo, mod1 + (size_t)2 * H * esz, nullptr, f.hidden, H, f.hidden, H, T, H, mix_dim,
                  kActNone, 0, true, st);
      if (rc) return rc;
    } else {
      rc = linear_ar(s, mix_out, mix_dim, w.wo, w.so, w.bo, tmp, nullptr, T, mix_dim, nullptr, nullptr, nullptr, st);
      if (rc) return rc;
      if (c.sandwich_norm) {
        rc = rf_rmsnorm(tmp, nullptr, w.post_attn_norm_w, tmp, nullptr, nullptr, 1, T, H, H, H, c.eps,
                        c.norm_kind == RF_NORM_RMS_GEMMA ? 1 : 0, c.dtype, st);
        if (rc) return rc;
      }
      if (c.gated_residual) rc = rf_gated_residual(f.hidden, tmp, mod1, f.rows_per_mod, T, H, c.dtype, st);
      else rc = rf_eltwise(0, f.hidden, tmp, f.hidden, (int64_t)T * H, 0, 1.f, c.dtype, st);
      if (rc) return rc;
    }
    // ---- MLP block
    if (twin) {
      rc = norm(s, f.hidden, w.norm2_w, w.norm2_b, xn, split, nullptr, 1, st);
      if (rc == RF_OK && split < T)
        rc = norm(s, (const uint8_t*)f.hidden + split * hrow, tw->norm2_w, tw->norm2_b, (uint8_t*)xn + split * hrow, T - split,
                  nullptr, 1, st);
      if (rc) return rc;
    } else if (!have_xn2 && !fuse_ss) {
      rc = norm(s, f.hidden, folded ? nullptr : w.norm2_w, w.norm2_b, xn, T, mod2, f.rows_per_mod, st);
      if (rc) return rc;
    }
    const bool moe = c.moe_experts > 0 && w.moe_router_w != nullptr;
    void* moe_dense = nullptr;
    if (moe) {
      // router: 16-bit logits -> top-k -> dense [tokens, experts] routing weights (zero where not picked)
      const int E = c.moe_experts, ldE = s.moe_ld();
      auto al = [](uint64_t v) { return (v + 1023) & ~uint64_t(1023); };
      uint8_t* mb = s.at<uint8_t>(s.off_moe);
      void* logits = mb;
      moe_dense = mb + (uint64_t)c.max_tokens * ldE * esz;
      uint8_t* picks = mb + al((uint64_t)c.max_tokens * ldE * esz * 2);
      rc = linear(s, xn, H, w.moe_router_w, nullptr, nullptr, logits, ldE, nullptr, 0, T, E, H, kActNone, 0, false, st);
      if (rc) return rc;
      rc = rf_moe_select(logits, ldE, w.moe_router_bias, T, E, c.moe_top_k, c.moe_score_fn, c.moe_norm_topk,
                         c.moe_routed_scale, reinterpret_cast<int32_t*>(picks),
                         reinterpret_cast<float*>(picks + (uint64_t)c.max_tokens * c.moe_top_k * 4), moe_dense, ldE,
                         c.dtype, st);
      if (rc) return rc;
    }
    hint_next_weights(s, w.w_down, w.s_down, H, I, 1, T);
    if (fuse_ss) t_ss_in = ss_attn;
    if (twin)
      rc = linear_twin(s, xn, H, w.w_up, w.s_up, w.b_up, tw->w_up, tw->s_up, tw->b_up, wide, I, nullptr, 0, T, split, I, H,
                       act_of(c.mlp_kind), s.glu() ? I : 0, st);
    else
      rc = linear(s, fuse_ss ? f.hidden : xn, H, w.w_up, w.s_up, w.b_up, wide, I, nullptr, 0, T, I, H, act_of(c.mlp_kind),
                  s.glu() ? I : 0, false, st);
    if (rc) return rc;
    if (moe) {
      rc = rf_moe_scale_blocks(wide, I, moe_dense, s.moe_ld(), T, c.moe_experts, c.moe_expert_inter, c.dtype, st);
      if (rc) return rc;
    }
    // the next layer's first norm can ride in this all-reduce unless something still changes hidden in between
    const bool hook_after = (f.deepstack && l < f.n_deepstack && f.deepstack[l]);
    const void* next_w = (norm_rides && l + 1 < le && !hook_after) ? s.layers[l + 1].norm1_w : nullptr;
    if (l + 1 < le && s.layers[l + 1].mixer != 1) hint_next_weights(s, s.layers[l + 1].wqkv, s.layers[l + 1].sqkv, QD, H, 1, T);
    if (fuse_ss && l + 1 < le && !hook_after) {
      t_ss_out = ss_mlp;
      ss_ready = true;
    }
    if (twin) {
      rc = linear_twin(s, wide, I, w.w_down, w.s_down, w.b_down, tw->w_down, tw->s_down, tw->b_down, f.hidden, H, f.hidden, H, T,
                       split, H, I, kActNone, 0, st);
      if (rc) return rc;
    } else if (!side) {
      // every rank needs all rows of the stream again after the last layer of this call and where a tap copies them
      bool tapped = false;
      for (int i = 0; i < f.n_taps; ++i) tapped |= f.tap_layers[i] == l;
      rc = linear_ar(s, wide, I, w.w_down, w.s_down, w.b_down, f.hidden, f.hidden, T, I, next_w, xn, &have_xn, st,
                     /*rows_stay=*/next_w != nullptr && !tapped);
      if (rc) return rc;
    } else if (fuse_gate && !w.b_down) {
      rc = linear(s, wide, I, w.w_down, mod2 + (size_t)2 * H * esz, nullptr, f.hidden, H, f.hidden, H, T, H, I, kActNone,
                  0, true, st);
      if (rc) return rc;
    } else {
      rc = linear_ar(s, wide, I, w.w_down, w.s_down, w.b_down, tmp, nullptr, T, I, nullptr, nullptr, nullptr, st);
      if (rc) return rc;
      if (c.sandwich_norm) {
        rc = rf_rmsnorm(tmp, nullptr, w.post_mlp_norm_w, tmp, nullptr, nullptr, 1, T, H, H, H, c.eps,
                        c.norm_kind == RF_NORM_RMS_GEMMA ? 1 : 0, c.dtype, st);
        if (rc) return rc;
      }
      if (c.gated_residual) rc = rf_gated_residual(f.hidden, tmp, mod2, f.rows_per_mod, T, H, c.dtype, st);
      else rc = rf_eltwise(0, f.hidden, tmp, f.hidden, (int64_t)T * H, 0, 1.f, c.dtype, st);
      if (rc) return rc;
    }
    // ---- hooks between layers
    if (f.deepstack && l < f.n_deepstack && f.deepstack[l]) {
      rc = rf_scatter_rows(f.hidden, f.deepstack[l], f.deepstack_rows, f.n_deepstack_rows, H, H, H, 1, c.dtype, st);
      if (rc) return rc;
    }
    for (int i = 0; i < f.n_taps; ++i) {
      if (f.tap_layers[i] == l)
        RF_CUDA_CHECK(cudaMemcpyAsync(f.taps[i], f.hidden, (size_t)T * H * esz, cudaMemcpyDeviceToDevice, st));
    }
  }
  return RF_OK;
}

__global__ void decode_advance_kernel(int32_t* pos, int pos_stride, int32_t* kv_len, int n,
                                      const int32_t* out_ids, int32_t* ids, int32_t* hist, int32_t* step,
                                      int hist_cap) {
  pdl_prologue();
  // single block: n <= 1024 sequences
  const int i = threadIdx.x;
  const int st = step ? *step : 0;
  __syncthreads();
  if (i < n) {
    if (pos) for (int a = 0; a < pos_stride; ++a) pos[i * pos_stride + a] += 1;
    if (kv_len) kv_len[i] += 1;
    if (out_ids) {
      const int t = out_ids[i];
      if (ids) ids[i] = t;
      if (hist && st < hist_cap) hist[(size_t)st * n + i] = t;
    }
  }
  if (i == 0 && step) *step = st + 1;
}

}  // namespace rf

using namespace rf;

extern "C" int64_t rf_stack_create(const RfStackConfig* cfg) {
  if (!cfg) { fail(RF_ERR_BAD_ARG, "null config"); return -1; }
  if (cfg->layers <= 0 || cfg->hidden <= 0 || cfg->hidden % 8 || cfg->Hq <= 0 || cfg->Hkv <= 0 ||
      cfg->Hq % cfg->Hkv || (cfg->hd != 64 && cfg->hd != 128 && cfg->hd != 256) || cfg->inter <= 0 ||
      cfg->inter % 8 || cfg->max_tokens <= 0 || cfg->max_seqs <= 0 || (cfg->dtype != 0 && cfg->dtype != 1) ||
      cfg->tp_world < 1 || cfg->tp_world > 8 || cfg->tp_rank < 0 || cfg->tp_rank >= cfg->tp_world) {
    fail(RF_ERR_BAD_ARG, "invalid stack config (layers=%d hidden=%d Hq=%d Hkv=%d hd=%d inter=%d)", cfg->layers,
         cfg->hidden, cfg->Hq, cfg->Hkv, cfg->hd, cfg->inter);
    return -1;
  }
  if (cfg->moe_experts > 0 &&
      (cfg->moe_top_k < 1 || cfg->moe_top_k > cfg->moe_experts || cfg->moe_expert_inter <= 0 ||
       (int64_t)cfg->moe_experts * cfg->moe_expert_inter > cfg->inter || cfg->weights_int8)) {
    fail(RF_ERR_BAD_ARG, "invalid MoE config (experts=%d top_k=%d expert_inter=%d inter=%d int8=%d)", cfg->moe_experts,
         cfg->moe_top_k, cfg->moe_expert_inter, cfg->inter, cfg->weights_int8);
    return -1;
  }
  auto s = std::make_unique<Stack>();
  s->cfg = *cfg;
  s->layers.resize(cfg->layers);
  s->plan();
  return registry().insert(std::move(s));
}

extern "C" int rf_stack_destroy(int64_t h) {
  return registry().erase(h) ? RF_OK : fail(RF_ERR_BAD_ARG, "unknown stack handle %lld", (long long)h);
}

#define RF_GET_STACK(h)                                                              \
  std::shared_ptr<Stack> sp = registry().get(h);                                     \
  if (!sp) return fail(RF_ERR_BAD_ARG, "unknown stack handle %lld", (long long)(h)); \
  Stack& s = *sp;

extern "C" int rf_stack_set_layer(int64_t h, int32_t layer, const RfLayerWeights* w) {
  RF_GET_STACK(h);
  RF_REQUIRE(w && layer >= 0 && layer < s.cfg.layers, "layer index %d out of range", layer);
  RF_REQUIRE(w->wqkv && w->wo && w->w_up && w->w_down, "layer %d: missing projection weights", layer);
  if (s.cfg.paged_kv && w->mixer == 0) RF_REQUIRE(w->k_pool && w->v_pool, "layer %d: missing KV pool", layer);
  if (w->mixer == 1)
    RF_REQUIRE(s.cfg.gdn_Hv > 0 && w->gdn_conv_w && w->gdn_A_log && w->gdn_dt_bias && w->gdn_norm_w && w->gdn_conv_state &&
                   w->gdn_rec_state, "layer %d: incomplete Gated-DeltaNet weight set", layer);
  if (s.cfg.weights_int8) RF_REQUIRE(w->sqkv && w->so && w->s_up && w->s_down, "layer %d: int8 weights need scales", layer);
  s.layers[layer] = *w;
  return RF_OK;
}

extern "C" int rf_stack_set_twin_layer(int64_t h, int32_t layer, const RfLayerWeights* w) {
  RF_GET_STACK(h);
  RF_REQUIRE(w && layer >= 0 && layer < s.cfg.layers, "twin layer index %d out of range", layer);
  RF_REQUIRE(w->wqkv && w->wo && w->w_up && w->w_down, "twin layer %d: missing projection weights", layer);
  RF_REQUIRE(w->mixer == 0 && s.cfg.tp_world == 1 && s.cfg.moe_experts == 0 && !s.cfg.norm_folded && !s.cfg.gated_residual &&
                 !s.cfg.sandwich_norm,
             "twin weights are for dense attention layers of a plain pre-norm stack on one GPU");
  if (s.cfg.weights_int8) RF_REQUIRE(w->sqkv && w->so && w->s_up && w->s_down, "twin layer %d: int8 weights need scales", layer);
  if (s.twins.size() != s.layers.size()) s.twins.assign(s.layers.size(), RfLayerWeights{});
  s.twins[layer] = *w;
  return RF_OK;
}

extern "C" int rf_stack_set_twin_head(int64_t h, const void* final_norm_w) {
  RF_GET_STACK(h);
  s.twin_final_norm_w = final_norm_w;
  return RF_OK;
}

extern "C" int rf_stack_set_kv(int64_t h, int32_t layer, void* k_pool, void* v_pool) {
  RF_GET_STACK(h);
  RF_REQUIRE(layer >= 0 && layer < s.cfg.layers && k_pool && v_pool, "set_kv: layer %d", layer);
  s.layers[layer].k_pool = k_pool;
  s.layers[layer].v_pool = v_pool;
  return RF_OK;
}

extern "C" int rf_stack_set_state(int64_t h, int32_t layer, void* conv_state, float* rec_state) {
  RF_GET_STACK(h);
  RF_REQUIRE(layer >= 0 && layer < s.cfg.layers && conv_state && rec_state, "set_state: layer %d", layer);
  s.layers[layer].gdn_conv_state = conv_state;
  s.layers[layer].gdn_rec_state = rec_state;
  return RF_OK;
}

extern "C" int rf_stack_set_head(int64_t h, const void* final_norm_w, const void* final_norm_b,
                                 const void* w_lm, const void* s_lm) {
  RF_GET_STACK(h);
  s.final_norm_w = final_norm_w; s.final_norm_b = final_norm_b; s.w_lm = w_lm; s.s_lm = s_lm;
  return RF_OK;
}

extern "C" int rf_stack_set_comm(int64_t h, const RfStackComm* c) {
  RF_GET_STACK(h);
  RF_REQUIRE(c && c->recv && c->flags && c->state, "comm buffers");
  s.comm = *c;
  s.has_comm = true;
  return RF_OK;
}

extern "C" uint64_t rf_stack_arena_bytes(int64_t h) {
  std::shared_ptr<Stack> sp = registry().get(h);
  return sp ? sp->total : 0;
}

extern "C" int rf_stack_bind_arena(int64_t h, void* base, uint64_t bytes) {
  RF_GET_STACK(h);
  RF_REQUIRE(base && bytes >= s.total, "arena of %llu B is smaller than the plan (%llu B)",
             (unsigned long long)bytes, (unsigned long long)s.total);
  RF_REQUIRE((reinterpret_cast<uintptr_t>(base) & 1023) == 0, "arena base must be 1024-byte aligned");
  s.base = static_cast<uint8_t*>(base);
  s.bytes = bytes;
  return RF_OK;
}

extern "C" int32_t* rf_stack_status_ptr(int64_t h) {
  std::shared_ptr<Stack> sp = registry().get(h);
  return sp ? sp->status() : nullptr;
}

extern "C" int rf_stack_forward(int64_t h, const RfStackForward* f, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_GET_STACK(h);
  RF_REQUIRE(f != nullptr, "null forward args");
  return forward(s, *f, static_cast<cudaStream_t>(stream));
}

extern "C" int rf_stack_final_norm(int64_t h, const void* hidden, void* out, int32_t rows, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_GET_STACK(h);
  RF_REQUIRE(s.final_norm_w, "stack has no final norm");
  RfStackConfig c = s.cfg;
  Stack tmp = s;
  if (c.norm_kind == RF_NORM_ADARMS) tmp.cfg.norm_kind = RF_NORM_RMS;
  return norm(tmp, hidden, s.final_norm_w, s.final_norm_b, out, rows, nullptr, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int rf_stack_final_norm_twin(int64_t h, const void* hidden, void* out, int32_t rows, int32_t twin_split,
                                        rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_GET_STACK(h);
  RF_REQUIRE(s.final_norm_w && s.twin_final_norm_w, "stack has no twin final norm");
  RF_REQUIRE(twin_split >= 0 && twin_split <= rows, "twin_split %d outside [0, %d]", twin_split, rows);
  Stack tmp = s;
  if (s.cfg.norm_kind == RF_NORM_ADARMS) tmp.cfg.norm_kind = RF_NORM_RMS;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t row_bytes = (size_t)s.cfg.hidden * 2;
  int rc = RF_OK;
  if (twin_split > 0) rc = norm(tmp, hidden, s.final_norm_w, s.final_norm_b, out, twin_split, nullptr, 1, st);
  if (rc == RF_OK && twin_split < rows)
    rc = norm(tmp, (const uint8_t*)hidden + twin_split * row_bytes, s.twin_final_norm_w, nullptr,
              (uint8_t*)out + twin_split * row_bytes, rows - twin_split, nullptr, 1, st);
  return rc;
}

extern "C" int rf_stack_head(int64_t h, const void* hidden, const int32_t* row_idx, int32_t rows,
                             int32_t* out_ids, float* out_vals, void* logits_out, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_GET_STACK(h);
  const RfStackConfig& c = s.cfg;
  RF_REQUIRE(s.base && s.final_norm_w && s.w_lm && c.vocab_local > 0, "stack has no lm head");
  RF_REQUIRE(rows > 0 && rows <= c.max_seqs, "head rows %d (max %d)", rows, c.max_seqs);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int H = c.hidden;
  void* hx = s.at(s.off_head_xn);
  const void* src = hidden;
  int rc;
  if (row_idx) {
    // gather the selected rows (embedding gather on the hidden matrix)
    rc = rf_embedding(hidden, row_idx, s.at(s.off_tmp), rows, H, H, 1.f, c.dtype, nullptr, st);
    if (rc) return rc;
    src = s.at(s.off_tmp);
  }
  Stack tmp = s;
  if (c.norm_kind == RF_NORM_ADARMS) tmp.cfg.norm_kind = RF_NORM_RMS;
  rc = norm(tmp, src, s.final_norm_w, s.final_norm_b, hx, rows, nullptr, 1, st);
  if (rc) return rc;
  void* logits = logits_out ? logits_out : s.at(s.off_logits);
  rc = linear(s, hx, H, s.w_lm, s.s_lm, nullptr, logits, c.vocab_local, nullptr, 0, rows, c.vocab_local, H,
              kActNone, 0, false, st);
  if (rc) return rc;
  if (out_ids)
    rc = rf_argmax(logits, rows, c.vocab_local, c.vocab_local, out_ids, out_vals, c.vocab_offset,
                   s.at(s.off_argmax), s.argmax_bytes, c.dtype, st);
  return rc;
}

extern "C" int rf_decode_advance(int32_t* pos, int32_t pos_stride, int32_t* kv_len, int32_t n,
                                 const int32_t* out_ids, int32_t* ids, int32_t* hist, int32_t* step,
                                 int32_t hist_cap, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  if (n <= 0) return RF_OK;
  RF_REQUIRE(n <= 1024, "decode_advance handles up to 1024 sequences, got %d", n);
  RF_CUDA_CHECK(::rf::launch_k(decode_advance_kernel, dim3(1), dim3(((n + 31) / 32) * 32), 0, static_cast<cudaStream_t>(stream), 1, 
      pos, pos_stride > 0 ? pos_stride : 1, kv_len, n, out_ids, ids, hist, step, hist_cap));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}

// sizeof of every argument block, in the order the Python binding checks them
extern "C" void rf_struct_sizes(int32_t* out) {
  out[0] = (int32_t)sizeof(RfGemm); out[1] = (int32_t)sizeof(RfRopeKv); out[2] = (int32_t)sizeof(RfAttn);
  out[3] = (int32_t)sizeof(RfStackConfig); out[4] = (int32_t)sizeof(RfLayerWeights);
  out[5] = (int32_t)sizeof(RfStackComm); out[6] = (int32_t)sizeof(RfStackForward); out[7] = 0;
  out[8] = (int32_t)sizeof(RfConv1d); out[9] = (int32_t)sizeof(RfGdn); out[10] = (int32_t)sizeof(RfArConsume);
}
