// C ABI of librf_b200: every entry point takes raw device pointers and a CUDA
// stream, allocates nothing unless its comment says so, and returns 0 on
// success or a negative RfError.  Python binds these through ctypes.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* rf_stream_t;  // cudaStream_t

enum RfError {
  RF_OK = 0,
  RF_ERR_BAD_ARG = -1,
  RF_ERR_CUDA = -2,
  RF_ERR_UNSUPPORTED = -3,
  RF_ERR_NO_MEMORY = -4,
  RF_ERR_STATE = -5,
};

const char* rf_last_error(void);
int rf_version(void);
uint64_t rf_launch_count(void);  // kernels enqueued by this library so far

// ---------------------------------------------------------------- GEMM ----
// out[M,N] = epilogue( x[M,K] . w[N,K]^T ), all row-major, 16-bit in, fp32 acc.
typedef struct RfGemm {
  const void* x; int64_t ldx;
  const void* w; int64_t ldw;
  void* out; int64_t ldo;
  const void* residual; int64_t ldr;  // optional, added last
  const void* bias;                   // optional [N] (dual: [dual_offset+N])
  const void* scale;                  // optional per-output-channel scale [N], same dtype
  const float* row_scale;             // optional per-token fp32 scale [M]
  int32_t M, N, K;
  int32_t dtype;        // 0 fp16, 1 bf16
  int32_t act;          // rf::Act
  int32_t dual_offset;  // >0: second weight block starts dual_offset rows below the first
  int32_t w_int8;       // 1: w is int8 [N,K] (scale required)
  float* ws; uint64_t ws_bytes;  // split-K scratch (fp32 partials), optional
  uint32_t* sem; int32_t sem_count;  // split-K tile semaphores, zero-initialised once
  int32_t* status;      // device status block, optional
  // fused all-reduce over peer memory (world > 1): partial tiles are pushed
  // into every rank's receive buffer, summed in rank order, residual added.
  int32_t ar_world, ar_rank;
  void* const* ar_recv;        // device array [world] of receive-buffer bases
  uint32_t* const* ar_flags;   // device array [world] of flag-array bases
  uint32_t* ar_state;          // local: [0] call counter, [1] finished-CTA counter
  uint64_t ar_recv_bytes;      // bytes of one half of the (double-buffered) receive buffer
  int32_t ar_flag_count;       // flags available per rank
  int32_t force_splits;        // 0 = heuristic
  int32_t force_swap;          // -1 = heuristic, 0/1 forced
  int32_t force_bn;            // 0 = heuristic
  // 1: w is in the tile-major layout (see rf_pack_weight_bytes): block (row tile rt, k block kb) of
  // 128 rows x 64 columns is contiguous, 16-bit blocks already in the 128-byte-swizzled shared-memory
  // image, so one 16 KB (int8: 8 KB) bulk copy per block streams HBM pages front to back.  Rows are
  // padded to 128 per section (dual: gate section, then up section), K to 64; ldw is ignored.
  int32_t w_packed;
  // W8A16 with more than 256 tokens: device scratch for the widened (16-bit, tile-major) weight image, twice
  // the bytes of the int8 image.  Null: the int8 tile is widened inside the main loop for every token count.
  void* w_scratch;
  uint64_t w_scratch_bytes;
  // Tensor parallel, at most 256 tokens: 1 = "publish and exit".  The epilogue only pushes this rank's partial
  // rows (16-byte vectors) into every rank's receive buffer and bumps counter ar_cnt_base + ar_rank on every rank;
  // it does not wait, reduce, add the residual or write `out`.  rf_ar_consume() finishes the all-reduce.
  int32_t ar_publish;
  int32_t ar_cnt_base;         // first of `world` arrival counters in every rank's flag array
  // Optional hint (weight-streaming shapes of at most 256 tokens): device memory the NEXT kernel on the stream will
  // read - normally the next linear layer's weights.  Once a CTA has issued its own last weight load it asks for its
  // share of the first prefetch_bytes of that memory to be brought into L2, so HBM keeps streaming through this
  // kernel's epilogue, the launch gap and the next kernel's prologue.  Never dereferenced; 16-byte aligned.
  const void* prefetch;
  uint64_t prefetch_bytes;
  // 4: `w` is the tile-major int4 image made by rf_pack_w4 / ops.kernels.pack_weight_int4 (w_int8 = 1, w_packed = 1):
  // block (row tile, k block) = 128 rows x 64 columns as 4096 bytes of nibbles (two's complement; inside each group of
  // eight columns the nibbles sit in the order 0,2,4,6,1,3,5,7) followed by the block's scales in the activation dtype,
  // 128 x (64 / min(w_group, 64)) of them.  w_group = 0: no scales in the image, `scale` holds one per output channel.
  int32_t w_bits;
  int32_t w_group;     // 0, 16 (fp4 only), 32, 64 or 128 columns per scale
  // 0: the nibbles are two's-complement integers (W4A16); 1: e2m1 floating-point codes (bit 3 sign, bits 0..2 index into
  // {0, 0.5, 1, 1.5, 2, 3, 4, 6}) as in NVFP4, whose e4m3 block scale times the tensor scale is stored per 16 columns
  // in the image, already multiplied out in the activation dtype.
  int32_t w_fp4;
  // RMSNorm folded around the GEMMs (at most 256 tokens, weights streamed with tokens on the MMA N axis):
  //  * ss_out: this GEMM also writes, for every token and every 128-wide tile of its output columns, the sum of
  //    squares of the finished (residual added, rounded) values: ss_out[tile * ss_ld + token], fp32.  Plain stores in
  //    a fixed layout, so the later sum has a fixed order.
  //  * ss_in: the input rows are un-normalised; the result is scaled per token by
  //    rsqrt(sum_{t < ss_tiles} ss_in[t * ss_ld + token] / ss_dim + ss_eps), which together with norm weights
  //    multiplied into the weight columns beforehand is the RMSNorm that would otherwise run as its own kernel.
  int32_t ss_tiles;
  float* ss_out;
  const float* ss_in;
  int32_t ss_ld, ss_dim;
  float ss_eps;
  int32_t streaming_only;      // 1: never the latency-bound mma.sync kernel (gemm_small.cu), whatever the shape
} RfGemm;
// bytes of the tile-major image of a [rows, K] weight with `sections` equal row sections
uint64_t rf_pack_weight_bytes(int64_t rows, int64_t K, int32_t sections, int32_t elem_bytes);
// bytes of the tile-major int4 image (see RfGemm.w_bits) and of one of its blocks
uint64_t rf_pack_w4_bytes(int64_t rows, int64_t K, int32_t sections, int32_t group);
int32_t rf_w4_block_bytes(int32_t group);

int rf_gemm(const RfGemm* g, rf_stream_t stream);
// Launch plan of a shape without launching: out[10] = {swap, bn, splits, stages, grid_x, grid_y, smem bytes, k_blocks,
// persistent kernel, two-shot all-reduce}.  Host-only.
int rf_gemm_plan_info(const RfGemm* g, int32_t* out);
// Scratch a split-K launch of this shape would need (bytes of ws, number of sems).
int rf_gemm_scratch(const RfGemm* g, uint64_t* ws_bytes, int32_t* sem_count);
// Same contract with int8 weights [N,K] and a per-output-channel scale (W8A16):
// the int8 tile is widened to the activation dtype inside the mainloop.
int rf_gemm_w8a16(const RfGemm* g, rf_stream_t stream);
// int4 weights (w_bits = 4) with per-channel or group-wise scales: nibbles are widened, and group scales applied, by the
// converter warps of the same main loop.
int rf_gemm_w4a16(const RfGemm* g, rf_stream_t stream);
// CUDA-core skinny GEMM (M <= 8): reference path and small-batch decode.
int rf_gemv(const RfGemm* g, rf_stream_t stream);
// CTAs of the launch rf_gemm / rf_gemm_w8a16 would make for this shape (each bumps the arrival counters once when
// ar_publish is set); negative RfError on a bad shape.  Host-only.
int rf_gemm_grid_ctas(const RfGemm* g);

// Second half of the tensor-parallel all-reduce of a row-parallel GEMM launched with ar_publish: waits (bounded)
// until every rank's arrival counter shows that all `pub_ctas` CTAs of its GEMM have published, sums the ranks'
// partial rows in rank order in fp32, adds the residual, writes `out`, and optionally applies the RMSNorm that
// follows in the layer (norm_mode 1: w * norm(x), 2: (1 + w) * norm(x)) into norm_out.  out may alias residual.
// Partials are fp32 up to RF_AR_F32_MAX_ROWS rows and the activation dtype above.
#define RF_AR_F32_MAX_ROWS 16
typedef struct RfArConsume {
  int32_t M, N;                // rows (tokens) and columns (hidden size); N a multiple of 8
  int32_t world, rank;
  void* const* ar_recv;        // device array [world] of receive-buffer bases (only [rank] is read here)
  uint32_t* const* ar_flags;   // device array [world] of flag-array bases (only [rank] is read here)
  uint32_t* ar_state;          // local state words: [0] call counter, [4] counter value consumed so far, [5] finished CTAs
  uint64_t ar_recv_bytes;      // bytes of one half of the double-buffered receive buffer
  int32_t ar_cnt_base;
  int32_t pub_ctas;            // rf_gemm_grid_ctas() of the producing GEMM
  const void* residual; int64_t ldr;   // optional
  void* out; int64_t ldo;
  const void* norm_w; void* norm_out; int64_t ldn;   // optional fused RMSNorm of the finished rows
  float eps; int32_t norm_mode;
  int32_t* status; int32_t dtype;
} RfArConsume;
int rf_ar_consume(const RfArConsume* a, rf_stream_t stream);

// Two-shot all-reduce for large token counts (prefill), over buffers that every rank allocated at the same offsets
// of its peer-mapped communication region ("symmetric" buffers; the tables hold one base pointer per rank).
// Every rank's row-parallel GEMM has written its partial result [M, N] into its own `partial` buffer.  Rank r owns
// rows [r * ceil(M / world), ...): it reads those rows of EVERY rank's partial over NVLink (reduce-scatter by peer
// loads, summed in rank order in fp32), adds the residual, and writes the finished rows -- and, when norm_mode != 0,
// the RMSNorm of them -- into every rank's `out` (and `norm_out`) buffer (all-gather by peer stores).  The residual is
// read from this rank's own `out` buffer when add_residual is set (the residual stream lives there).  With out_local
// the finished rows are written on their owner only: each rank then holds M / world rows of the residual stream, and
// what crosses NVLink is a reduce-scatter of the partials plus an all-gather of the normalised rows.  Flags:
// world "partial ready" + world "rows written" words per rank at flag_base; state word 6 is the epoch.
typedef struct RfArRows {
  int32_t M, N, world, rank;
  void* const* partial_tab;    // device array [world]: every rank's partial [M, N]
  void* const* out_tab;        // device array [world]: every rank's destination [M, N]
  void* const* norm_tab;       // device array [world]: every rank's normalised destination (optional)
  uint32_t* const* ar_flags;   // device array [world] of flag-array bases
  uint32_t* ar_state;
  int32_t flag_base;
  int32_t add_residual;
  const void* norm_w; float eps; int32_t norm_mode;
  int32_t* status; int32_t dtype;
  int32_t out_local;           // 1: the finished rows stay on their owner (sequence-sharded residual stream); only the
                               // normalised rows are gathered on every rank
} RfArRows;
int rf_ar_rows(const RfArRows* a, rf_stream_t stream);


// ------------------------------------------------------ norms / glue ----
int rf_rmsnorm(const void* x, const void* residual, const void* w, void* y, void* residual_out,
               const void* mod, int rows_per_mod, int rows, int H, int64_t ldx, int64_t ldy,
               float eps, int mode, int dtype, rf_stream_t stream);
int rf_layernorm(const void* x, const void* w, const void* b, void* y, int rows, int H,
                 int64_t ldx, int64_t ldy, float eps, int dtype, rf_stream_t stream);
int rf_l2norm(const void* x, void* y, int rows, int H, float eps, float out_scale, int dtype,
              rf_stream_t stream);
int rf_gated_residual(void* x, const void* y, const void* mod, int rows_per_mod, int rows, int H,
                      int dtype, rf_stream_t stream);

// Per-head RMSNorm(q,k) -> RoPE -> KV page insert on a packed [tokens, (Hq+2Hkv)*hd] buffer.
typedef struct RfRopeKv {
  void* qkv; int64_t ld;
  void* q_out; int64_t ldq;        // optional: rotated q goes here instead of in place
  int32_t tokens, Hq, Hkv, hd, rot_dim;
  const void* q_norm_w; const void* k_norm_w;  // optional [hd]
  float eps; int32_t norm_mode;     // bit0: (1+w) weight
  const float* cos; const float* sin;  // [max_pos, rot_dim/2] fp32, optional
  const int32_t* pos; int32_t pos_stride;  // [tokens, pos_stride]
  const int8_t* axis_of_freq;       // optional [rot_dim/2]: which position axis a frequency uses
  void* k_pool; void* v_pool;       // optional [pages, Hkv, 16, hd]
  const int32_t* page_table; int32_t pt_stride;  // [seqs, pt_stride]
  const int32_t* seq_of_tok;        // optional [tokens]; default token index
  const int32_t* cache_pos;         // optional [tokens]; default pos[tok, 0]
  int32_t rope_before_norm;
  int32_t write_k_inplace;          // also write rotated k back into qkv
  int32_t dtype;
  int32_t v_norm;                   // unweighted RMSNorm of every value head (in place, before the cache insert)
} RfRopeKv;
int rf_qk_norm_rope_kv(const RfRopeKv* a, rf_stream_t stream);

// out[i] = table[ids[i]] (row gather); ids < 0 give zero rows.  scale multiplies (Gemma sqrt(H)).
int rf_embedding(const void* table, const int32_t* ids, void* out, int n_ids, int H, int64_t ldo,
                 float scale, int dtype, const void* row_scale_i8, rf_stream_t stream);
// dst[rows[i]] = src[i]  (splice vision rows into text rows)
int rf_scatter_rows(void* dst, const void* src, const int32_t* rows, int n, int H, int64_t ldd,
                    int64_t lds, int accumulate, int dtype, rf_stream_t stream);
// Elementwise: op 0 add, 1 mul, 2 silu(a)*b, 3 gelu_tanh(a)*b, 4 a + alpha*b, 5 gelu_tanh(a),
// 6 gelu_erf(a), 7 silu(a), 8 a*alpha, 9 sigmoid(a)*b, 10 a*(broadcast row vector b), 11 tanh(a)
int rf_eltwise(int op, const void* a, const void* b, void* out, int64_t n, int64_t b_period,
               float alpha, int dtype, rf_stream_t stream);
int rf_cast_u8_f16(const uint8_t* src, void* dst, int64_t n, float scale, float shift, int dtype,
                   rf_stream_t stream);
// Greedy top-1 over the last dim; two-stage, writes int32 ids (and fp32 max when vals != null).
// offset is added to every id (vocab shard base).
int rf_argmax(const void* logits, int rows, int V, int64_t ld, int32_t* out_ids, float* out_vals,
              int32_t offset, void* scratch, uint64_t scratch_bytes, int dtype, rf_stream_t stream);
uint64_t rf_argmax_scratch_bytes(int rows, int V);


// ----------------------------------------------------------- attention ----
// q/out: [q_rows_total, Hq*hd] (pitch ldq/ldo).  KV comes either from the paged
// pool ([pages, Hkv, 16, hd], page_table[seq, i] -> page id) or from contiguous
// rows k/v[kv_rows_total, Hkv*hd].  The pool must only ever hold finite values
// (it is zero-filled at creation): masked tokens still pass through the MMA.
typedef struct RfAttn {
  const void* q; int64_t ldq;
  void* out; int64_t ldo;
  int64_t q_rows_total;
  const void* k_pool; const void* v_pool; int64_t pool_pages;
  const int32_t* page_table; int32_t pt_stride;
  const void* k; const void* v; int64_t ldk, ldv; int64_t kv_rows_total;
  int32_t num_seqs, Hq, Hkv, hd;
  const int32_t* q_start;   // [num_seqs] first q row (prefill)
  const int32_t* q_len;     // [num_seqs] (prefill)
  const int32_t* kv_start;  // [num_seqs] first kv row (contiguous mode)
  const int32_t* kv_len;    // [num_seqs] valid kv tokens, device
  int32_t max_q_len, max_kv_len;  // host-side bounds used for grid sizing
  int32_t causal;           // q row i sits at position kv_len - q_len + i
  int32_t window;           // > 0: sliding window
  const uint8_t* mask; int64_t mask_ld, mask_seq_stride;  // optional boolean [q, kv] per sequence
  const int32_t* seg_q; const int32_t* seg_k;             // optional segment ids per q row / kv row
  float scale;              // <= 0: 1/sqrt(hd)
  float* ws; uint64_t ws_bytes;  // decode split-KV scratch, optional
  int32_t* status; int32_t dtype;
} RfAttn;
int rf_attn_prefill(const RfAttn* a, rf_stream_t stream);
int rf_attn_decode(const RfAttn* a, rf_stream_t stream);
uint64_t rf_attn_decode_scratch_bytes(int num_seqs, int Hq, int hd);


// --------------------------------------------- linear attention (GDN) ----
// Causal depthwise conv1d (kernel size 4) + optional SiLU over C channels of packed varlen rows,
// with a carried state [slots, K-1, C] (oldest row first) that is read, then replaced by the last
// K-1 inputs of every sequence.  q_start/q_len null: one token per sequence (decode), row = seq.
// x and y must not alias.
typedef struct RfConv1d {
  const void* x; int64_t ldx;
  void* y; int64_t ldy;
  const void* w;            // [C, K]
  void* state;              // [slots, K-1, C]
  const int32_t* q_start; const int32_t* q_len; const int32_t* slot;   // device, [num_seqs]; slot null: seq
  int32_t num_seqs, max_q_len, C, K, silu, dtype;
} RfConv1d;
int rf_causal_conv1d(const RfConv1d* a, rf_stream_t stream);

// Gated delta rule over n tokens per sequence (n = 1: decode step):
//   beta = sigmoid(b), g = -exp(A_log) * softplus(a + dt_bias), q,k L2-normalised, q /= sqrt(Dk)
//   S *= exp(g);  kv = k^T S;  d = (v - kv) * beta;  S += k (x) d;  o = q^T S
// qkv rows hold [q: Hk*Dk | k: Hk*Dk | v: Hv*Dv]; value head h reads key head h / (Hv/Hk).
// state: fp32 [slots, Hv, Dk, Dv]; fresh[seq] != 0 starts that sequence from a zero state.
typedef struct RfGdn {
  const void* qkv; int64_t ld;
  const void* b; const void* a; int64_t ld_ba;     // [rows, >= Hv] each
  void* out; int64_t ldo;                           // [rows, Hv*Dv]
  float* state;
  const float* A_log; const float* dt_bias;         // [Hv] fp32
  const int32_t* q_start; const int32_t* q_len; const int32_t* slot; const int32_t* fresh;
  int32_t num_seqs, Hk, Hv, Dk, Dv, dtype;
} RfGdn;
int rf_gdn_recurrent(const RfGdn* a, rf_stream_t stream);
// Same contract, evaluated 64 tokens at a time on the tensor cores (prefill; decode keeps the recurrent kernel).
int rf_gdn_chunked(const RfGdn* a, rf_stream_t stream);
// y[t, h, :] = (w * rmsnorm(x[t, h, :])) * silu(z[t, h, :]), D values per (token, head)
int rf_rmsnorm_gated(const void* x, int64_t ldx, const void* z, int64_t ldz, const void* w, void* y, int64_t ldy,
                     int tokens, int heads, int D, float eps, int dtype, rf_stream_t stream);
// a[t, c] *= sigmoid(g[t, c]) (output gate of the gated full-attention layers)
int rf_sigmoid_gate(void* a, int64_t lda, const void* g, int64_t ldg, int rows, int cols, int dtype, rf_stream_t stream);
// helpers of the chunked delta-rule formulation
int rf_cumsum_f32(const float* x, float* y, int rows, int n, rf_stream_t stream);
int rf_unit_tril_inv_f32(const float* m, float* out, int batch, int n, rf_stream_t stream);


// ------------------------------------------------- mixture of experts ----
// Router: scores = sigmoid(logits) (score_fn 0) or softmax(logits) (1); the k experts with the largest
// (score + bias) are selected, ties to the lower index; weights are the UNBIASED scores, divided by their
// sum when norm_topk, times scale.  Any of out_ids [rows,k], out_w [rows,k], dense_w [rows,E] (zero for
// unselected experts) may be null.  E <= 256, k <= 32.
int rf_moe_select(const void* logits, int64_t ld, const float* bias, int rows, int E, int k, int score_fn,
                  int norm_topk, float scale, int32_t* out_ids, float* out_w, void* dense_w, int64_t ldd, int dtype,
                  rf_stream_t stream);
// h[t, e*I + c] *= dense_w[t, e] for the E routed expert blocks of width I (dense-einsum expert MLP)
int rf_moe_scale_blocks(void* h, int64_t ldh, const void* dense_w, int64_t ldd, int rows, int E, int I, int dtype,
                        rf_stream_t stream);


// Grouped expert GEMM.  The (token, pick) pairs of a batch are bucketed by expert (rf_moe_group), their rows are
// gathered in that order, and ONE persistent launch multiplies every 128-row block of one expert's rows with that
// expert's weights out of the packed expert bank: out[s, :] = act(x[s, :] . W_e^T) (* row_scale[s]) for every sorted
// row s of expert e.  Only the experts that were picked are read, and only for as many row blocks as they have rows.
//   up / gate projections: the bank stacks the experts along N (rt_per_expert row tiles apart, kb_per_expert = 0);
//   down projection:       the bank concatenates the experts along K (kb_per_expert k blocks apart, rt_per_expert = 0).
typedef struct RfMoeGroupedGemm {
  const void* x; int64_t ldx;          // sorted rows [max_rows, K]
  const void* w;                       // tile-major image of the whole expert bank (rf_pack_weight_bytes layout)
  void* out; int64_t ldo;              // [max_rows, N]
  const float* row_scale;              // optional [max_rows] (routing weight of the row)
  const int32_t* tiles;                // device: [0] number of row blocks, then {expert, first row, end row, 0} per block
  int32_t max_rows, N, K;              // upper bound of sorted rows; per-expert GEMM shape
  int32_t dual, act;                   // dual = 1: GLU pair (gate section, then up section of the bank)
  int32_t bank_section_row_tiles;      // 128-row tiles of one section of the bank image
  int32_t bank_kb_total;               // 64-column k blocks of one row tile of the bank image
  int32_t rt_per_expert, kb_per_expert;
  int32_t dtype; int32_t* status;
} RfMoeGroupedGemm;
int rf_moe_grouped_gemm(const RfMoeGroupedGemm* a, rf_stream_t stream);
// Bucket the picks by expert.  ids / w: [rows, k] (rf_moe_select).  Outputs (device): slot_of [rows*k] = sorted row
// of pick (t, j); token_of_slot [rows*k]; slot_w [rows*k] (fp32 routing weight per sorted row); tiles = the list
// rf_moe_grouped_gemm takes (1 + 4 * (rows*k/128 + E) int32).  One CTA; rows * k <= 1 << 20, E <= 256.
int rf_moe_group(const int32_t* ids, const float* w, int rows, int k, int E, int32_t* slot_of, int32_t* token_of_slot,
                 float* slot_w, int32_t* tiles, rf_stream_t stream);
// out[t, :] += sum_j y[slot_of[t, j], :]  (fp32, picks in order j = 0..k-1, one rounding)
int rf_moe_combine(void* out, int64_t ldo, const void* y, int64_t ldy, const int32_t* slot_of, int rows, int k, int H,
                   int dtype, rf_stream_t stream);


// ------------------------------------------------------------- KV pool ----
int64_t rf_kvpool_create(int32_t num_pages, int32_t max_seqs, int32_t pages_per_seq);
int rf_kvpool_destroy(int64_t h);
int rf_kvpool_reserve(int64_t h, int32_t seq, int32_t tokens, int32_t* table_row);
int rf_kvpool_release(int64_t h, int32_t seq);
int32_t rf_kvpool_free_pages(int64_t h);


// ------------------------------------------------ peer memory (TP) ----
int rf_comm_alloc(uint64_t bytes, void** out);   // cudaMalloc + zero fill
int rf_comm_free(void* p);
int rf_ipc_export(void* p, uint8_t* handle64);
int rf_ipc_import(const uint8_t* handle64, void** out);
int rf_ipc_close(void* p);
int rf_tp_argmax_merge(void* const* aux, uint32_t* const* flags, int flag_base, uint32_t* state, int world,
                       int rank, int rows, int max_rows, const float* vals, int32_t* ids, int32_t* status,
                       rf_stream_t stream);
int rf_peer_barrier(uint32_t* const* flags, int flag_base, uint32_t* state, int world, int rank,
                    int32_t* status, rf_stream_t stream);

#ifdef __cplusplus
}
#endif
