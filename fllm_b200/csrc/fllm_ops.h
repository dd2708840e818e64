// Launcher declarations of the sm_100a kernels. Everything takes raw device
// pointers and a stream, so the kernels can be driven from the torch bindings,
// from the C ABI and from stream capture alike. Leading dimensions are in elements.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace fllm {

// ---- dense bf16 GEMM (tcgen05) ------------------------------------------------------
// Optional behaviour of one linear call.
//   glu            gated activation inside the epilogue (y is then [T][N / 2]): 1 SwiGLU, 2 GeGLU (tanh),
//                  3 clamped SwiGLU-OAI. The weight rows must interleave gate and up rows: blocks of 16
//                  (glu_pd = 16: rows 32j..32j+15 gate, 32j+16..32j+31 up of features 16j..16j+15) or pairs
//                  (glu_pd = 1: row 2i gate, 2i+1 up).
//   defer_reduce   when the call picks split-K, skip its reduction kernel and leave the fp32 partial sums
//                  [splits][T][N] (bias NOT added) at workspace + kLinearPartialsOffset; the consumer
//                  (a norm, rope or activation kernel) adds them. deferred_splits reports the split count
//                  (0: y is complete).
constexpr size_t kLinearPartialsOffset = 64 * 1024;
struct LinearExtras {
  int glu = 0, glu_pd = 16;
  float glu_alpha = 1.702f, glu_limit = 7.f;
  int defer_reduce = 0;
  int deferred_splits = 0;
};
// returns the number of kernels launched (2 when split-K adds its reduction)
int linear_bf16(const void* x, long long ldx, const void* w, long long ldw, const void* bias,
                 void* y, long long ldy, int T, int N, int K, void* workspace,
                 size_t workspace_bytes, int* status, int force_splits, cudaStream_t stream,
                 LinearExtras* ex = nullptr);
size_t gemm_bf16_workspace_bytes(int tokens, int features);
void gemm_bf16_prepare_device();   // per-device set-up of every tile width (attributes, module load)
int gemm_bf16_occupancy(int bn);

// Tensor-parallel hooks of the GEMM (see gemm_bf16.cu). Zero-initialise, then fill the half
// that is wanted: rs_* turns the epilogue into a reduce-scatter over peer memory, ag_* makes the
// TMA producer wait for rows that peers deliver into the (local) activation operand.
struct TpLinearArgs {
  void* rs_bufs[8];
  uint32_t* rs_flags[8];
  int tp, my_rank, rows_per;
  int rs_bcast;              // 1: push every row to every rank (one-shot all-reduce layout)
  long long rs_ld;
  const uint32_t* ag_flags;
  uint32_t* ag_consumed;
  unsigned int* cta_done;
  int* expected_out;         // host int: arrival-counter bumps every destination will see from this rank
};
int linear_bf16_tp(const void* x, long long ldx, const void* w, long long ldw, const void* bias,
                   void* y, long long ldy, int T, int N, int K, void* workspace,
                   size_t workspace_bytes, int* status, int force_splits, const TpLinearArgs* tpa,
                   cudaStream_t stream, LinearExtras* ex = nullptr);
int linear_rs_expected_signals(int T, int N, int rows_per, int dest);

// Sequence-sharded residual update + RMSNorm + all-gather of the normalised rows (comm_tp.cu).
struct TpNormArgs {
  void* residual;            // [rows_per][hidden] bf16, this rank's rows of the residual stream
  const void* rs_buf;        // local receive buffer [tp][rows_per][hidden]; null = nothing to add
  const uint32_t* rs_flags;  // [tp] bumped by the sources' GEMM epilogues
  uint32_t* rs_consumed;     // [tp]
  uint32_t rs_expected;      // bumps expected from each source for this step
  const void* norm_w;
  float eps, w_offset;
  void* ag_bufs[8];          // every rank's gathered-activation buffer [tokens][hidden]
  uint32_t* ag_flags[8];     // every rank's arrival counters; this rank bumps entry [my_rank]
  int tp, my_rank, rows_per, tokens, hidden;
  int bcast;                 // 1: all rows are local (partials were broadcast); output stays local
  unsigned int* cta_done;
  int* status;
};
void tp_reduce_norm_allgather(const TpNormArgs& a, cudaStream_t s);

// One-shot all-reduce (sum) of a small message through peer slots.
struct TpAllReduceArgs {
  const void* input;
  void* output;
  size_t bytes;              // multiple of 16, at most slot_bytes
  size_t slot_bytes;
  int is_fp32;               // else bf16
  int gather;                // 1: output [tp][bytes] = every rank's vector (no sum)
  void* slots[8];            // every rank's slot buffer [tp][slot_bytes]
  uint32_t* flags[8];        // every rank's arrival counters [tp]
  const uint32_t* my_flags;  // == flags[my_rank]
  uint32_t* consumed;        // local [tp]
  int tp, my_rank;
  unsigned int* cta_done;
  int* status;
};
void tp_allreduce(const TpAllReduceArgs& a, cudaStream_t s);

// Peer memory through CUDA IPC (one process per GPU on one node).
void* symm_alloc(size_t bytes);
void symm_free(void* p);
void symm_export(void* p, unsigned char out[64]);
void* symm_import(const unsigned char in[64]);
void symm_close(void* p);

// ---- block-scaled FP8 ------------------------------------------------------------------
// Large-batch bf16 GEMM on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles): T >= 256, N >= 256, N % 8 == 0, K % 8 == 0.
bool linear_bf16_pair_supported(int T, int N, int K);
int linear_bf16_pair(const void* x, long long ldx, const void* w, long long ldw, const void* bias, void* y, long long ldy,
                     int T, int N, int K, int* status, cudaStream_t stream, const struct LinearExtras* ex = nullptr);

// Packed 4-bit weights x at most 4 tokens on dp4a (int8 activations quantised inside the kernel); formats as linear_w4a16.
bool gemv_w4_supported(int T, int K);
int gemv_w4(const void* x, long long ldx, const void* codes, const void* scales, int fmt, float alpha, const void* bias,
            void* y, long long ldy, int T, int N, int K, cudaStream_t stream);

// GGUF Q5_K (fmt 5) / Q6_K (6) / Q8_0 (8) in planar device form: dp4a product for at most 4 tokens, bf16 expansion.
bool gemv_wk_supported(int T, int K, int fmt);
int gemv_wk(const void* x, long long ldx, const void* codes, const void* high, const void* sub, const void* sup, int fmt,
            const void* bias, void* y, long long ldy, int T, int N, int K, cudaStream_t stream);
void wk_dequant_bf16(const void* codes, const void* high, const void* sub, const void* sup, int fmt, void* out,
                     long long rows, int K, cudaStream_t s);

// Block-scaled GEMMs (tcgen05 kind::mxf8f6f4 / kind::mxf4nvf4 .block_scale). kind 0: e4m3 weights, kind 1: packed
// e2m1 weights, both with e4m3 activations and one e8m0 scale per 32 values; kind 2: NVFP4 on both sides (packed
// e2m1, one e4m3 scale per 16, tensor scale x per-token scale). Scale factors travel in 512-byte atoms (128 rows x
// 4 scales). The token tile (16 / 32 / 64 / 128) is a function of T alone, so quantiser and GEMM agree on the atoms.
int mx_token_tile(int T);
size_t mx_act_scale_bytes(int T, int K, int kind);
void quant_mx(const void* x, long long ldx, void* xq, void* sf, int T, int K, cudaStream_t s);
void quant_nvfp4(const void* x, long long ldx, void* xq, void* sf, float* tok_scale, int T, int K, cudaStream_t s);
// kinds 3 / 4: e4m3 / int8 on both sides without scale atoms (sfa = sfb = null): feat_scale[N] and tok_scale[T].
void quant_rows_8bit(const void* x, long long ldx, void* xq, float* tok_scale, int T, int K, int is_int8, cudaStream_t s);
int linear_mx(const void* xq, const void* sfb, const void* wq, const void* sfa, int kind, float alpha,
              const float* tok_scale, const float* feat_scale, const void* bias, void* y, long long ldy, int T, int N, int K,
              void* workspace, size_t workspace_bytes, int* status, cudaStream_t stream);
void quant_fp8_1x128(const void* x, long long ldx, void* xq, float* sx, int tokens, int K, cudaStream_t s);
int linear_fp8_block(const void* xq, const float* sx, const void* wq, const float* sw, const void* bias, void* y,
                     long long ldy, int T, int N, int K, int* status, cudaStream_t stream, void* workspace = nullptr,
                     size_t workspace_bytes = 0);   // workspace: fp32 split-K partials (few tiles, or K above 8192)

// ---- packed 4-bit weights x bf16 activations (fmt 0 = NVFP4: e4m3 scale per 16; 1 = MXFP4: e8m0 per 32)
int linear_w4a16(const void* x, long long ldx, const void* codes, const void* scales, int fmt, float alpha,
                 const void* bias, void* y, long long ldy, int T, int N, int K, void* workspace, size_t workspace_bytes,
                 int* status, cudaStream_t stream);
int moe_grouped_linear_w4(const void* xp, long long ldx, const void* codes_stack, const void* scales_stack, int fmt,
                          float alpha, const void* bias_stack, void* y, long long ldy, int rows_cap, int n_out, int K,
                          int experts, const int* tile_expert, const int* tile_row0, const int* num_tiles, int max_tiles,
                          int bn, int* status, cudaStream_t stream);
void w4_dequant_bf16(const void* codes, const void* scales, int fmt, float alpha, void* out, long long rows, int K,
                     cudaStream_t s);

// ---- expert-parallel all-to-all over peer memory (csrc/moe_a2a.cu) -----------------------
constexpr int kMaxEp = 8;
struct EpArgs {
  void* recv_x[kMaxEp];       // [cap][hidden] bf16 on each rank
  void* recv_meta[kMaxEp];    // [cap] int4 on each rank
  void* ctrl[kMaxEp];         // 32 uint32 on each rank, zero-initialised
  void* comb_y[kMaxEp];       // [max entries][hidden] bf16 on each rank
  int ranks, my_rank, cap, hidden, experts_per_rank;
};
// call_ctr: the rank's device-side call counter (dispatch advances it, the others read it); null = use `epoch`.
void ep_dispatch(const EpArgs& a, const void* x, long long ldx, const int* ids, int tokens, int k, unsigned epoch,
                 unsigned* call_ctr, int* status, cudaStream_t s);
void ep_ingest(const EpArgs& a, unsigned epoch, const unsigned* call_ctr, int* ids_out, int* count_out, int* status,
               cudaStream_t s);
void ep_return(const EpArgs& a, const void* y, long long ldy, const int* row_of, const int* count, unsigned epoch,
               const unsigned* call_ctr, cudaStream_t s);
void ep_wait_returns(const EpArgs& a, unsigned epoch, const unsigned* call_ctr, int* status, cudaStream_t s);

// ---- mixture of experts ---------------------------------------------------------------
int moe_grouped_linear_bf16(const void* xp, long long ldx, const void* w_stack, long long ldw,
                            const void* bias_stack, void* y, long long ldy, int rows_cap, int n_out, int K,
                            int experts, const int* tile_expert, const int* tile_row0, const int* num_tiles,
                            int max_tiles, int bn, int* status, cudaStream_t stream);
// score-weighted routers (score_kind 1 softmax over all experts, 2 sigmoid; selection on score + select_bias; optional renormalisation; scale)
void moe_route_scored(const void* logits, long long ld, const float* select_bias, int tokens, int experts, int k, int score_kind,
                      int renorm, float scale, int* ids, float* weights, cudaStream_t s);
void moe_route(const void* logits, long long ld, const void* bias, int tokens, int experts, int k, int softmax_all,
               int* ids, float* weights, cudaStream_t s);
void moe_align(const int* ids, int tokens, int k, int experts, int expert_lo, int expert_hi, int bn, int* row_of,
               int* token_of, int rows_cap, int* tile_expert, int* tile_row0, int* num_tiles, int max_tiles,
               cudaStream_t s);
void moe_gather(const void* x, long long ldx, const int* token_of, void* xp, int rows_cap, int hidden, cudaStream_t s);
void moe_combine(const void* y, long long ldy, const int* row_of, const float* weights, int tokens, int k, void* out,
                 long long ldo, int hidden, cudaStream_t s);

// ---- elementwise --------------------------------------------------------------------
void embed_bf16(const int* ids, const void* table, void* out, int tokens, int hidden, int vocab,
                float scale, cudaStream_t s);
void rmsnorm_bf16(void* residual, long long ld_res, const void* delta, long long ld_delta,
                  const void* w, void* y, long long ld_y, int rows, int hidden, float eps,
                  float w_offset, cudaStream_t s);
void rope_qknorm_kvwrite_bf16(void* qkv, long long ld_qkv, const int* positions, const int* slots,
                              const float* inv_freq, const void* q_norm_w, const void* k_norm_w,
                              void* k_cache, void* v_cache, int tokens, int hq, int hkv,
                              int head_dim, int block_size, int rot_dim, int rope_style, float eps,
                              float attn_factor, cudaStream_t s, int kv_fp8 = 0,   // kv_fp8: caches hold e4m3 bytes
                              // optional: read the heads from fp32 split-K partials [splits][tokens][width]
                              // (+ bias) instead of qkv, and write the rotated query heads to q_out
                              const float* partials = nullptr, int splits = 0, const void* bias = nullptr,
                              void* q_out = nullptr, long long ld_q = 0);
// residual += bf16(sum of partials + bias); y = rmsnorm(residual) * w: the split-K reduction of the
// projection before the norm, the residual add and the norm as one kernel
void rmsnorm_splitk_bf16(void* residual, long long ld_res, const float* partials, int splits, const void* bias,
                         const void* w, void* y, long long ld_y, int rows, int hidden, float eps, float w_offset,
                         cudaStream_t s);
// layout 16: gate / up columns interleaved in blocks of 16; partials: split-K sums instead of x
void glu_bf16(const void* x, long long ldx, void* out, long long ldo, int rows, int inter,
              int act_kind, float alpha, float limit, cudaStream_t s, int layout = 0,
              const float* partials = nullptr, int splits = 0, const void* bias = nullptr);
void gather_rows_bf16(const void* x, long long ldx, const int* rows, void* out, int n_rows,
                      int hidden, cudaStream_t s);

// ---- attention ----------------------------------------------------------------------
void attention_generic_bf16(const void* q, long long ldq, const void* k_cache, const void* v_cache,
                            const int* block_tables, int max_blocks, const int* row_seq,
                            const int* positions, void* out, long long ldo, int tokens, int hq,
                            int hkv, int head_dim, int block_size, float scale, int window,
                            const float* sinks, float softcap, cudaStream_t s, int kv_fp8 = 0,
                            const unsigned long long* tree_mask = nullptr, const int* tree_base = nullptr);   // draft trees: see the kernel

// Tensor-core paged attention over a ragged batch described per sequence (q_starts, kv_lens).
// Returns the number of kernels launched.
int attention_tc_bf16(const void* q, long long ldq, const void* k_cache, const void* v_cache,
                      const int* block_tables, int max_blocks, const int* q_starts, const int* kv_lens,
                      void* out, long long ldo, int tokens, int num_seqs, int max_q_len, int min_q_len,
                      int max_kv_len, int hq, int hkv, int head_dim, int block_size, float scale,
                      int window, const float* sinks, float softcap, void* workspace,
                      size_t workspace_bytes, cudaStream_t s, long long num_kv_blocks = 0, int* status = nullptr,
                      int kv_fp8 = 0,    // the caches hold e4m3 bytes (decode-shaped batches only)
                      int bidir = 0);    // no causal mask: every query row sees all kv_len tokens (encoder batches)
// Prefill on tcgen05 with tensor-memory accumulators (head_dim 64 or 128, group size dividing 128).
bool attention_prefill_tmem_supported(int head_dim, int group, int block_size);
void attention_prefill_tmem(const void* q, long long ldq, const void* k_cache, const void* v_cache, long long num_blocks,
                            const int* block_tables, int max_blocks, const int* q_starts, const int* kv_lens,
                            void* out, long long ldo, int num_seqs, int max_q_len, int min_q, int hq, int hkv,
                            int head_dim, float scale, int window, const float* sinks, float softcap, int* status,
                            cudaStream_t s, int tile_variant = 0, int bidir = 0);
size_t attention_tc_workspace_bytes(int tokens, int hq, int head_dim, int max_splits);

// ---- sampling -----------------------------------------------------------------------
struct SampleRow {
  float temperature;         // <= 0: greedy
  float top_p;               // 0 or 1: off
  float min_p;               // 0: off
  float repetition_penalty;  // 1: off
  float presence_penalty;
  float frequency_penalty;
  int top_k;                 // 0: off
  uint32_t draw;             // per-request draw counter (position of the token being sampled)
  unsigned long long seed;
};

void argmax_rows(const void* logits, int is_fp32, long long ld, int rows, int vocab, int* out_ids,
                 float* out_vals, int id_offset, cudaStream_t s);
// argmax with every row cut over several CTAs; `scratch` starts with one zeroed counter per row (the kernel
// re-zeroes them). out_pairs: optional [rows][2] = (value, float(id)).
size_t argmax_split_scratch_bytes(int rows, int parts);
void argmax_rows_split(const void* logits, int is_fp32, long long ld, int rows, int vocab, int* out_ids, float* out_vals,
                       float* out_pairs, int id_offset, void* scratch, size_t scratch_bytes, cudaStream_t s);
// winner per row among the (value, id) pairs of `ranks` vocabulary slices: pairs [ranks][rows][2]
void argmax_pairs_select(const float* pairs, int ranks, int rows, int* out_ids, cudaStream_t s);
void sample_rows(void* logits, int is_fp32, long long ld, int rows, int vocab, const SampleRow* prm,
                 const int* pen_ids, const int* pen_counts, int pen_stride, const int* bias_ids,
                 const float* bias_vals, int bias_stride, const uint32_t* allow_mask, int mask_words,
                 int* out_ids, float* out_logprobs, cudaStream_t s);
// row_start (optional): first verify row of each sequence in the target arrays (ragged steps); without it
// sequence b owns rows b * (k + 1) ... b * (k + 1) + k. draft_logits may be null (point-mass drafts).
void spec_verify_greedy(const int* draft_ids, const int* target_ids, int batch, int k,
                        const int* row_start, const int* n_draft, int* n_accept, int* out_tokens,
                        cudaStream_t s);
void spec_verify_sampled(const void* target_logits, long long ld_t, const void* draft_logits,
                         long long ld_d, int is_fp32, int vocab, const int* draft_ids, int batch,
                         int k, const int* row_start, const int* n_draft, const SampleRow* prm,
                         int* n_accept, int* out_tokens, cudaStream_t s);

// ---- recurrent token mixers on ragged batches (recurrent.cu) -------------------------------------------------------
// q_starts [B + 1] first token row per sequence, seq_state [B] row of the state pool, positions [T]: a sequence whose
// first token of the step is at position 0 starts from zeros. Activations bf16 with leading dimensions in elements;
// scan states fp32, convolution windows bf16 [slots][W - 1][C]. A negative return value means an argument was rejected
// before anything was launched.
int causal_conv1d(const void* x, long long ldx, const float* w, const float* bias, void* state, const int* q_starts,
                  const int* seq_state, const int* positions, void* y, long long ldy, int B, int C, int W, int act,
                  int max_q_len, cudaStream_t stream);   // max_q_len: host-side bound on a sequence's tokens in the step
// Segmented scans (seg_len > 0, segs > 1): seg_state holds B * segs states (segs - 1 per sequence, then one start state per
// sequence), seg_dt B * (segs - 1) sums of time steps per head (Mamba-2) or channel (Mamba-1).
int mamba2_scan(const void* x, long long ldx, const void* dt, long long lddt, const void* Bm, long long ldb, const void* Cm,
                long long ldc, const float* A, const float* D, const float* dt_bias, float* state, const int* q_starts,
                const int* seq_state, const int* positions, void* y, long long ldy, int B, int H, int P, int G, int N,
                float dt_min, float dt_max, int seg_len, int segs, float* seg_state, float* seg_dt, int skip_from,
                cudaStream_t stream);
int mamba1_scan(const void* x, long long ldx, const void* dt, long long lddt, const void* Bm, long long ldb, const void* Cm,
                long long ldc, const void* z, long long ldz, const float* A, const float* D, const float* dt_bias, float* state,
                const int* q_starts, const int* seq_state, const int* positions, void* y, long long ldy, int B, int Dm, int N,
                int seg_len, int segs, float* seg_state, float* seg_dt, cudaStream_t stream);
// kind: 0 RWKV-6, 1 RWKV-7, 2 gated delta rule (one decay per head), 3 delta rule with a decay per key channel.
// Kind 2 with w == nullptr takes raw gates: beta = logit of the step size, gate_raw [T][H] = logit of the decay,
// log decay = gate_A[h] * softplus(gate_raw + gate_dt_bias[h]).
int matrix_state_scan(int kind, const void* r, long long ldr, const void* k, long long ldk, const void* v, long long ldv,
                      const void* a, long long lda, const void* b, long long ldb, const float* w, long long ldw, const float* u,
                      const void* beta, long long ldbeta, float* state, const int* q_starts, const int* seq_state,
                      const int* positions, void* y, long long ldy, int B, int H, int DK, int DV, int kv_ratio, int l2norm,
                      float q_scale, const void* gate_raw, long long ldgate, const float* gate_A, const float* gate_dt_bias,
                      cudaStream_t stream);
void gated_rmsnorm(const void* x, long long ldx, const void* z, long long ldz, const void* w, int wlen, void* y, long long ldy, int T,
                   int D, int group_size, float eps, int norm_before_gate, cudaStream_t stream);

// Latent attention (attention_mla.cu). Element (t, h, e) of the absorbed query part sits at q_abs[t * qa_t + h * qa_h + e]
// (e < 512), the rotated part in q_pe [tokens][H][64]; cache [blocks][block_size][576] = latent | rotated key part; output
// element (t, h, e) at out[t * o_t + h * o_h + e].
void attention_mla_bf16(const void* q_abs, long long qa_t, long long qa_h, const void* q_pe, const void* cache, const int* block_tables,
                        int max_blocks, const int* row_seq, const int* positions, void* out, long long o_t, long long o_h, int tokens,
                        int H, int block_size, float scale, cudaStream_t s);
// Tensor-core form of the same attention (16 heads per CTA as the rows of m16n8k16 MMAs, 64-key tiles by cp.async, split over
// `splits` key slices with a merge kernel; workspace of attention_mla_workspace_bytes when splits > 1).
size_t attention_mla_workspace_bytes(int tokens, int H, int splits);
int attention_mla_splits(int tokens, int H, int max_kv_len);
void attention_mla_tc_bf16(const void* q_abs, long long qa_t, long long qa_h, const void* q_pe, const void* cache, const int* block_tables,
                           int max_blocks, const int* row_seq, const int* positions, void* out, long long o_t, long long o_h, int tokens,
                           int H, int block_size, float scale, int splits, void* workspace, size_t workspace_bytes, cudaStream_t s);
// RMSNorm of the latent + rotation of the shared key part into the cache row of each token (slot < 0: no write), and rotation
// of every head's rotary query values into q_pe [tokens][H][64].
void mla_prepare_bf16(const void* ckv, long long ldc, const void* q, long long ldq, int q_head_stride, int q_rope_offset,
                      const int* positions, const int* slots, const float* inv_freq, float attn_factor, const void* norm_w, float eps,
                      void* cache, void* q_pe, int tokens, int H, cudaStream_t s);

// x = cap * tanh(x / cap) in place over bf16 rows
void softcap_rows_bf16(void* x, long long ldx, int rows, int cols, float cap, cudaStream_t s);

// x += delta (in place, delta may be null), y = LayerNorm(x) * (w + w_offset) + b (b may be null)
void add_layernorm_bf16(void* x, long long ldx, const void* delta, long long ldd, const void* w, const void* b, void* y, long long ldy,
                        int rows, int cols, float eps, float w_offset, cudaStream_t s);
// in-place activation: 0 gelu (erf), 1 gelu (tanh), 2 squared relu, 3 silu, 4 relu
void act_rows_bf16(void* x, long long ldx, int rows, int cols, int kind, cudaStream_t s);

}  // namespace fllm
