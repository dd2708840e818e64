// Launcher declarations of the sm_100a kernels. Everything takes raw device
// pointers and a stream, so the kernels can be driven from the torch bindings,
// from the C ABI and from stream capture alike. Leading dimensions are in elements.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace fllm {

// ---- dense bf16 GEMM (tcgen05) ------------------------------------------------------
// returns the number of kernels launched (2 when split-K adds its reduction)
int linear_bf16(const void* x, long long ldx, const void* w, long long ldw, const void* bias,
                 void* y, long long ldy, int T, int N, int K, void* workspace,
                 size_t workspace_bytes, int* status, int force_splits, cudaStream_t stream);
size_t gemm_bf16_workspace_bytes(int tokens, int features);

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
                              float attn_factor, cudaStream_t s);
void glu_bf16(const void* x, long long ldx, void* out, long long ldo, int rows, int inter,
              int act_kind, float alpha, float limit, cudaStream_t s);
void gather_rows_bf16(const void* x, long long ldx, const int* rows, void* out, int n_rows,
                      int hidden, cudaStream_t s);

// ---- attention ----------------------------------------------------------------------
void attention_generic_bf16(const void* q, long long ldq, const void* k_cache, const void* v_cache,
                            const int* block_tables, int max_blocks, const int* row_seq,
                            const int* positions, void* out, long long ldo, int tokens, int hq,
                            int hkv, int head_dim, int block_size, float scale, int window,
                            const float* sinks, float softcap, cudaStream_t s);

// Tensor-core paged attention over a ragged batch described per sequence (q_starts, kv_lens).
// Returns the number of kernels launched.
int attention_tc_bf16(const void* q, long long ldq, const void* k_cache, const void* v_cache,
                      const int* block_tables, int max_blocks, const int* q_starts, const int* kv_lens,
                      void* out, long long ldo, int tokens, int num_seqs, int max_q_len, int min_q_len,
                      int max_kv_len, int hq, int hkv, int head_dim, int block_size, float scale,
                      int window, const float* sinks, float softcap, void* workspace,
                      size_t workspace_bytes, cudaStream_t s);
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
void sample_rows(void* logits, int is_fp32, long long ld, int rows, int vocab, const SampleRow* prm,
                 const int* pen_ids, const int* pen_counts, int pen_stride, const int* bias_ids,
                 const float* bias_vals, int bias_stride, const uint32_t* allow_mask, int mask_words,
                 int* out_ids, float* out_logprobs, cudaStream_t s);
void spec_verify_greedy(const int* draft_ids, const int* target_ids, int batch, int k,
                        const int* n_draft, int* n_accept, int* out_tokens, cudaStream_t s);
void spec_verify_sampled(const void* target_logits, long long ld_t, const void* draft_logits,
                         long long ld_d, int is_fp32, int vocab, const int* draft_ids, int batch,
                         int k, const int* n_draft, const SampleRow* prm, int* n_accept,
                         int* out_tokens, cudaStream_t s);

}  // namespace fllm
