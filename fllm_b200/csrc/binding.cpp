// torch.ops.fllm_b200.* : thin argument checking around the kernel launchers.
// No kernel is implemented here and nothing falls back to ATen math: when the
// library is loaded, every op below runs the hand-written sm_100a code.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include "fllm_ops.h"

namespace {

using at::Tensor;
using c10::optional;

inline cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

inline void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
}
inline void check_i32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kInt, name, " must be int32");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
inline void check_rows(const Tensor& t, const char* name) {
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, name, " must be 2-D with a unit inner stride");
}
template <typename T>
inline const T* opt_ptr(const optional<Tensor>& t) {
  return t.has_value() && t->defined() ? reinterpret_cast<const T*>(t->data_ptr()) : nullptr;
}

// y = x @ w^T (+ bias). `workspace` (uint8) enables split-K; `status` (int32[1]) receives a
// non-zero code if a pipeline wait inside the kernel ran out.
int64_t linear(const Tensor& x, const Tensor& w, const optional<Tensor>& bias, Tensor y,
            const optional<Tensor>& workspace, const optional<Tensor>& status, int64_t force_splits) {
  check_bf16(x, "x"); check_bf16(w, "w"); check_bf16(y, "y");
  check_rows(x, "x"); check_rows(w, "w"); check_rows(y, "y");
  TORCH_CHECK(x.size(1) == w.size(1), "linear: K mismatch");
  TORCH_CHECK(y.size(0) == x.size(0) && y.size(1) == w.size(0), "linear: output shape mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  void* ws = nullptr;
  size_t ws_bytes = 0;
  if (workspace.has_value() && workspace->defined()) {
    ws = workspace->data_ptr();
    ws_bytes = workspace->nbytes();
  }
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  return fllm::linear_bf16(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), opt_ptr<void>(bias),
                    y.data_ptr(), y.stride(0), (int)x.size(0), (int)w.size(0), (int)x.size(1), ws,
                    ws_bytes, st, (int)force_splits, cur_stream());
}

// y = x @ w^T (+ bias) on CTA pairs (cta_group::2, 256 x 256 tiles): at least 256 tokens.
int64_t linear_pair(const Tensor& x, const Tensor& w, const optional<Tensor>& bias, Tensor y, const optional<Tensor>& status) {
  check_bf16(x, "x"); check_bf16(w, "w"); check_bf16(y, "y");
  check_rows(x, "x"); check_rows(w, "w"); check_rows(y, "y");
  TORCH_CHECK(x.size(1) == w.size(1), "linear_pair: K mismatch");
  TORCH_CHECK(y.size(0) == x.size(0) && y.size(1) == w.size(0), "linear_pair: output shape mismatch");
  TORCH_CHECK(fllm::linear_bf16_pair_supported((int)x.size(0), (int)w.size(0), (int)x.size(1)), "linear_pair: shape not supported");
  c10::cuda::CUDAGuard guard(x.device());
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  return fllm::linear_bf16_pair(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), opt_ptr<void>(bias), y.data_ptr(),
                                y.stride(0), (int)x.size(0), (int)w.size(0), (int)x.size(1), st, cur_stream());
}

// linear with the optional behaviours of fllm::LinearExtras. glu > 0: y is [T, N / 2] (the activation runs in the
// epilogue, or in the caller's consumer when the call deferred split-K). Returns [kernels launched, deferred splits].
std::vector<int64_t> linear_ex(const Tensor& x, const Tensor& w, const optional<Tensor>& bias, Tensor y,
                               const optional<Tensor>& workspace, const optional<Tensor>& status, int64_t force_splits,
                               int64_t glu, int64_t glu_pd, double glu_alpha, double glu_limit, bool defer_reduce) {
  check_bf16(x, "x"); check_bf16(w, "w"); check_bf16(y, "y");
  check_rows(x, "x"); check_rows(w, "w"); check_rows(y, "y");
  TORCH_CHECK(x.size(1) == w.size(1), "linear: K mismatch");
  TORCH_CHECK(y.size(0) == x.size(0) && y.size(1) == (glu ? w.size(0) / 2 : w.size(0)), "linear: output shape mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  void* ws = nullptr;
  size_t ws_bytes = 0;
  if (workspace.has_value() && workspace->defined()) {
    ws = workspace->data_ptr();
    ws_bytes = workspace->nbytes();
  }
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  fllm::LinearExtras ex;
  ex.glu = (int)glu; ex.glu_pd = (int)glu_pd; ex.glu_alpha = (float)glu_alpha; ex.glu_limit = (float)glu_limit;
  ex.defer_reduce = defer_reduce ? 1 : 0;
  const int n = fllm::linear_bf16(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), opt_ptr<void>(bias),
                                  y.data_ptr(), y.stride(0), (int)x.size(0), (int)w.size(0), (int)x.size(1), ws,
                                  ws_bytes, st, (int)force_splits, cur_stream(), &ex);
  return {n, ex.deferred_splits};
}

inline const float* partials_ptr(const Tensor& workspace, int64_t splits, int64_t rows, int64_t cols) {
  TORCH_CHECK(workspace.is_cuda() && workspace.is_contiguous(), "workspace must be a contiguous CUDA tensor");
  TORCH_CHECK(splits >= 1 && (size_t)workspace.nbytes() >= fllm::kLinearPartialsOffset + (size_t)splits * rows * cols * 4,
              "workspace too small for the split-K partials");
  return reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(workspace.data_ptr()) + fllm::kLinearPartialsOffset);
}

// residual += bf16(sum of the split-K partials in `workspace` + bias); y = rmsnorm(residual) * w
void rmsnorm_splitk(Tensor residual, const Tensor& workspace, int64_t splits, const optional<Tensor>& bias,
                    const Tensor& w, Tensor y, double eps, double w_offset) {
  check_bf16(residual, "residual"); check_bf16(w, "w"); check_bf16(y, "y");
  check_rows(residual, "residual"); check_rows(y, "y");
  c10::cuda::CUDAGuard guard(y.device());
  const float* ws = partials_ptr(workspace, splits, residual.size(0), residual.size(1));
  fllm::rmsnorm_splitk_bf16(residual.data_ptr(), residual.stride(0), ws, (int)splits, opt_ptr<void>(bias), w.data_ptr(),
                            y.data_ptr(), y.stride(0), (int)residual.size(0), (int)residual.size(1), (float)eps,
                            (float)w_offset, cur_stream());
}

void embed(const Tensor& ids, const Tensor& table, Tensor out, double scale) {
  check_i32(ids, "ids"); check_bf16(table, "table"); check_bf16(out, "out");
  TORCH_CHECK(table.is_contiguous() && out.is_contiguous(), "embed: contiguous tensors expected");
  c10::cuda::CUDAGuard guard(out.device());
  fllm::embed_bf16(ids.data_ptr<int>(), table.data_ptr(), out.data_ptr(), (int)ids.numel(),
                   (int)table.size(1), (int)table.size(0), (float)scale, cur_stream());
}

// y = rmsnorm(residual [+ delta]) * w ; with delta the sum is written back to residual.
void rmsnorm(Tensor residual, const optional<Tensor>& delta, const Tensor& w, Tensor y, double eps,
             double w_offset) {
  check_bf16(residual, "residual"); check_bf16(w, "w"); check_bf16(y, "y");
  check_rows(residual, "residual"); check_rows(y, "y");
  const Tensor* d = delta.has_value() && delta->defined() ? &*delta : nullptr;
  if (d) { check_bf16(*d, "delta"); check_rows(*d, "delta"); }
  c10::cuda::CUDAGuard guard(y.device());
  fllm::rmsnorm_bf16(residual.data_ptr(), residual.stride(0), d ? d->data_ptr() : nullptr,
                     d ? d->stride(0) : 0, w.data_ptr(), y.data_ptr(), y.stride(0),
                     (int)residual.size(0), (int)residual.size(1), (float)eps, (float)w_offset,
                     cur_stream());
}

void rope_kv_write(Tensor qkv, const Tensor& positions, const optional<Tensor>& slots,
                   const Tensor& inv_freq, const optional<Tensor>& q_norm_w,
                   const optional<Tensor>& k_norm_w, Tensor k_cache, Tensor v_cache, int64_t hq,
                   int64_t hkv, int64_t head_dim, int64_t rot_dim, int64_t rope_style, double eps,
                   double attn_factor) {
  check_bf16(qkv, "qkv"); check_rows(qkv, "qkv"); check_i32(positions, "positions");
  const bool kv_fp8 = k_cache.element_size() == 1;            // e4m3 cache
  TORCH_CHECK(k_cache.is_cuda() && k_cache.element_size() == v_cache.element_size() &&
              (kv_fp8 || k_cache.scalar_type() == at::kBFloat16), "caches must be bf16 or 1-byte e4m3 tensors");
  TORCH_CHECK(inv_freq.scalar_type() == at::kFloat && inv_freq.is_cuda(), "inv_freq must be fp32 CUDA");
  TORCH_CHECK(qkv.size(1) == (hq + 2 * hkv) * head_dim, "rope_kv_write: qkv width mismatch");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(),
              "caches must be [blocks, kv_heads, block_size, head_dim]");
  c10::cuda::CUDAGuard guard(qkv.device());
  fllm::rope_qknorm_kvwrite_bf16(
      qkv.data_ptr(), qkv.stride(0), positions.data_ptr<int>(), opt_ptr<int>(slots),
      inv_freq.data_ptr<float>(), opt_ptr<void>(q_norm_w), opt_ptr<void>(k_norm_w),
      k_cache.data_ptr(), v_cache.data_ptr(), (int)qkv.size(0), (int)hq, (int)hkv, (int)head_dim,
      (int)k_cache.size(2), (int)rot_dim, (int)rope_style, (float)eps, (float)attn_factor,
      cur_stream(), kv_fp8 ? 1 : 0);
}

// QK-norm + RoPE + KV write reading the q|k|v heads from split-K partials; rotated queries go to q_out
void rope_kv_write_splitk(const Tensor& workspace, int64_t splits, const optional<Tensor>& bias, Tensor q_out,
                          const Tensor& positions, const optional<Tensor>& slots, const Tensor& inv_freq,
                          const optional<Tensor>& q_norm_w, const optional<Tensor>& k_norm_w, Tensor k_cache,
                          Tensor v_cache, int64_t hq, int64_t hkv, int64_t head_dim, int64_t rot_dim,
                          int64_t rope_style, double eps, double attn_factor) {
  check_bf16(q_out, "q_out"); check_rows(q_out, "q_out"); check_i32(positions, "positions");
  const bool kv_fp8 = k_cache.element_size() == 1;
  TORCH_CHECK(k_cache.is_cuda() && k_cache.element_size() == v_cache.element_size() &&
              (kv_fp8 || k_cache.scalar_type() == at::kBFloat16), "caches must be bf16 or 1-byte e4m3 tensors");
  TORCH_CHECK(inv_freq.scalar_type() == at::kFloat && inv_freq.is_cuda(), "inv_freq must be fp32 CUDA");
  TORCH_CHECK(q_out.size(1) == hq * head_dim, "rope_kv_write_splitk: q width mismatch");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(),
              "caches must be [blocks, kv_heads, block_size, head_dim]");
  c10::cuda::CUDAGuard guard(q_out.device());
  const int tokens = (int)q_out.size(0);
  const float* ws = partials_ptr(workspace, splits, tokens, (hq + 2 * hkv) * head_dim);
  fllm::rope_qknorm_kvwrite_bf16(
      nullptr, 0, positions.data_ptr<int>(), opt_ptr<int>(slots), inv_freq.data_ptr<float>(),
      opt_ptr<void>(q_norm_w), opt_ptr<void>(k_norm_w), k_cache.data_ptr(), v_cache.data_ptr(), tokens, (int)hq,
      (int)hkv, (int)head_dim, (int)k_cache.size(2), (int)rot_dim, (int)rope_style, (float)eps, (float)attn_factor,
      cur_stream(), kv_fp8 ? 1 : 0, ws, (int)splits, opt_ptr<void>(bias), q_out.data_ptr(), q_out.stride(0));
}

// glu with a column layout (0 natural, 16 blocked) and, when splits > 0, split-K partials as the source
void glu_ex(const optional<Tensor>& x, Tensor out, int64_t act_kind, double alpha, double limit, int64_t layout,
            const optional<Tensor>& workspace, int64_t splits, const optional<Tensor>& bias) {
  check_bf16(out, "out"); check_rows(out, "out");
  c10::cuda::CUDAGuard guard(out.device());
  const float* ws = nullptr;
  const void* xp = nullptr;
  long long ldx = 0;
  if (splits > 0) {
    TORCH_CHECK(workspace.has_value(), "glu_ex: workspace expected");
    ws = partials_ptr(*workspace, splits, out.size(0), 2 * out.size(1));
  } else {
    TORCH_CHECK(x.has_value(), "glu_ex: x expected");
    check_bf16(*x, "x"); check_rows(*x, "x");
    TORCH_CHECK(x->size(1) == 2 * out.size(1) && x->size(0) == out.size(0), "glu: shape mismatch");
    xp = x->data_ptr(); ldx = x->stride(0);
  }
  fllm::glu_bf16(xp, ldx, out.data_ptr(), out.stride(0), (int)out.size(0), (int)out.size(1), (int)act_kind,
                 (float)alpha, (float)limit, cur_stream(), (int)layout, ws, (int)splits, opt_ptr<void>(bias));
}

void glu(const Tensor& x, Tensor out, int64_t act_kind, double alpha, double limit) {
  check_bf16(x, "x"); check_bf16(out, "out"); check_rows(x, "x"); check_rows(out, "out");
  TORCH_CHECK(x.size(1) == 2 * out.size(1) && x.size(0) == out.size(0), "glu: shape mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::glu_bf16(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), (int)x.size(0),
                 (int)out.size(1), (int)act_kind, (float)alpha, (float)limit, cur_stream());
}

void gather_rows(const Tensor& x, const Tensor& rows, Tensor out) {
  check_bf16(x, "x"); check_rows(x, "x"); check_i32(rows, "rows"); check_bf16(out, "out");
  TORCH_CHECK(out.is_contiguous() && out.size(1) == x.size(1), "gather_rows: bad output");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::gather_rows_bf16(x.data_ptr(), x.stride(0), rows.data_ptr<int>(), out.data_ptr(),
                         (int)rows.numel(), (int)x.size(1), cur_stream());
}

void add_layernorm(Tensor x, const optional<Tensor>& delta, const Tensor& w, const optional<Tensor>& b, Tensor y, double eps, double w_offset) {
  check_bf16(x, "x"); check_rows(x, "x"); check_bf16(y, "y"); check_rows(y, "y"); check_bf16(w, "w");
  TORCH_CHECK(y.sizes() == x.sizes() && w.is_contiguous() && w.numel() == x.size(1), "add_layernorm: shapes");
  const void* d = nullptr;
  long long ldd = 0;
  if (delta.has_value() && delta->defined()) {
    check_bf16(*delta, "delta"); check_rows(*delta, "delta");
    TORCH_CHECK(delta->sizes() == x.sizes(), "add_layernorm: delta shape");
    d = delta->data_ptr();
    ldd = delta->stride(0);
  }
  const void* bp = nullptr;
  if (b.has_value() && b->defined()) {
    check_bf16(*b, "b");
    TORCH_CHECK(b->is_contiguous() && b->numel() == x.size(1), "add_layernorm: bias shape");
    bp = b->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  fllm::add_layernorm_bf16(x.data_ptr(), x.stride(0), d, ldd, w.data_ptr(), bp, y.data_ptr(), y.stride(0), (int)x.size(0), (int)x.size(1),
                           (float)eps, (float)w_offset, cur_stream());
}

void act_(Tensor x, int64_t kind) {
  check_bf16(x, "x"); check_rows(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::act_rows_bf16(x.data_ptr(), x.stride(0), (int)x.size(0), (int)x.size(1), (int)kind, cur_stream());
}

void softcap_(Tensor x, double cap) {
  check_bf16(x, "x"); check_rows(x, "x");
  TORCH_CHECK(cap > 0, "softcap_: the cap must be positive");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::softcap_rows_bf16(x.data_ptr(), x.stride(0), (int)x.size(0), (int)x.size(1), (float)cap, cur_stream());
}

void attention_generic(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache,
                       const Tensor& block_tables, const Tensor& row_seq, const Tensor& positions,
                       Tensor out, int64_t hq, int64_t hkv, int64_t head_dim, double scale,
                       int64_t window, const optional<Tensor>& sinks, double softcap,
                       const optional<Tensor>& tree_mask, const optional<Tensor>& tree_base) {
  check_bf16(q, "q"); check_rows(q, "q"); check_bf16(out, "out"); check_rows(out, "out");
  check_i32(block_tables, "block_tables"); check_i32(row_seq, "row_seq");
  check_i32(positions, "positions");
  const unsigned long long* tm = nullptr;
  const int* tb = nullptr;
  if (tree_mask.has_value() && tree_mask->defined()) {        // draft trees: one 64-bit ancestor mask and one context length per row
    TORCH_CHECK(tree_base.has_value() && tree_base->defined(), "attention_generic: tree_mask needs tree_base");
    TORCH_CHECK(tree_mask->scalar_type() == at::kLong && tree_mask->is_contiguous() && tree_mask->numel() == q.size(0), "tree_mask: int64 [rows]");
    check_i32(*tree_base, "tree_base");
    TORCH_CHECK(tree_base->numel() == q.size(0), "tree_base: int32 [rows]");
    tm = reinterpret_cast<const unsigned long long*>(tree_mask->data_ptr<int64_t>());
    tb = tree_base->data_ptr<int>();
  }
  const bool kv_fp8 = k_cache.element_size() == 1;            // e4m3 bytes instead of bf16
  TORCH_CHECK(k_cache.is_cuda() && k_cache.is_contiguous() && v_cache.is_contiguous() &&
              k_cache.element_size() == v_cache.element_size() && (kv_fp8 || k_cache.scalar_type() == at::kBFloat16),
              "caches must be contiguous bf16 or 1-byte e4m3 tensors");
  c10::cuda::CUDAGuard guard(q.device());
  fllm::attention_generic_bf16(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                               block_tables.data_ptr<int>(), (int)block_tables.size(1),
                               row_seq.data_ptr<int>(), positions.data_ptr<int>(), out.data_ptr(),
                               out.stride(0), (int)q.size(0), (int)hq, (int)hkv, (int)head_dim,
                               (int)k_cache.size(2), (float)scale, (int)window,
                               opt_ptr<float>(sinks), (float)softcap, cur_stream(), kv_fp8 ? 1 : 0, tm, tb);
}

int64_t attention_tc(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache,
                     const Tensor& block_tables, const Tensor& q_starts, const Tensor& kv_lens, Tensor out,
                     int64_t num_seqs, int64_t max_q_len, int64_t min_q_len, int64_t max_kv_len, int64_t hq,
                     int64_t hkv, int64_t head_dim, double scale, int64_t window,
                     const optional<Tensor>& sinks, double softcap, const optional<Tensor>& workspace,
                     const optional<Tensor>& status, bool bidirectional) {
  check_bf16(q, "q"); check_rows(q, "q"); check_bf16(out, "out"); check_rows(out, "out");
  const bool kv_fp8 = k_cache.element_size() == 1;            // e4m3 bytes: the decode kernel widens them to f16
  TORCH_CHECK(k_cache.is_cuda() && v_cache.is_cuda() && k_cache.is_contiguous() && v_cache.is_contiguous() &&
              k_cache.element_size() == v_cache.element_size() && (kv_fp8 || k_cache.scalar_type() == at::kBFloat16),
              "caches must be contiguous bf16 or 1-byte e4m3 tensors");
  check_i32(q_starts, "q_starts"); check_i32(kv_lens, "kv_lens");
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && block_tables.dim() == 2 &&
              block_tables.stride(1) == 1 && block_tables.stride(0) == block_tables.size(1),
              "block_tables must be a dense int32 matrix");
  TORCH_CHECK(q_starts.numel() >= num_seqs + 1 && kv_lens.numel() >= num_seqs, "attention_tc: metadata too short");
  c10::cuda::CUDAGuard guard(q.device());
  void* ws = nullptr;
  size_t ws_bytes = 0;
  if (workspace.has_value() && workspace->defined()) { ws = workspace->data_ptr(); ws_bytes = workspace->nbytes(); }
  return fllm::attention_tc_bf16(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                                 block_tables.data_ptr<int>(), (int)block_tables.size(1),
                                 q_starts.data_ptr<int>(), kv_lens.data_ptr<int>(), out.data_ptr(),
                                 out.stride(0), (int)q.size(0), (int)num_seqs, (int)max_q_len,
                                 (int)min_q_len, (int)max_kv_len, (int)hq, (int)hkv, (int)head_dim,
                                 (int)k_cache.size(2), (float)scale, (int)window, opt_ptr<float>(sinks),
                                 (float)softcap, ws, ws_bytes, cur_stream(), (long long)k_cache.size(0),
                                 const_cast<int*>(opt_ptr<int>(status)), kv_fp8 ? 1 : 0, bidirectional ? 1 : 0);
}

void argmax(const Tensor& logits, Tensor out_ids, const optional<Tensor>& out_vals,
            int64_t id_offset) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "argmax: bad logits");
  const bool f32 = logits.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || logits.scalar_type() == at::kBFloat16, "argmax: logits must be fp32 or bf16");
  check_i32(out_ids, "out_ids");
  c10::cuda::CUDAGuard guard(logits.device());
  float* ov = out_vals.has_value() && out_vals->defined() ? out_vals->data_ptr<float>() : nullptr;
  fllm::argmax_rows(logits.data_ptr(), f32, logits.stride(0), (int)logits.size(0),
                    (int)logits.size(1), out_ids.data_ptr<int>(), ov, (int)id_offset, cur_stream());
}

void argmax_split(const Tensor& logits, Tensor out_ids, const optional<Tensor>& out_vals, const optional<Tensor>& out_pairs,
                  int64_t id_offset, Tensor scratch) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "argmax: bad logits");
  const bool f32 = logits.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || logits.scalar_type() == at::kBFloat16, "argmax: logits must be fp32 or bf16");
  check_i32(out_ids, "out_ids");
  TORCH_CHECK(scratch.is_cuda() && scratch.is_contiguous(), "argmax_split: scratch must be a contiguous CUDA tensor");
  c10::cuda::CUDAGuard guard(logits.device());
  float* ov = out_vals.has_value() && out_vals->defined() ? out_vals->data_ptr<float>() : nullptr;
  float* op = nullptr;
  if (out_pairs.has_value() && out_pairs->defined()) {
    TORCH_CHECK(out_pairs->scalar_type() == at::kFloat && out_pairs->is_contiguous() && out_pairs->numel() >= 2 * logits.size(0),
                "argmax_split: out_pairs must be fp32 [rows, 2]");
    op = out_pairs->data_ptr<float>();
  }
  fllm::argmax_rows_split(logits.data_ptr(), f32, logits.stride(0), (int)logits.size(0), (int)logits.size(1),
                          out_ids.data_ptr<int>(), ov, op, (int)id_offset, scratch.data_ptr(), scratch.nbytes(), cur_stream());
}

void argmax_pairs_select(const Tensor& pairs, Tensor out_ids) {
  TORCH_CHECK(pairs.is_cuda() && pairs.scalar_type() == at::kFloat && pairs.is_contiguous() && pairs.dim() == 3 &&
              pairs.size(2) == 2, "argmax_pairs_select: pairs must be fp32 [ranks, rows, 2]");
  check_i32(out_ids, "out_ids");
  c10::cuda::CUDAGuard guard(pairs.device());
  fllm::argmax_pairs_select(pairs.data_ptr<float>(), (int)pairs.size(0), (int)pairs.size(1), out_ids.data_ptr<int>(), cur_stream());
}

// params: uint8 tensor holding rows x sizeof(SampleRow) bytes laid out like fllm::SampleRow.
void sample(Tensor logits, const Tensor& params, const optional<Tensor>& pen_ids,
            const optional<Tensor>& pen_counts, const optional<Tensor>& bias_ids,
            const optional<Tensor>& bias_vals, const optional<Tensor>& allow_mask, Tensor out_ids,
            const optional<Tensor>& out_logprobs) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "sample: bad logits");
  const bool f32 = logits.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || logits.scalar_type() == at::kBFloat16, "sample: logits must be fp32 or bf16");
  const int rows = (int)logits.size(0);
  TORCH_CHECK(params.is_cuda() && params.nbytes() >= rows * sizeof(fllm::SampleRow),
              "sample: params too small");
  check_i32(out_ids, "out_ids");
  c10::cuda::CUDAGuard guard(logits.device());
  const bool pen = pen_ids.has_value() && pen_ids->defined();
  const bool bias = bias_ids.has_value() && bias_ids->defined();
  const bool mask = allow_mask.has_value() && allow_mask->defined();
  fllm::sample_rows(
      logits.data_ptr(), f32, logits.stride(0), rows, (int)logits.size(1),
      reinterpret_cast<const fllm::SampleRow*>(params.data_ptr()),
      pen ? pen_ids->data_ptr<int>() : nullptr, pen ? pen_counts->data_ptr<int>() : nullptr,
      pen ? (int)pen_ids->size(1) : 0, bias ? bias_ids->data_ptr<int>() : nullptr,
      bias ? bias_vals->data_ptr<float>() : nullptr, bias ? (int)bias_ids->size(1) : 0,
      mask ? reinterpret_cast<const uint32_t*>(allow_mask->data_ptr()) : nullptr,
      mask ? (int)allow_mask->size(1) : 0, out_ids.data_ptr<int>(),
      out_logprobs.has_value() && out_logprobs->defined() ? out_logprobs->data_ptr<float>() : nullptr,
      cur_stream());
}

void spec_verify_greedy(const Tensor& draft_ids, const Tensor& target_ids,
                        const optional<Tensor>& n_draft, Tensor n_accept, Tensor out_tokens,
                        const optional<Tensor>& row_start) {
  check_i32(draft_ids, "draft_ids"); check_i32(target_ids, "target_ids");
  check_i32(n_accept, "n_accept"); check_i32(out_tokens, "out_tokens");
  const int batch = (int)draft_ids.size(0), k = (int)draft_ids.size(1);
  const bool ragged = row_start.has_value() && row_start->defined();
  TORCH_CHECK(out_tokens.size(0) == batch && out_tokens.size(1) == k + 1 && n_accept.numel() == batch, "spec_verify: shapes");
  TORCH_CHECK(ragged ? row_start->numel() == batch
                     : (target_ids.dim() == 2 && target_ids.size(0) == batch && target_ids.size(1) == k + 1),
              "spec_verify: target shape");
  TORCH_CHECK(target_ids.is_contiguous() && draft_ids.is_contiguous() && out_tokens.is_contiguous(), "spec_verify: contiguous");
  c10::cuda::CUDAGuard guard(draft_ids.device());
  fllm::spec_verify_greedy(draft_ids.data_ptr<int>(), target_ids.data_ptr<int>(), batch, k,
                           opt_ptr<int>(row_start), opt_ptr<int>(n_draft), n_accept.data_ptr<int>(),
                           out_tokens.data_ptr<int>(), cur_stream());
}

void spec_verify_sampled(const Tensor& target_logits, const optional<Tensor>& draft_logits,
                         const Tensor& draft_ids, const optional<Tensor>& n_draft,
                         const Tensor& params, Tensor n_accept, Tensor out_tokens,
                         const optional<Tensor>& row_start) {
  const bool f32 = target_logits.scalar_type() == at::kFloat;
  const bool has_q = draft_logits.has_value() && draft_logits->defined();
  check_i32(draft_ids, "draft_ids");
  const int batch = (int)draft_ids.size(0), k = (int)draft_ids.size(1);
  const bool ragged = row_start.has_value() && row_start->defined();
  TORCH_CHECK(target_logits.dim() == 2 && target_logits.stride(1) == 1 &&
              (ragged ? row_start->numel() == batch : target_logits.size(0) == (int64_t)batch * (k + 1)),
              "spec_verify: target rows");
  if (has_q) {
    TORCH_CHECK(target_logits.scalar_type() == draft_logits->scalar_type(), "spec_verify: dtype mismatch");
    TORCH_CHECK(draft_logits->dim() == 2 && draft_logits->size(0) == (int64_t)batch * k &&
                draft_logits->size(1) == target_logits.size(1) && draft_logits->stride(1) == 1, "spec_verify: draft rows");
  }
  TORCH_CHECK(params.numel() * params.element_size() >= (int64_t)batch * (int64_t)sizeof(fllm::SampleRow), "spec_verify: params");
  TORCH_CHECK(out_tokens.size(0) == batch && out_tokens.size(1) == k + 1 && n_accept.numel() == batch, "spec_verify: shapes");
  c10::cuda::CUDAGuard guard(draft_ids.device());
  fllm::spec_verify_sampled(target_logits.data_ptr(), target_logits.stride(0),
                            has_q ? draft_logits->data_ptr() : nullptr, has_q ? draft_logits->stride(0) : 0, f32,
                            (int)target_logits.size(1), draft_ids.data_ptr<int>(), batch, k,
                            opt_ptr<int>(row_start), opt_ptr<int>(n_draft),
                            reinterpret_cast<const fllm::SampleRow*>(params.data_ptr()),
                            n_accept.data_ptr<int>(), out_tokens.data_ptr<int>(), cur_stream());
}

int64_t gemm_occupancy(int64_t bn) { return fllm::gemm_bf16_occupancy((int)bn); }

int64_t sample_row_bytes() { return (int64_t)sizeof(fllm::SampleRow); }

}  // namespace

TORCH_LIBRARY(fllm_b200, m) {
  m.def("linear(Tensor x, Tensor w, Tensor? bias, Tensor(a!) y, Tensor? workspace, Tensor? status, int force_splits) -> int", &linear);
  m.def("linear_pair(Tensor x, Tensor w, Tensor? bias, Tensor(a!) y, Tensor? status) -> int", &linear_pair);
  m.def("linear_ex(Tensor x, Tensor w, Tensor? bias, Tensor(a!) y, Tensor? workspace, Tensor? status, int force_splits, int glu, int glu_pd, float glu_alpha, float glu_limit, bool defer_reduce) -> int[]", &linear_ex);
  m.def("rmsnorm_splitk(Tensor(a!) residual, Tensor workspace, int splits, Tensor? bias, Tensor w, Tensor(b!) y, float eps, float w_offset) -> ()", &rmsnorm_splitk);
  m.def("rope_kv_write_splitk(Tensor workspace, int splits, Tensor? bias, Tensor(a!) q_out, Tensor positions, Tensor? slots, Tensor inv_freq, Tensor? q_norm_w, Tensor? k_norm_w, Tensor(b!) k_cache, Tensor(c!) v_cache, int hq, int hkv, int head_dim, int rot_dim, int rope_style, float eps, float attn_factor) -> ()", &rope_kv_write_splitk);
  m.def("glu_ex(Tensor? x, Tensor(a!) out, int act_kind, float alpha, float limit, int layout, Tensor? workspace, int splits, Tensor? bias) -> ()", &glu_ex);
  m.def("embed(Tensor ids, Tensor table, Tensor(a!) out, float scale) -> ()", &embed);
  m.def("rmsnorm(Tensor(a!) residual, Tensor? delta, Tensor w, Tensor(b!) y, float eps, float w_offset) -> ()", &rmsnorm);
  m.def("rope_kv_write(Tensor(a!) qkv, Tensor positions, Tensor? slots, Tensor inv_freq, Tensor? q_norm_w, Tensor? k_norm_w, Tensor(b!) k_cache, Tensor(c!) v_cache, int hq, int hkv, int head_dim, int rot_dim, int rope_style, float eps, float attn_factor) -> ()", &rope_kv_write);
  m.def("glu(Tensor x, Tensor(a!) out, int act_kind, float alpha, float limit) -> ()", &glu);
  m.def("gather_rows(Tensor x, Tensor rows, Tensor(a!) out) -> ()", &gather_rows);
  m.def("softcap_(Tensor(a!) x, float cap) -> ()", &softcap_);
  m.def("add_layernorm(Tensor(a!) x, Tensor? delta, Tensor w, Tensor? b, Tensor(b!) y, float eps, float w_offset) -> ()", &add_layernorm);
  m.def("act_(Tensor(a!) x, int kind) -> ()", &act_);
  m.def("attention_generic(Tensor q, Tensor k_cache, Tensor v_cache, Tensor block_tables, Tensor row_seq, Tensor positions, Tensor(a!) out, int hq, int hkv, int head_dim, float scale, int window, Tensor? sinks, float softcap, Tensor? tree_mask=None, Tensor? tree_base=None) -> ()", &attention_generic);
  m.def("attention_tc(Tensor q, Tensor k_cache, Tensor v_cache, Tensor block_tables, Tensor q_starts, Tensor kv_lens, Tensor(a!) out, int num_seqs, int max_q_len, int min_q_len, int max_kv_len, int hq, int hkv, int head_dim, float scale, int window, Tensor? sinks, float softcap, Tensor? workspace, Tensor? status=None, bool bidirectional=False) -> int", &attention_tc);
  m.def("argmax(Tensor logits, Tensor(a!) out_ids, Tensor? out_vals, int id_offset) -> ()", &argmax);
  m.def("argmax_split(Tensor logits, Tensor(a!) out_ids, Tensor? out_vals, Tensor? out_pairs, int id_offset, Tensor(b!) scratch) -> ()", &argmax_split);
  m.def("argmax_pairs_select(Tensor pairs, Tensor(a!) out_ids) -> ()", &argmax_pairs_select);
  m.def("sample(Tensor(a!) logits, Tensor params, Tensor? pen_ids, Tensor? pen_counts, Tensor? bias_ids, Tensor? bias_vals, Tensor? allow_mask, Tensor(b!) out_ids, Tensor? out_logprobs) -> ()", &sample);
  m.def("spec_verify_greedy(Tensor draft_ids, Tensor target_ids, Tensor? n_draft, Tensor(a!) n_accept, Tensor(b!) out_tokens, Tensor? row_start=None) -> ()", &spec_verify_greedy);
  m.def("spec_verify_sampled(Tensor target_logits, Tensor? draft_logits, Tensor draft_ids, Tensor? n_draft, Tensor params, Tensor(a!) n_accept, Tensor(b!) out_tokens, Tensor? row_start=None) -> ()", &spec_verify_sampled);
  m.def("sample_row_bytes() -> int", &sample_row_bytes);
  m.def("gemm_occupancy(int bn) -> int", &gemm_occupancy);
}
