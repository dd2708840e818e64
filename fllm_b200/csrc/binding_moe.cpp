// torch.ops.fllm_b200 bindings of the mixture-of-experts kernels.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include "fllm_ops.h"

namespace {
using at::Tensor;
using c10::optional;
inline cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }
inline const void* optp(const optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

void moe_route(const Tensor& logits, const optional<Tensor>& bias, int64_t k, bool softmax_all, Tensor ids, Tensor weights) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 && logits.stride(1) == 1, "logits: bf16 rows");
  TORCH_CHECK(ids.scalar_type() == at::kInt && weights.scalar_type() == at::kFloat && ids.is_contiguous() && weights.is_contiguous(), "ids int32, weights fp32");
  c10::cuda::CUDAGuard guard(logits.device());
  fllm::moe_route(logits.data_ptr(), logits.stride(0), optp(bias), (int)logits.size(0), (int)logits.size(1), (int)k,
                  softmax_all ? 1 : 0, ids.data_ptr<int>(), weights.data_ptr<float>(), cur_stream());
}

void moe_align(const Tensor& ids, int64_t experts, int64_t expert_lo, int64_t expert_hi, int64_t bn, Tensor row_of,
               Tensor token_of, Tensor tile_expert, Tensor tile_row0, Tensor num_tiles) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kInt && ids.dim() == 2 && ids.is_contiguous(), "ids: [tokens, k] int32");
  TORCH_CHECK(num_tiles.numel() >= 2, "num_tiles needs two ints");
  c10::cuda::CUDAGuard guard(ids.device());
  fllm::moe_align(ids.data_ptr<int>(), (int)ids.size(0), (int)ids.size(1), (int)experts, (int)expert_lo, (int)expert_hi,
                  (int)bn, row_of.data_ptr<int>(), token_of.data_ptr<int>(), (int)token_of.numel(),
                  tile_expert.data_ptr<int>(), tile_row0.data_ptr<int>(), num_tiles.data_ptr<int>(),
                  (int)tile_expert.numel(), cur_stream());
}

void moe_gather(const Tensor& x, const Tensor& token_of, Tensor xp) {
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.stride(1) == 1 && xp.is_contiguous() && xp.size(1) == x.size(1), "moe_gather: shapes");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::moe_gather(x.data_ptr(), x.stride(0), token_of.data_ptr<int>(), xp.data_ptr(), (int)xp.size(0), (int)x.size(1), cur_stream());
}

// w_stack: [experts, n_out, K]; xp: [rows_cap, K]; y: [rows_cap, n_out]
int64_t moe_grouped_linear(const Tensor& xp, const Tensor& w_stack, const optional<Tensor>& bias_stack, Tensor y,
                           const Tensor& tile_expert, const Tensor& tile_row0, const Tensor& num_tiles, int64_t bn,
                           const optional<Tensor>& status) {
  TORCH_CHECK(w_stack.dim() == 3 && w_stack.is_contiguous() && w_stack.scalar_type() == at::kBFloat16, "w_stack: contiguous [E, n, k] bf16");
  TORCH_CHECK(xp.dim() == 2 && xp.stride(1) == 1 && xp.size(1) == w_stack.size(2), "xp: [rows, k]");
  TORCH_CHECK(y.dim() == 2 && y.stride(1) == 1 && y.size(0) == xp.size(0) && y.size(1) == w_stack.size(1), "y: [rows, n]");
  c10::cuda::CUDAGuard guard(xp.device());
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  return fllm::moe_grouped_linear_bf16(xp.data_ptr(), xp.stride(0), w_stack.data_ptr(), w_stack.stride(1), optp(bias_stack),
                                       y.data_ptr(), y.stride(0), (int)xp.size(0), (int)w_stack.size(1), (int)w_stack.size(2),
                                       (int)w_stack.size(0), tile_expert.data_ptr<int>(), tile_row0.data_ptr<int>(),
                                       num_tiles.data_ptr<int>(), (int)tile_expert.numel(), (int)bn, st, cur_stream());
}

void moe_combine(const Tensor& y, const Tensor& row_of, const Tensor& weights, Tensor out) {
  TORCH_CHECK(y.stride(1) == 1 && out.stride(1) == 1 && y.size(1) == out.size(1), "moe_combine: shapes");
  c10::cuda::CUDAGuard guard(y.device());
  fllm::moe_combine(y.data_ptr(), y.stride(0), row_of.data_ptr<int>(), weights.data_ptr<float>(), (int)out.size(0),
                    (int)row_of.size(1), out.data_ptr(), out.stride(0), (int)out.size(1), cur_stream());
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(fllm_b200, m) {
  m.def("moe_route(Tensor logits, Tensor? bias, int k, bool softmax_all, Tensor(a!) ids, Tensor(b!) weights) -> ()", &moe_route);
  m.def("moe_align(Tensor ids, int experts, int expert_lo, int expert_hi, int bn, Tensor(a!) row_of, Tensor(b!) token_of, Tensor(c!) tile_expert, Tensor(d!) tile_row0, Tensor(e!) num_tiles) -> ()", &moe_align);
  m.def("moe_gather(Tensor x, Tensor token_of, Tensor(a!) xp) -> ()", &moe_gather);
  m.def("moe_grouped_linear(Tensor xp, Tensor w_stack, Tensor? bias_stack, Tensor(a!) y, Tensor tile_expert, Tensor tile_row0, Tensor num_tiles, int bn, Tensor? status) -> int", &moe_grouped_linear);
  m.def("moe_combine(Tensor y, Tensor row_of, Tensor weights, Tensor(a!) out) -> ()", &moe_combine);
}
