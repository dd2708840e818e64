// torch.ops.fllm_b200 bindings of the mixture-of-experts kernels.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <vector>

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

void moe_route_scored(const Tensor& logits, const optional<Tensor>& select_bias, int64_t k, int64_t score_kind, bool renorm, double scale,
                      Tensor ids, Tensor weights) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 && logits.stride(1) == 1, "logits: bf16 rows");
  TORCH_CHECK(ids.scalar_type() == at::kInt && weights.scalar_type() == at::kFloat && ids.is_contiguous() && weights.is_contiguous(), "ids int32, weights fp32");
  const float* sb = nullptr;
  if (select_bias.has_value() && select_bias->defined()) {
    TORCH_CHECK(select_bias->scalar_type() == at::kFloat && select_bias->is_contiguous() && select_bias->numel() == logits.size(1), "select_bias: fp32 [experts]");
    sb = select_bias->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(logits.device());
  fllm::moe_route_scored(logits.data_ptr(), logits.stride(0), sb, (int)logits.size(0), (int)logits.size(1), (int)k, (int)score_kind,
                         renorm ? 1 : 0, (float)scale, ids.data_ptr<int>(), weights.data_ptr<float>(), cur_stream());
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

// Same over packed 4-bit expert stacks: codes [E, n, k/2] bytes, scales [E, n, k/16] (NVFP4), [E, n, k/32] (MXFP4)
// bytes or [E, n, k/32, 2] bf16 (INT4 group-affine).
int64_t moe_grouped_linear_w4(const Tensor& xp, const Tensor& codes, const Tensor& scales, int64_t fmt, double alpha,
                              const optional<Tensor>& bias_stack, Tensor y, const Tensor& tile_expert,
                              const Tensor& tile_row0, const Tensor& num_tiles, int64_t bn, const optional<Tensor>& status) {
  TORCH_CHECK(codes.dim() == 3 && codes.is_contiguous() && codes.element_size() == 1, "codes: contiguous [E, n, k/2] bytes");
  TORCH_CHECK(scales.is_contiguous() && scales.is_cuda(), "scales: contiguous device tensor");
  TORCH_CHECK(xp.dim() == 2 && xp.stride(1) == 1 && xp.size(1) == codes.size(2) * 2 && xp.scalar_type() == at::kBFloat16, "xp: [rows, k] bf16");
  TORCH_CHECK(y.dim() == 2 && y.stride(1) == 1 && y.size(0) == xp.size(0) && y.size(1) == codes.size(1), "y: [rows, n]");
  c10::cuda::CUDAGuard guard(xp.device());
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  return fllm::moe_grouped_linear_w4(xp.data_ptr(), xp.stride(0), codes.data_ptr(), scales.data_ptr(), (int)fmt, (float)alpha,
                                     optp(bias_stack), y.data_ptr(), y.stride(0), (int)xp.size(0), (int)codes.size(1),
                                     (int)codes.size(2) * 2, (int)codes.size(0), tile_expert.data_ptr<int>(),
                                     tile_row0.data_ptr<int>(), num_tiles.data_ptr<int>(), (int)tile_expert.numel(), (int)bn,
                                     st, cur_stream());
}

void moe_combine(const Tensor& y, const Tensor& row_of, const Tensor& weights, Tensor out) {
  TORCH_CHECK(y.stride(1) == 1 && out.stride(1) == 1 && y.size(1) == out.size(1), "moe_combine: shapes");
  c10::cuda::CUDAGuard guard(y.device());
  fllm::moe_combine(y.data_ptr(), y.stride(0), row_of.data_ptr<int>(), weights.data_ptr<float>(), (int)out.size(0),
                    (int)row_of.size(1), out.data_ptr(), out.stride(0), (int)out.size(1), cur_stream());
}

// ---- expert-parallel all-to-all: a context of every rank's buffer addresses, then the four steps
std::vector<fllm::EpArgs> g_ep;

int64_t ep_ctx_create(int64_t ranks, int64_t my_rank, int64_t cap, int64_t hidden, int64_t experts_per_rank,
                      std::vector<int64_t> recv_x, std::vector<int64_t> recv_meta, std::vector<int64_t> ctrl,
                      std::vector<int64_t> comb_y) {
  TORCH_CHECK(ranks >= 1 && ranks <= fllm::kMaxEp, "1..8 ranks");
  TORCH_CHECK((int64_t)recv_x.size() == ranks && (int64_t)recv_meta.size() == ranks && (int64_t)ctrl.size() == ranks &&
              (int64_t)comb_y.size() == ranks, "one address per rank expected");
  fllm::EpArgs a{};
  for (int i = 0; i < ranks; ++i) {
    a.recv_x[i] = reinterpret_cast<void*>(recv_x[i]);
    a.recv_meta[i] = reinterpret_cast<void*>(recv_meta[i]);
    a.ctrl[i] = reinterpret_cast<void*>(ctrl[i]);
    a.comb_y[i] = reinterpret_cast<void*>(comb_y[i]);
  }
  a.ranks = (int)ranks; a.my_rank = (int)my_rank; a.cap = (int)cap; a.hidden = (int)hidden;
  a.experts_per_rank = (int)experts_per_rank;
  g_ep.push_back(a);
  return (int64_t)g_ep.size() - 1;
}

// the rank's call counter: one int32 / uint32 in device memory, or none (host-passed call number)
unsigned* ctr_ptr(const optional<Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->element_size() == 4 && t->numel() >= 1, "call counter: one 32-bit integer on the device");
  return reinterpret_cast<unsigned*>(t->data_ptr());
}

const fllm::EpArgs& ep_at(int64_t h) {
  TORCH_CHECK(h >= 0 && h < (int64_t)g_ep.size(), "invalid expert-parallel context handle");
  return g_ep[h];
}

void ep_dispatch(int64_t h, const Tensor& x, const Tensor& ids, int64_t epoch, const optional<Tensor>& status,
                 const optional<Tensor>& call_ctr) {
  const auto& a = ep_at(h);
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 && x.size(1) == a.hidden, "x: [tokens, hidden] bf16");
  TORCH_CHECK(ids.scalar_type() == at::kInt && ids.is_contiguous() && ids.dim() == 2 && ids.size(0) == x.size(0), "ids: [tokens, k] int32");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::ep_dispatch(a, x.data_ptr(), x.stride(0), ids.data_ptr<int>(), (int)x.size(0), (int)ids.size(1), (unsigned)epoch, ctr_ptr(call_ctr),
                    status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr, cur_stream());
}

void ep_ingest(int64_t h, int64_t epoch, Tensor ids_out, Tensor count_out, const optional<Tensor>& status,
               const optional<Tensor>& call_ctr) {
  const auto& a = ep_at(h);
  TORCH_CHECK(ids_out.scalar_type() == at::kInt && ids_out.is_contiguous() && ids_out.numel() == a.cap, "ids_out: [cap] int32");
  TORCH_CHECK(count_out.scalar_type() == at::kInt && count_out.numel() >= 1, "count_out: int32");
  c10::cuda::CUDAGuard guard(ids_out.device());
  fllm::ep_ingest(a, (unsigned)epoch, ctr_ptr(call_ctr), ids_out.data_ptr<int>(), count_out.data_ptr<int>(),
                  status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr, cur_stream());
}

void ep_return(int64_t h, const Tensor& y, const Tensor& row_of, const Tensor& count, int64_t epoch,
               const optional<Tensor>& call_ctr) {
  const auto& a = ep_at(h);
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.stride(1) == 1 && y.size(1) == a.hidden, "y: [rows, hidden] bf16");
  TORCH_CHECK(row_of.scalar_type() == at::kInt && row_of.is_contiguous() && row_of.numel() == a.cap, "row_of: [cap] int32");
  c10::cuda::CUDAGuard guard(y.device());
  fllm::ep_return(a, y.data_ptr(), y.stride(0), row_of.data_ptr<int>(), count.data_ptr<int>(), (unsigned)epoch, ctr_ptr(call_ctr),
                  cur_stream());
}

void ep_wait_returns(int64_t h, int64_t epoch, const Tensor& status, const optional<Tensor>& call_ctr) {
  c10::cuda::CUDAGuard guard(status.device());
  fllm::ep_wait_returns(ep_at(h), (unsigned)epoch, ctr_ptr(call_ctr), status.data_ptr<int>(), cur_stream());
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(fllm_b200, m) {
  m.def("moe_route_scored(Tensor logits, Tensor? select_bias, int k, int score_kind, bool renorm, float scale, Tensor(a!) ids, Tensor(b!) weights) -> ()",
        &moe_route_scored);
  m.def("moe_route(Tensor logits, Tensor? bias, int k, bool softmax_all, Tensor(a!) ids, Tensor(b!) weights) -> ()", &moe_route);
  m.def("moe_align(Tensor ids, int experts, int expert_lo, int expert_hi, int bn, Tensor(a!) row_of, Tensor(b!) token_of, Tensor(c!) tile_expert, Tensor(d!) tile_row0, Tensor(e!) num_tiles) -> ()", &moe_align);
  m.def("moe_gather(Tensor x, Tensor token_of, Tensor(a!) xp) -> ()", &moe_gather);
  m.def("moe_grouped_linear(Tensor xp, Tensor w_stack, Tensor? bias_stack, Tensor(a!) y, Tensor tile_expert, Tensor tile_row0, Tensor num_tiles, int bn, Tensor? status) -> int", &moe_grouped_linear);
  m.def("moe_grouped_linear_w4(Tensor xp, Tensor codes, Tensor scales, int fmt, float alpha, Tensor? bias_stack, Tensor(a!) y, Tensor tile_expert, Tensor tile_row0, Tensor num_tiles, int bn, Tensor? status) -> int", &moe_grouped_linear_w4);
  m.def("moe_combine(Tensor y, Tensor row_of, Tensor weights, Tensor(a!) out) -> ()", &moe_combine);
  m.def("ep_ctx_create(int ranks, int my_rank, int cap, int hidden, int experts_per_rank, int[] recv_x, int[] recv_meta, int[] ctrl, int[] comb_y) -> int", &ep_ctx_create);
  m.def("ep_dispatch(int ctx, Tensor x, Tensor ids, int epoch, Tensor? status, Tensor(a!)? call_ctr=None) -> ()", &ep_dispatch);
  m.def("ep_ingest(int ctx, int epoch, Tensor(a!) ids_out, Tensor(b!) count_out, Tensor? status, Tensor? call_ctr=None) -> ()", &ep_ingest);
  m.def("ep_return(int ctx, Tensor y, Tensor row_of, Tensor count, int epoch, Tensor? call_ctr=None) -> ()", &ep_return);
  m.def("ep_wait_returns(int ctx, int epoch, Tensor(a!) status, Tensor? call_ctr=None) -> ()", &ep_wait_returns);
}
