// torch.ops.fllm_b200 bindings of the tensor-parallel kernels: symmetric (IPC) buffers, a
// per-process context holding every rank's buffer and flag addresses, and the three fused
// steps (GEMM -> reduce-scatter, reduce + norm + all-gather, all-gather -> GEMM).
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <mutex>
#include <vector>

#include "fllm_ops.h"

namespace {

using at::Tensor;
using c10::optional;

inline cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

// word offsets inside a rank's flag buffer (uint32). The first three groups are written by
// peers; the rest is local bookkeeping.
enum : int { kRsFlags = 0, kAgFlags = 8, kArFlags = 16, kRsConsumed = 24, kAgConsumed = 32, kArConsumed = 40,
             kGemmDone = 48, kNormDone = 49, kArDone = 50, kFlagWords = 64 };

struct TpContext {
  int tp = 1, rank = 0, hidden = 0, max_tokens = 0, device = 0;
  int bcast_rows = 0;        // row capacity per source of the receive buffer in broadcast mode
  void* rs_bufs[8] = {nullptr};
  void* ag_bufs[8] = {nullptr};
  uint32_t* flags[8] = {nullptr};
  void* ar_slots[8] = {nullptr};
  size_t ar_slot_bytes = 0;
  int* status = nullptr;
};

std::mutex g_mu;
std::vector<TpContext> g_ctx;

TpContext& ctx_at(int64_t h) {
  std::lock_guard<std::mutex> l(g_mu);
  TORCH_CHECK(h >= 0 && h < (int64_t)g_ctx.size(), "invalid tensor-parallel context handle");
  return g_ctx[h];
}

int64_t symm_alloc(int64_t bytes) { return reinterpret_cast<int64_t>(fllm::symm_alloc((size_t)bytes)); }
void symm_free(int64_t p) { fllm::symm_free(reinterpret_cast<void*>(p)); }

Tensor symm_export(int64_t p) {
  Tensor t = at::empty({64}, at::kByte);
  fllm::symm_export(reinterpret_cast<void*>(p), t.data_ptr<uint8_t>());
  return t;
}

int64_t symm_import(const Tensor& handle) {
  TORCH_CHECK(!handle.is_cuda() && handle.scalar_type() == at::kByte && handle.numel() == 64, "bad IPC handle");
  return reinterpret_cast<int64_t>(fllm::symm_import(handle.contiguous().data_ptr<uint8_t>()));
}

void symm_close(int64_t p) { fllm::symm_close(reinterpret_cast<void*>(p)); }

// View of device memory we own elsewhere (no ownership transfer).
Tensor symm_view(int64_t p, int64_t bytes, int64_t device) {
  auto opts = at::TensorOptions().dtype(at::kByte).device(at::kCUDA, (c10::DeviceIndex)device);
  return at::from_blob(reinterpret_cast<void*>(p), {bytes}, opts);
}

int64_t flag_words() { return kFlagWords; }

int64_t tp_ctx_create(int64_t tp, int64_t rank, int64_t hidden, int64_t max_tokens, int64_t bcast_rows, int64_t device,
                      std::vector<int64_t> rs_bufs, std::vector<int64_t> ag_bufs, std::vector<int64_t> flag_bufs,
                      std::vector<int64_t> ar_slots, int64_t ar_slot_bytes, const Tensor& status) {
  TORCH_CHECK(tp >= 1 && tp <= 8, "tensor-parallel degree must be in [1, 8]");
  TORCH_CHECK((int64_t)rs_bufs.size() == tp && (int64_t)ag_bufs.size() == tp && (int64_t)flag_bufs.size() == tp &&
              (int64_t)ar_slots.size() == tp, "one address per rank expected");
  TpContext c;
  c.tp = (int)tp; c.rank = (int)rank; c.hidden = (int)hidden; c.max_tokens = (int)max_tokens; c.device = (int)device;
  c.bcast_rows = (int)bcast_rows;
  for (int i = 0; i < tp; ++i) {
    c.rs_bufs[i] = reinterpret_cast<void*>(rs_bufs[i]);
    c.ag_bufs[i] = reinterpret_cast<void*>(ag_bufs[i]);
    c.flags[i] = reinterpret_cast<uint32_t*>(flag_bufs[i]);
    c.ar_slots[i] = reinterpret_cast<void*>(ar_slots[i]);
  }
  c.ar_slot_bytes = (size_t)ar_slot_bytes;
  c.status = status.data_ptr<int>();
  std::lock_guard<std::mutex> l(g_mu);
  g_ctx.push_back(c);
  return (int64_t)g_ctx.size() - 1;
}

int64_t rows_per(const TpContext& c, int64_t tokens) { return (tokens + c.tp - 1) / c.tp; }

// Row-parallel linear whose partial sums go straight to the owning ranks (no local output).
int64_t tp_linear_rs(int64_t h, const Tensor& x, const Tensor& w, const optional<Tensor>& bias,
                     const optional<Tensor>& workspace, bool bcast) {
  TpContext& c = ctx_at(h);
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "x: bf16 rows");
  TORCH_CHECK(w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.stride(1) == 1 && w.size(0) == c.hidden, "w: [hidden, k]");
  TORCH_CHECK(x.size(0) <= c.max_tokens, "more tokens than the tensor-parallel buffers hold");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::TpLinearArgs a{};
  a.tp = c.tp; a.my_rank = c.rank; a.rows_per = bcast ? c.bcast_rows : (int)rows_per(c, x.size(0)); a.rs_ld = c.hidden;
  a.rs_bcast = bcast ? 1 : 0;
  TORCH_CHECK(!bcast || x.size(0) <= c.bcast_rows, "too many tokens for the broadcast receive buffer");
  for (int i = 0; i < c.tp; ++i) { a.rs_bufs[i] = c.rs_bufs[i]; a.rs_flags[i] = c.flags[i] + kRsFlags; }
  const void* b = bias.has_value() && bias->defined() ? bias->data_ptr() : nullptr;
  void* ws = nullptr;
  size_t ws_bytes = 0;
  if (workspace.has_value() && workspace->defined()) { ws = workspace->data_ptr(); ws_bytes = workspace->nbytes(); }
  int expected = 0;
  a.expected_out = &expected;
  fllm::linear_bf16_tp(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), b, nullptr, c.hidden,
                       (int)x.size(0), (int)w.size(0), (int)x.size(1), ws, ws_bytes, c.status, 0, &a, cur_stream());
  return expected;      // what the consumer's norm kernel has to wait for from every source rank
}

// Column-parallel linear whose activation operand is the gathered buffer peers fill.
int64_t tp_linear_ag(int64_t h, int64_t tokens, const Tensor& w, const optional<Tensor>& bias, Tensor y,
                     const optional<Tensor>& workspace) {
  TpContext& c = ctx_at(h);
  TORCH_CHECK(w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.stride(1) == 1 && w.size(1) == c.hidden, "w: [n, hidden]");
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.stride(1) == 1 && y.size(0) == tokens &&
              y.size(1) == w.size(0), "y: [tokens, n]");
  TORCH_CHECK(tokens <= c.max_tokens, "more tokens than the tensor-parallel buffers hold");
  c10::cuda::CUDAGuard guard(y.device());
  fllm::TpLinearArgs a{};
  a.tp = c.tp; a.my_rank = c.rank; a.rows_per = (int)rows_per(c, tokens);
  uint32_t* f = c.flags[c.rank];
  a.ag_flags = f + kAgFlags; a.ag_consumed = f + kAgConsumed; a.cta_done = f + kGemmDone;
  void* ws = nullptr;
  size_t ws_bytes = 0;
  if (workspace.has_value() && workspace->defined()) { ws = workspace->data_ptr(); ws_bytes = workspace->nbytes(); }
  const void* b = bias.has_value() && bias->defined() ? bias->data_ptr() : nullptr;
  return fllm::linear_bf16_tp(c.ag_bufs[c.rank], c.hidden, w.data_ptr(), w.stride(0), b, y.data_ptr(), y.stride(0),
                              (int)tokens, (int)w.size(0), c.hidden, ws, ws_bytes, c.status, 0, &a, cur_stream());
}

// residual_shard (+= reduced partials) -> RMSNorm -> every rank's gathered buffer.
void tp_norm(int64_t h, Tensor residual_shard, int64_t tokens, int64_t expected, const Tensor& norm_w, double eps,
             double w_offset, bool bcast) {
  const bool has_partials = expected > 0;
  TpContext& c = ctx_at(h);
  TORCH_CHECK(residual_shard.scalar_type() == at::kBFloat16 && residual_shard.is_contiguous(), "residual shard: contiguous bf16");
  TORCH_CHECK(tokens <= c.max_tokens, "more tokens than the tensor-parallel buffers hold");
  c10::cuda::CUDAGuard guard(residual_shard.device());
  fllm::TpNormArgs a{};
  a.residual = residual_shard.data_ptr();
  uint32_t* f = c.flags[c.rank];
  a.rs_buf = has_partials ? c.rs_bufs[c.rank] : nullptr;
  a.rs_flags = f + kRsFlags; a.rs_consumed = f + kRsConsumed;
  a.tp = c.tp; a.my_rank = c.rank; a.rows_per = bcast ? c.bcast_rows : (int)rows_per(c, tokens); a.tokens = (int)tokens; a.hidden = c.hidden;
  a.bcast = bcast ? 1 : 0;
  a.rs_expected = (uint32_t)expected;
  a.norm_w = norm_w.data_ptr(); a.eps = (float)eps; a.w_offset = (float)w_offset;
  for (int i = 0; i < c.tp; ++i) { a.ag_bufs[i] = c.ag_bufs[i]; a.ag_flags[i] = c.flags[i] + kAgFlags; }
  a.cta_done = f + kNormDone; a.status = c.status;
  const int my_rows = bcast ? (int)tokens : (int)std::max<int64_t>(0, std::min<int64_t>(tokens, (int64_t)(c.rank + 1) * a.rows_per) - (int64_t)c.rank * a.rows_per);
  TORCH_CHECK(residual_shard.numel() >= (int64_t)my_rows * c.hidden, "residual shard too small");
  fllm::tp_reduce_norm_allgather(a, cur_stream());
}

void tp_allreduce(int64_t h, const Tensor& input, Tensor output) {
  TpContext& c = ctx_at(h);
  TORCH_CHECK(input.is_contiguous() && output.is_contiguous() && input.nbytes() == output.nbytes(), "tp_allreduce: shapes");
  const bool f32 = input.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || input.scalar_type() == at::kBFloat16, "tp_allreduce: fp32 or bf16");
  c10::cuda::CUDAGuard guard(input.device());
  fllm::TpAllReduceArgs a{};
  a.input = input.data_ptr(); a.output = output.data_ptr(); a.bytes = input.nbytes(); a.slot_bytes = c.ar_slot_bytes;
  a.is_fp32 = f32; a.tp = c.tp; a.my_rank = c.rank;
  for (int i = 0; i < c.tp; ++i) { a.slots[i] = c.ar_slots[i]; a.flags[i] = c.flags[i] + kArFlags; }
  uint32_t* f = c.flags[c.rank];
  a.my_flags = f + kArFlags; a.consumed = f + kArConsumed; a.cta_done = f + kArDone; a.status = c.status;
  fllm::tp_allreduce(a, cur_stream());
}

// output [tp, ...input shape]: every rank's `input`, through the same peer slots and flags.
void tp_allgather(int64_t h, const Tensor& input, Tensor output) {
  TpContext& c = ctx_at(h);
  TORCH_CHECK(input.is_contiguous() && output.is_contiguous() && output.nbytes() == input.nbytes() * (size_t)c.tp, "tp_allgather: shapes");
  c10::cuda::CUDAGuard guard(input.device());
  fllm::TpAllReduceArgs a{};
  a.input = input.data_ptr(); a.output = output.data_ptr(); a.bytes = input.nbytes(); a.slot_bytes = c.ar_slot_bytes;
  a.is_fp32 = 1; a.gather = 1; a.tp = c.tp; a.my_rank = c.rank;
  for (int i = 0; i < c.tp; ++i) { a.slots[i] = c.ar_slots[i]; a.flags[i] = c.flags[i] + kArFlags; }
  uint32_t* f = c.flags[c.rank];
  a.my_flags = f + kArFlags; a.consumed = f + kArConsumed; a.cta_done = f + kArDone; a.status = c.status;
  fllm::tp_allreduce(a, cur_stream());
}

int64_t linear_rs_expected(int64_t tokens, int64_t n, int64_t rows_per, int64_t dest) {
  return fllm::linear_rs_expected_signals((int)tokens, (int)n, (int)rows_per, (int)dest);
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(fllm_b200, m) {
  m.def("symm_alloc(int bytes) -> int", &symm_alloc);
  m.def("symm_free(int ptr) -> ()", &symm_free);
  m.def("symm_export(int ptr) -> Tensor", &symm_export);
  m.def("symm_import(Tensor handle) -> int", &symm_import);
  m.def("symm_close(int ptr) -> ()", &symm_close);
  m.def("symm_view(int ptr, int bytes, int device) -> Tensor", &symm_view);
  m.def("flag_words() -> int", &flag_words);
  m.def("tp_ctx_create(int tp, int rank, int hidden, int max_tokens, int bcast_rows, int device, int[] rs_bufs, int[] ag_bufs, int[] flag_bufs, int[] ar_slots, int ar_slot_bytes, Tensor status) -> int", &tp_ctx_create);
  m.def("tp_linear_rs(int ctx, Tensor x, Tensor w, Tensor? bias, Tensor? workspace, bool bcast) -> int", &tp_linear_rs);
  m.def("tp_linear_ag(int ctx, int tokens, Tensor w, Tensor? bias, Tensor(a!) y, Tensor? workspace) -> int", &tp_linear_ag);
  m.def("tp_norm(int ctx, Tensor(a!) residual_shard, int tokens, int expected, Tensor norm_w, float eps, float w_offset, bool bcast) -> ()", &tp_norm);
  m.def("tp_allreduce(int ctx, Tensor input, Tensor(a!) output) -> ()", &tp_allreduce);
  m.def("tp_allgather(int ctx, Tensor input, Tensor(a!) output) -> ()", &tp_allgather);
  m.def("linear_rs_expected(int tokens, int n, int rows_per, int dest) -> int", &linear_rs_expected);
}
