// torch.ops.fllm_b200 bindings of the low-precision GEMMs (block-scaled FP8; FP4 formats).
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include "fllm_ops.h"

namespace {
using at::Tensor;
using c10::optional;
inline cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

// x bf16 [T, K] -> (xq uint8 [T, K] holding e4m3, sx fp32 [T, K/128])
void quant_fp8_1x128(const Tensor& x, Tensor xq, Tensor sx) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "x: bf16 rows");
  TORCH_CHECK(xq.is_contiguous() && xq.element_size() == 1 && xq.numel() == x.numel(), "xq: contiguous 1-byte [T, K]");
  TORCH_CHECK(sx.is_contiguous() && sx.scalar_type() == at::kFloat && sx.numel() == x.size(0) * (x.size(1) / 128), "sx: [T, K/128]");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::quant_fp8_1x128(x.data_ptr(), x.stride(0), xq.data_ptr(), sx.data_ptr<float>(), (int)x.size(0), (int)x.size(1), cur_stream());
}

int64_t linear_fp8_block(const Tensor& xq, const Tensor& sx, const Tensor& wq, const Tensor& sw, const optional<Tensor>& bias,
                         Tensor y, const optional<Tensor>& status, const optional<Tensor>& workspace) {
  TORCH_CHECK(xq.is_cuda() && xq.is_contiguous() && wq.is_contiguous() && xq.element_size() == 1 && wq.element_size() == 1, "xq, wq: contiguous e4m3 bytes");
  TORCH_CHECK(xq.dim() == 2 && wq.dim() == 2 && xq.size(1) == wq.size(1), "K mismatch");
  const int64_t T = xq.size(0), N = wq.size(0), K = xq.size(1);
  TORCH_CHECK(sx.scalar_type() == at::kFloat && sx.is_contiguous() && sx.numel() == T * (K / 128), "sx: [T, K/128]");
  TORCH_CHECK(sw.scalar_type() == at::kFloat && sw.is_contiguous() && sw.numel() == (N / 128) * (K / 128), "sw: [N/128, K/128]");
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.stride(1) == 1 && y.size(0) == T && y.size(1) == N, "y: [T, N] bf16");
  c10::cuda::CUDAGuard guard(xq.device());
  const void* b = bias.has_value() && bias->defined() ? bias->data_ptr() : nullptr;
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  void* ws = nullptr;
  size_t ws_bytes = 0;                 // the first 64 KiB of the shared workspace hold the dense GEMM's tile counters
  if (workspace.has_value() && workspace->defined() && workspace->numel() * workspace->element_size() > (64 << 10)) {
    ws = static_cast<char*>(workspace->data_ptr()) + (64 << 10);
    ws_bytes = workspace->numel() * workspace->element_size() - (64 << 10);
  }
  return fllm::linear_fp8_block(xq.data_ptr(), sx.data_ptr<float>(), wq.data_ptr(), sw.data_ptr<float>(), b, y.data_ptr(),
                                y.stride(0), (int)T, (int)N, (int)K, st, cur_stream(), ws, ws_bytes);
}

// codes uint8 [N, K/2]; scales uint8 [N, K/16] e4m3 (fmt 0), [N, K/32] e8m0 (fmt 1) or bf16 [N, K/32, 2] = {scale, min} (fmt 2)
int64_t linear_w4a16(const Tensor& x, const Tensor& codes, const Tensor& scales, int64_t fmt, double alpha,
                     const optional<Tensor>& bias, Tensor y, const optional<Tensor>& workspace, const optional<Tensor>& status) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "x: bf16 rows");
  TORCH_CHECK(codes.is_contiguous() && codes.element_size() == 1 && codes.dim() == 2 && codes.size(1) * 2 == x.size(1), "codes: [N, K/2] bytes");
  const int64_t T = x.size(0), N = codes.size(0), K = x.size(1);
  TORCH_CHECK(scales.is_contiguous() && scales.numel() * scales.element_size() == N * (K / (fmt == 0 ? 16 : 32)) * (fmt == 2 ? 4 : 1),
              "scales: one byte per block (FP4) or {bf16 scale, bf16 min} per 32 values (INT4G)");
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.stride(1) == 1 && y.size(0) == T && y.size(1) == N, "y: [T, N] bf16");
  c10::cuda::CUDAGuard guard(x.device());
  const void* b = bias.has_value() && bias->defined() ? bias->data_ptr() : nullptr;
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  // the first 64 KiB of the shared workspace hold the dense GEMM's tile counters: partial sums go after them
  void* ws = nullptr;
  size_t ws_bytes = 0;
  if (workspace.has_value() && workspace->defined() && workspace->numel() * workspace->element_size() > (64 << 10)) {
    ws = static_cast<char*>(workspace->data_ptr()) + (64 << 10);
    ws_bytes = workspace->numel() * workspace->element_size() - (64 << 10);
  }
  return fllm::linear_w4a16(x.data_ptr(), x.stride(0), codes.data_ptr(), scales.data_ptr(), (int)fmt, (float)alpha, b,
                            y.data_ptr(), y.stride(0), (int)T, (int)N, (int)K, ws, ws_bytes, st, cur_stream());
}

// x bf16 [T, K] -> xq uint8 [T, K] (e4m3) + sf uint8 [mx_act_scale_bytes(T, K, 0)] (e8m0 atoms per token tile)
void quant_mx(const Tensor& x, Tensor xq, Tensor sf) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 && x.stride(0) % 4 == 0, "x: bf16 rows");
  TORCH_CHECK(xq.is_contiguous() && xq.element_size() == 1 && xq.numel() == x.numel(), "xq: contiguous 1-byte [T, K]");
  TORCH_CHECK(sf.is_contiguous() && sf.element_size() == 1 &&
              (size_t)sf.numel() >= fllm::mx_act_scale_bytes((int)x.size(0), (int)x.size(1), 0), "sf: too small");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::quant_mx(x.data_ptr(), x.stride(0), xq.data_ptr(), sf.data_ptr(), (int)x.size(0), (int)x.size(1), cur_stream());
}

// x bf16 [T, K] -> xq uint8 [T, K/2] (e2m1 pairs) + sf uint8 [mx_act_scale_bytes(T, K, 2)] (e4m3 atoms) + tok_scale fp32 [T]
void quant_nvfp4(const Tensor& x, Tensor xq, Tensor sf, Tensor tok_scale) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 && x.stride(0) % 8 == 0, "x: bf16 rows");
  TORCH_CHECK(xq.is_contiguous() && xq.element_size() == 1 && xq.numel() * 2 == x.numel(), "xq: contiguous bytes [T, K/2]");
  TORCH_CHECK(sf.is_contiguous() && sf.element_size() == 1 &&
              (size_t)sf.numel() >= fllm::mx_act_scale_bytes((int)x.size(0), (int)x.size(1), 2), "sf: too small");
  TORCH_CHECK(tok_scale.is_contiguous() && tok_scale.scalar_type() == at::kFloat && tok_scale.numel() >= x.size(0), "tok_scale: fp32 [T]");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::quant_nvfp4(x.data_ptr(), x.stride(0), xq.data_ptr(), sf.data_ptr(), tok_scale.data_ptr<float>(), (int)x.size(0),
                    (int)x.size(1), cur_stream());
}

int64_t mx_act_scale_bytes(int64_t T, int64_t K, int64_t kind) { return (int64_t)fllm::mx_act_scale_bytes((int)T, (int)K, (int)kind); }

// kind 0: wq e4m3 [N, K], xq e4m3 [T, K]; kind 1: wq e2m1 codes [N, K/2], xq e4m3 [T, K]; kind 2: both e2m1 codes.
// sfa: weight scale atoms [ceil(N/128), K/128 (K/64 for kind 2), 512]
void quant_rows_8bit(const Tensor& x, Tensor xq, Tensor tok_scale, bool is_int8) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 && x.stride(0) % 8 == 0 && x.size(1) % 8 == 0, "x: bf16 rows, K % 8 == 0");
  TORCH_CHECK(xq.is_contiguous() && xq.element_size() == 1 && xq.numel() == x.numel(), "xq: contiguous 1-byte [T, K]");
  TORCH_CHECK(tok_scale.is_contiguous() && tok_scale.scalar_type() == at::kFloat && tok_scale.numel() >= x.size(0), "tok_scale: fp32 [T]");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::quant_rows_8bit(x.data_ptr(), x.stride(0), xq.data_ptr(), tok_scale.data_ptr<float>(), (int)x.size(0), (int)x.size(1),
                        is_int8 ? 1 : 0, cur_stream());
}

// y = (xq * tok_scale) (wq * feat_scale)^T (+ bias): e4m3 (is_int8 false) or int8 codes on both sides, one scale per row
int64_t linear_w8a8(const Tensor& xq, const Tensor& tok_scale, const Tensor& wq, const Tensor& feat_scale, bool is_int8,
                    const optional<Tensor>& bias, Tensor y, const optional<Tensor>& workspace, const optional<Tensor>& status) {
  TORCH_CHECK(xq.is_cuda() && xq.is_contiguous() && wq.is_contiguous() && xq.element_size() == 1 && wq.element_size() == 1 &&
              xq.dim() == 2 && wq.dim() == 2 && xq.size(1) == wq.size(1) && xq.size(1) % 128 == 0, "xq, wq: contiguous byte matrices, K % 128 == 0");
  const int64_t T = xq.size(0), K = xq.size(1), N = wq.size(0);
  TORCH_CHECK(tok_scale.scalar_type() == at::kFloat && tok_scale.is_contiguous() && tok_scale.numel() >= T, "tok_scale: fp32 [T]");
  TORCH_CHECK(feat_scale.scalar_type() == at::kFloat && feat_scale.is_contiguous() && feat_scale.numel() == N, "feat_scale: fp32 [N]");
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.stride(1) == 1 && y.size(0) == T && y.size(1) == N, "y: [T, N] bf16");
  c10::cuda::CUDAGuard guard(xq.device());
  const void* b = bias.has_value() && bias->defined() ? bias->data_ptr() : nullptr;
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  void* ws = nullptr;
  size_t ws_bytes = 0;
  if (workspace.has_value() && workspace->defined() && workspace->numel() * workspace->element_size() > (64 << 10)) {
    ws = static_cast<char*>(workspace->data_ptr()) + (64 << 10);
    ws_bytes = workspace->numel() * workspace->element_size() - (64 << 10);
  }
  return fllm::linear_mx(xq.data_ptr(), nullptr, wq.data_ptr(), nullptr, is_int8 ? 4 : 3, 1.f, tok_scale.data_ptr<float>(),
                         feat_scale.data_ptr<float>(), b, y.data_ptr(), y.stride(0), (int)T, (int)N, (int)K, ws, ws_bytes, st,
                         cur_stream());
}

int64_t linear_mx(const Tensor& xq, const Tensor& sfb, const Tensor& wq, const Tensor& sfa, int64_t kind, double alpha,
                  const optional<Tensor>& tok_scale, const optional<Tensor>& bias, Tensor y, const optional<Tensor>& workspace,
                  const optional<Tensor>& status) {
  TORCH_CHECK(xq.is_cuda() && xq.is_contiguous() && wq.is_contiguous() && xq.element_size() == 1 && wq.element_size() == 1 &&
              xq.dim() == 2 && wq.dim() == 2, "xq, wq: contiguous byte matrices");
  TORCH_CHECK(kind >= 0 && kind <= 2, "kind: 0, 1 or 2");
  const int64_t T = xq.size(0), K = xq.size(1) * (kind == 2 ? 2 : 1), N = wq.size(0);
  const int64_t atom_k = kind == 2 ? 64 : 128;
  TORCH_CHECK(wq.size(1) * (kind == 0 ? 1 : 2) == K && K % (kind == 2 ? 256 : 128) == 0, "K mismatch (multiple of 128; 256 for NVFP4)");
  TORCH_CHECK(sfa.is_contiguous() && sfa.element_size() == 1 && sfa.numel() == ((N + 127) / 128) * (K / atom_k) * 512, "sfa: [ceil(N/128), K/atom, 512]");
  TORCH_CHECK(sfb.is_contiguous() && sfb.element_size() == 1 &&
              (size_t)sfb.numel() >= fllm::mx_act_scale_bytes((int)T, (int)K, (int)kind), "sfb: too small");
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.stride(1) == 1 && y.size(0) == T && y.size(1) == N, "y: [T, N] bf16");
  const float* ts = nullptr;
  if (tok_scale.has_value() && tok_scale->defined()) {
    TORCH_CHECK(tok_scale->scalar_type() == at::kFloat && tok_scale->is_contiguous() && tok_scale->numel() >= T, "tok_scale: fp32 [T]");
    ts = tok_scale->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(xq.device());
  const void* b = bias.has_value() && bias->defined() ? bias->data_ptr() : nullptr;
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  void* ws = nullptr;
  size_t ws_bytes = 0;
  if (workspace.has_value() && workspace->defined() && workspace->numel() * workspace->element_size() > (64 << 10)) {
    ws = static_cast<char*>(workspace->data_ptr()) + (64 << 10);
    ws_bytes = workspace->numel() * workspace->element_size() - (64 << 10);
  }
  return fllm::linear_mx(xq.data_ptr(), sfb.data_ptr(), wq.data_ptr(), sfa.data_ptr(), (int)kind, (float)alpha, ts, nullptr, b,
                         y.data_ptr(), y.stride(0), (int)T, (int)N, (int)K, ws, ws_bytes, st, cur_stream());
}

// the dp4a path of linear_w4a16 for at most 4 tokens (same operands)
int64_t gemv_w4(const Tensor& x, const Tensor& codes, const Tensor& scales, int64_t fmt, double alpha,
                const optional<Tensor>& bias, Tensor y) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "x: bf16 rows");
  TORCH_CHECK(codes.is_contiguous() && codes.element_size() == 1 && codes.dim() == 2 && codes.size(1) * 2 == x.size(1), "codes: [N, K/2] bytes");
  const int64_t T = x.size(0), N = codes.size(0), K = x.size(1);
  TORCH_CHECK(fllm::gemv_w4_supported((int)T, (int)K), "gemv_w4: at most 4 tokens, K % 32 == 0");
  TORCH_CHECK(scales.is_contiguous() && scales.numel() * scales.element_size() == N * (K / (fmt == 0 ? 16 : 32)) * (fmt == 2 ? 4 : 1),
              "scales: one byte per block (FP4) or {bf16 scale, bf16 min} per 32 values (INT4G)");
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.stride(1) == 1 && y.size(0) == T && y.size(1) == N, "y: [T, N] bf16");
  c10::cuda::CUDAGuard guard(x.device());
  const void* b = bias.has_value() && bias->defined() ? bias->data_ptr() : nullptr;
  return fllm::gemv_w4(x.data_ptr(), x.stride(0), codes.data_ptr(), scales.data_ptr(), (int)fmt, (float)alpha, b, y.data_ptr(),
                       y.stride(0), (int)T, (int)N, (int)K, cur_stream());
}

// planes of ops/intk.py: codes (low nibbles [N, K/2] or int8 [N, K]), high-bit words, sub-scales, fp16 super-scales
int64_t gemv_wk(const Tensor& x, const Tensor& codes, const Tensor& high, const Tensor& sub, const Tensor& sup, int64_t fmt,
                const optional<Tensor>& bias, Tensor y) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "x: bf16 rows");
  const int64_t T = x.size(0), K = x.size(1), N = codes.size(0);
  TORCH_CHECK(fllm::gemv_wk_supported((int)T, (int)K, (int)fmt), "gemv_wk: at most 4 tokens, fmt 5 / 6 / 8, K % 256 == 0 (32 for Q8_0)");
  TORCH_CHECK(codes.is_contiguous() && codes.element_size() == 1 && codes.dim() == 2 && codes.size(1) == (fmt == 8 ? K : K / 2), "codes: planar bytes");
  TORCH_CHECK(sup.is_contiguous() && sup.scalar_type() == at::kHalf && sup.numel() == N * (fmt == 8 ? K / 32 : (fmt == 5 ? K / 128 : K / 256)), "sup: fp16 super-scales");
  if (fmt != 8) {
    TORCH_CHECK(high.is_contiguous() && high.element_size() == 4 && high.numel() == N * (K / 32) * (fmt == 6 ? 2 : 1), "high: bit planes");
    TORCH_CHECK(sub.is_contiguous() && sub.element_size() == 1 && sub.numel() == N * (K / 16), "sub: one byte per 16 values");
  }
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.stride(1) == 1 && y.size(0) == T && y.size(1) == N, "y: [T, N] bf16");
  c10::cuda::CUDAGuard guard(x.device());
  const void* b = bias.has_value() && bias->defined() ? bias->data_ptr() : nullptr;
  return fllm::gemv_wk(x.data_ptr(), x.stride(0), codes.data_ptr(), high.data_ptr(), sub.data_ptr(), sup.data_ptr(), (int)fmt, b,
                       y.data_ptr(), y.stride(0), (int)T, (int)N, (int)K, cur_stream());
}

void wk_dequant(const Tensor& codes, const Tensor& high, const Tensor& sub, const Tensor& sup, int64_t fmt, Tensor out) {
  TORCH_CHECK(codes.is_cuda() && codes.is_contiguous() && codes.dim() == 2 && out.is_contiguous() && out.scalar_type() == at::kBFloat16 &&
              out.dim() == 2 && out.size(0) == codes.size(0), "codes planar bytes, out bf16 [N, K]");
  TORCH_CHECK(codes.size(1) == (fmt == 8 ? out.size(1) : out.size(1) / 2) && sup.scalar_type() == at::kHalf &&
              high.is_contiguous() && sub.is_contiguous() && sup.is_contiguous(), "plane shapes");
  c10::cuda::CUDAGuard guard(codes.device());
  fllm::wk_dequant_bf16(codes.data_ptr(), high.data_ptr(), sub.data_ptr(), sup.data_ptr(), (int)fmt, out.data_ptr(), out.size(0),
                        (int)out.size(1), cur_stream());
}

void w4_dequant(const Tensor& codes, const Tensor& scales, int64_t fmt, double alpha, Tensor out) {
  TORCH_CHECK(codes.is_cuda() && codes.is_contiguous() && codes.dim() == 2 && out.is_contiguous() && out.scalar_type() == at::kBFloat16, "codes [N, K/2], out bf16 [N, K]");
  TORCH_CHECK(out.numel() == codes.numel() * 2 && (codes.size(1) * 2) % 32 == 0, "out: [N, K], K % 32 == 0");
  c10::cuda::CUDAGuard guard(codes.device());
  fllm::w4_dequant_bf16(codes.data_ptr(), scales.data_ptr(), (int)fmt, (float)alpha, out.data_ptr(), codes.size(0),
                        (int)codes.size(1) * 2, cur_stream());
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(fllm_b200, m) {
  m.def("quant_fp8_1x128(Tensor x, Tensor(a!) xq, Tensor(b!) sx) -> ()", &quant_fp8_1x128);
  m.def("linear_fp8_block(Tensor xq, Tensor sx, Tensor wq, Tensor sw, Tensor? bias, Tensor(a!) y, Tensor? status, Tensor? workspace=None) -> int", &linear_fp8_block);
  m.def("linear_w4a16(Tensor x, Tensor codes, Tensor scales, int fmt, float alpha, Tensor? bias, Tensor(a!) y, Tensor? workspace, Tensor? status) -> int", &linear_w4a16);
  m.def("quant_mx(Tensor x, Tensor(a!) xq, Tensor(b!) sf) -> ()", &quant_mx);
  m.def("quant_rows_8bit(Tensor x, Tensor(a!) xq, Tensor(b!) tok_scale, bool is_int8) -> ()", &quant_rows_8bit);
  m.def("linear_w8a8(Tensor xq, Tensor tok_scale, Tensor wq, Tensor feat_scale, bool is_int8, Tensor? bias, Tensor(a!) y, Tensor? workspace, Tensor? status) -> int", &linear_w8a8);
  m.def("quant_nvfp4(Tensor x, Tensor(a!) xq, Tensor(b!) sf, Tensor(c!) tok_scale) -> ()", &quant_nvfp4);
  m.def("mx_act_scale_bytes(int T, int K, int kind) -> int", &mx_act_scale_bytes);
  m.def("linear_mx(Tensor xq, Tensor sfb, Tensor wq, Tensor sfa, int kind, float alpha, Tensor? tok_scale, Tensor? bias, Tensor(a!) y, Tensor? workspace, Tensor? status) -> int", &linear_mx);
  m.def("gemv_w4(Tensor x, Tensor codes, Tensor scales, int fmt, float alpha, Tensor? bias, Tensor(a!) y) -> int", &gemv_w4);
  m.def("gemv_wk(Tensor x, Tensor codes, Tensor high, Tensor sub, Tensor sup, int fmt, Tensor? bias, Tensor(a!) y) -> int", &gemv_wk);
  m.def("wk_dequant(Tensor codes, Tensor high, Tensor sub, Tensor sup, int fmt, Tensor(a!) out) -> ()", &wk_dequant);
  m.def("w4_dequant(Tensor codes, Tensor scales, int fmt, float alpha, Tensor(a!) out) -> ()", &w4_dequant);
}
