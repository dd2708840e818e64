// torch.ops.fllm_b200 bindings of the recurrent token mixers (recurrent.cu).
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include "fllm_ops.h"

namespace {
using at::Tensor;
using c10::optional;
inline cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }
inline bool rows_bf16(const Tensor& t) { return t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1; }
inline const void* opt_ptr(const optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }
inline const float* opt_f32(const optional<Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous(), "parameter vectors are contiguous fp32");
  return t->data_ptr<float>();
}
inline long long opt_ld(const optional<Tensor>& t) { return t.has_value() && t->defined() ? t->stride(0) : 0; }
inline void check_batch(const Tensor& q_starts, const Tensor& seq_state, const Tensor& positions) {
  TORCH_CHECK(q_starts.scalar_type() == at::kInt && seq_state.scalar_type() == at::kInt && positions.scalar_type() == at::kInt &&
                  q_starts.is_contiguous() && seq_state.is_contiguous() && positions.is_contiguous() &&
                  q_starts.numel() == seq_state.numel() + 1,
              "q_starts [B + 1], seq_state [B], positions [T]: contiguous int32");
}

void causal_conv1d(const Tensor& x, const Tensor& w, const optional<Tensor>& bias, Tensor state, const Tensor& q_starts,
                   const Tensor& seq_state, const Tensor& positions, Tensor y, bool act, int64_t max_q_len) {
  TORCH_CHECK(rows_bf16(x) && rows_bf16(y) && x.sizes() == y.sizes(), "x, y: bf16 rows of one shape");
  const int64_t C = x.size(1), W = w.size(1);
  TORCH_CHECK(w.scalar_type() == at::kFloat && w.is_contiguous() && w.dim() == 2 && w.size(0) == C, "w: fp32 [C, W]");
  TORCH_CHECK(state.scalar_type() == at::kBFloat16 && state.is_contiguous() && state.dim() == 3 && state.size(1) == W - 1 && state.size(2) == C,
              "state: bf16 [slots, W - 1, C]");
  check_batch(q_starts, seq_state, positions);
  c10::cuda::CUDAGuard guard(x.device());
  const int rc = fllm::causal_conv1d(x.data_ptr(), x.stride(0), w.data_ptr<float>(), opt_f32(bias), state.data_ptr(), q_starts.data_ptr<int>(),
                                     seq_state.data_ptr<int>(), positions.data_ptr<int>(), y.data_ptr(), y.stride(0), (int)seq_state.numel(),
                                     (int)C, (int)W, act ? 1 : 0, (int)(max_q_len > 0 ? max_q_len : x.size(0)), cur_stream());
  TORCH_CHECK(rc == 0, "causal_conv1d: unsupported arguments (code ", rc, "): even C and strides, 2 <= W <= 4, y distinct from x");
}

void mamba2_scan(const Tensor& x, const Tensor& dt, const Tensor& Bm, const Tensor& Cm, const Tensor& A, const optional<Tensor>& D,
                 const optional<Tensor>& dt_bias, Tensor state, const Tensor& q_starts, const Tensor& seq_state, const Tensor& positions,
                 Tensor y, int64_t H, int64_t P, int64_t G, int64_t N, double dt_min, double dt_max, int64_t seg_len, int64_t segs,
                 const optional<Tensor>& seg_scratch, int64_t skip_from) {
  TORCH_CHECK(rows_bf16(x) && rows_bf16(dt) && rows_bf16(Bm) && rows_bf16(Cm) && rows_bf16(y), "activations: bf16 rows");
  TORCH_CHECK(x.size(1) == H * P && y.size(1) == H * P && dt.size(1) == H && Bm.size(1) == G * N && Cm.size(1) == G * N, "widths");
  TORCH_CHECK(state.scalar_type() == at::kFloat && state.is_contiguous() && state.dim() == 4 && state.size(1) == H && state.size(2) == P &&
                  state.size(3) == N, "state: fp32 [slots, H, P, N]");
  check_batch(q_starts, seq_state, positions);
  c10::cuda::CUDAGuard guard(x.device());
  float *seg_state = nullptr, *seg_dt = nullptr;
  const int64_t B = seq_state.numel();
  if (seg_len > 0 && segs > 1) {                 // scratch: B * segs states of [H][P][N], then [B][segs - 1][H] step sums
    const int64_t n_state = B * segs * H * P * N, n_dt = B * (segs - 1) * H;
    TORCH_CHECK(seg_scratch.has_value() && seg_scratch->scalar_type() == at::kFloat && seg_scratch->is_contiguous() &&
                    seg_scratch->numel() >= n_state + n_dt, "seg_scratch: fp32, at least B * (segs * H * P * N + (segs - 1) * H) values");
    seg_state = seg_scratch->data_ptr<float>();
    seg_dt = seg_state + n_state;
  }
  const int rc = fllm::mamba2_scan(x.data_ptr(), x.stride(0), dt.data_ptr(), dt.stride(0), Bm.data_ptr(), Bm.stride(0), Cm.data_ptr(),
                                   Cm.stride(0), opt_f32(A), opt_f32(D), opt_f32(dt_bias), state.data_ptr<float>(), q_starts.data_ptr<int>(),
                                   seq_state.data_ptr<int>(), positions.data_ptr<int>(), y.data_ptr(), y.stride(0), (int)B,
                                   (int)H, (int)P, (int)G, (int)N, (float)dt_min, (float)dt_max, (int)seg_len, (int)segs, seg_state, seg_dt,
                                   (int)skip_from, cur_stream());
  TORCH_CHECK(rc == 0, "mamba2_scan: unsupported arguments (code ", rc, "): state width 16 / 32 / 64 / 128 / 256, B and C 16-byte aligned");
}

void mamba1_scan(const Tensor& x, const Tensor& dt, const Tensor& Bm, const Tensor& Cm, const optional<Tensor>& z, const Tensor& A,
                 const optional<Tensor>& D, const optional<Tensor>& dt_bias, Tensor state, const Tensor& q_starts, const Tensor& seq_state,
                 const Tensor& positions, Tensor y, int64_t seg_len, int64_t segs, const optional<Tensor>& seg_scratch) {
  TORCH_CHECK(rows_bf16(x) && rows_bf16(dt) && rows_bf16(Bm) && rows_bf16(Cm) && rows_bf16(y), "activations: bf16 rows");
  const int64_t Dm = x.size(1), N = Bm.size(1);
  TORCH_CHECK(A.scalar_type() == at::kFloat && A.is_contiguous() && A.dim() == 2 && A.size(0) == Dm && A.size(1) == N, "A: fp32 [D, N]");
  TORCH_CHECK(state.scalar_type() == at::kFloat && state.is_contiguous() && state.dim() == 3 && state.size(1) == Dm && state.size(2) == N,
              "state: fp32 [slots, D, N]");
  check_batch(q_starts, seq_state, positions);
  c10::cuda::CUDAGuard guard(x.device());
  float *seg_state = nullptr, *seg_dt = nullptr;
  const int64_t B = seq_state.numel();
  if (seg_len > 0 && segs > 1) {                 // scratch: B * segs states of [Dm][N], then [B][segs - 1][Dm] step sums
    const int64_t n_state = B * segs * Dm * N, n_dt = B * (segs - 1) * Dm;
    TORCH_CHECK(seg_scratch.has_value() && seg_scratch->scalar_type() == at::kFloat && seg_scratch->is_contiguous() &&
                    seg_scratch->numel() >= n_state + n_dt, "seg_scratch: fp32, at least B * Dm * (segs * N + segs - 1) values");
    seg_state = seg_scratch->data_ptr<float>();
    seg_dt = seg_state + n_state;
  }
  const int rc = fllm::mamba1_scan(x.data_ptr(), x.stride(0), dt.data_ptr(), dt.stride(0), Bm.data_ptr(), Bm.stride(0), Cm.data_ptr(),
                                   Cm.stride(0), opt_ptr(z), opt_ld(z), A.data_ptr<float>(), opt_f32(D), opt_f32(dt_bias),
                                   state.data_ptr<float>(), q_starts.data_ptr<int>(), seq_state.data_ptr<int>(), positions.data_ptr<int>(),
                                   y.data_ptr(), y.stride(0), (int)B, (int)Dm, (int)N, (int)seg_len, (int)segs, seg_state, seg_dt,
                                   cur_stream());
  TORCH_CHECK(rc == 0, "mamba1_scan: unsupported arguments (code ", rc, "): state width 8 / 16, B and C 16-byte aligned");
}

void matrix_state_scan(int64_t kind, const Tensor& r, const Tensor& k, const Tensor& v, const optional<Tensor>& a, const optional<Tensor>& b,
                       const optional<Tensor>& w_opt, const optional<Tensor>& u, const optional<Tensor>& beta, Tensor state, const Tensor& q_starts,
                       const Tensor& seq_state, const Tensor& positions, Tensor y, int64_t H, int64_t DK, int64_t DV, int64_t kv_ratio,
                       bool l2norm, double q_scale, const optional<Tensor>& gate_raw, const optional<Tensor>& gate_A,
                       const optional<Tensor>& gate_dt_bias) {
  TORCH_CHECK(rows_bf16(r) && rows_bf16(k) && rows_bf16(v) && rows_bf16(y), "activations: bf16 rows");
  TORCH_CHECK(v.size(1) == H * DV && y.size(1) == H * DV && r.size(1) == (H / kv_ratio) * DK && k.size(1) == r.size(1), "widths");
  const bool raw = !(w_opt.has_value() && w_opt->defined());
  const float* w_ptr = nullptr;
  long long w_ld = 0;
  if (!raw) {
    const Tensor& w = *w_opt;
    TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kFloat && w.dim() == 2 && w.stride(1) == 1, "w: fp32 rows of log decays");
    TORCH_CHECK(w.size(1) == (kind == 2 ? H : r.size(1)), "w: one decay per head (kind 2) or per key channel");
    w_ptr = w.data_ptr<float>();
    w_ld = w.stride(0);
  } else {
    TORCH_CHECK(kind == 2 && gate_raw.has_value() && rows_bf16(*gate_raw) && gate_raw->size(1) == H && gate_A.has_value() &&
                    gate_dt_bias.has_value() && gate_A->numel() == H && gate_dt_bias->numel() == H,
                "raw gates: kind 2 with gate_raw bf16 [T, H], gate_A and gate_dt_bias fp32 [H]");
  }
  TORCH_CHECK(kind != 1 || (a.has_value() && b.has_value() && rows_bf16(*a) && rows_bf16(*b)), "RWKV-7 needs a and b");
  TORCH_CHECK(kind != 0 || (u.has_value() && u->numel() == r.size(1)), "RWKV-6 needs the bonus u");
  TORCH_CHECK(kind < 2 || (beta.has_value() && rows_bf16(*beta) && beta->size(1) == H), "delta rules need beta [T, H]");
  TORCH_CHECK(state.scalar_type() == at::kFloat && state.is_contiguous() && state.dim() == 4 && state.size(1) == H && state.size(2) == DV &&
                  state.size(3) == DK, "state: fp32 [slots, H, DV, DK]");
  check_batch(q_starts, seq_state, positions);
  c10::cuda::CUDAGuard guard(r.device());
  const int rc = fllm::matrix_state_scan((int)kind, r.data_ptr(), r.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), opt_ptr(a),
                                         opt_ld(a), opt_ptr(b), opt_ld(b), w_ptr, w_ld, opt_f32(u), opt_ptr(beta),
                                         opt_ld(beta), state.data_ptr<float>(), q_starts.data_ptr<int>(), seq_state.data_ptr<int>(),
                                         positions.data_ptr<int>(), y.data_ptr(), y.stride(0), (int)seq_state.numel(), (int)H, (int)DK, (int)DV,
                                         (int)kv_ratio, l2norm ? 1 : 0, (float)q_scale, opt_ptr(gate_raw), opt_ld(gate_raw), opt_f32(gate_A),
                                         opt_f32(gate_dt_bias), cur_stream());
  TORCH_CHECK(rc == 0, "matrix_state_scan: unsupported arguments (code ", rc, "): key width 32 / 64 / 128 / 256, 16-byte aligned rows");
}

void gated_rmsnorm(const Tensor& x, const optional<Tensor>& z, const Tensor& w, Tensor y, int64_t group_size, double eps, bool norm_before_gate) {
  TORCH_CHECK(rows_bf16(x) && rows_bf16(y) && x.sizes() == y.sizes(), "x, y: bf16 rows of one shape");
  TORCH_CHECK(w.scalar_type() == at::kBFloat16 && w.is_contiguous() && x.size(1) % group_size == 0, "w: bf16; D a multiple of the group");
  TORCH_CHECK(!z.has_value() || !z->defined() || (rows_bf16(*z) && z->sizes() == x.sizes()), "z: bf16 rows like x");
  c10::cuda::CUDAGuard guard(x.device());
  fllm::gated_rmsnorm(x.data_ptr(), x.stride(0), opt_ptr(z), opt_ld(z), w.data_ptr(), (int)w.numel(), y.data_ptr(), y.stride(0), (int)x.size(0),
                      (int)x.size(1), (int)group_size, (float)eps, norm_before_gate ? 1 : 0, cur_stream());
}

// q_abs [H, T, 512] or [T, H, 512] (any strides with a unit inner one), q_pe [T, H, 64], out like q_abs
int64_t attention_mla_splits(int64_t tokens, int64_t H, int64_t max_kv_len) {
  return fllm::attention_mla_splits((int)tokens, (int)H, (int)max_kv_len);
}
int64_t attention_mla_workspace_bytes(int64_t tokens, int64_t H, int64_t splits) {
  return (int64_t)fllm::attention_mla_workspace_bytes((int)tokens, (int)H, (int)splits);
}

// splits = 0: the CUDA-core kernel; >= 1: the tensor-core kernel over that many key slices (workspace needed above 1)
void attention_mla(const Tensor& q_abs, const Tensor& q_pe, const Tensor& cache, const Tensor& block_tables, const Tensor& row_seq,
                   const Tensor& positions, Tensor out, bool head_major, double scale, int64_t splits, const optional<Tensor>& workspace) {
  TORCH_CHECK(q_abs.is_cuda() && q_abs.scalar_type() == at::kBFloat16 && q_abs.dim() == 3 && q_abs.stride(2) == 1 && q_abs.size(2) == 512,
              "q_abs: bf16 [., ., 512] with a unit inner stride");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.dim() == 3 && out.stride(2) == 1 && out.sizes() == q_abs.sizes(), "out: like q_abs");
  const int td = head_major ? 1 : 0, hd = head_major ? 0 : 1;
  const int64_t T = q_abs.size(td), H = q_abs.size(hd);
  TORCH_CHECK(q_pe.scalar_type() == at::kBFloat16 && q_pe.is_contiguous() && q_pe.dim() == 3 && q_pe.size(0) == T && q_pe.size(1) == H &&
                  q_pe.size(2) == 64, "q_pe: contiguous bf16 [T, H, 64]");
  TORCH_CHECK(cache.scalar_type() == at::kBFloat16 && cache.dim() == 3 && cache.is_contiguous() && cache.size(2) == 576,
              "cache: contiguous bf16 [blocks, block_size, 576]");
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && block_tables.dim() == 2 && block_tables.stride(1) == 1 &&
                  row_seq.scalar_type() == at::kInt && positions.scalar_type() == at::kInt && row_seq.is_contiguous() &&
                  positions.is_contiguous() && row_seq.numel() >= T && positions.numel() >= T,
              "block_tables [B, max_blocks], row_seq [T], positions [T]: int32");
  c10::cuda::CUDAGuard guard(q_abs.device());
  if (splits >= 1) {
    void* ws = nullptr;
    size_t ws_bytes = 0;
    if (workspace.has_value() && workspace->defined()) {
      TORCH_CHECK(workspace->is_cuda() && workspace->is_contiguous(), "workspace: contiguous CUDA tensor");
      ws = workspace->data_ptr();
      ws_bytes = workspace->numel() * workspace->element_size();
    }
    fllm::attention_mla_tc_bf16(q_abs.data_ptr(), q_abs.stride(td), q_abs.stride(hd), q_pe.data_ptr(), cache.data_ptr(),
                                block_tables.data_ptr<int>(), (int)block_tables.stride(0), row_seq.data_ptr<int>(), positions.data_ptr<int>(),
                                out.data_ptr(), out.stride(td), out.stride(hd), (int)T, (int)H, (int)cache.size(1), (float)scale, (int)splits,
                                ws, ws_bytes, cur_stream());
    return;
  }
  fllm::attention_mla_bf16(q_abs.data_ptr(), q_abs.stride(td), q_abs.stride(hd), q_pe.data_ptr(), cache.data_ptr(), block_tables.data_ptr<int>(),
                           (int)block_tables.stride(0), row_seq.data_ptr<int>(), positions.data_ptr<int>(), out.data_ptr(), out.stride(td),
                           out.stride(hd), (int)T, (int)H, (int)cache.size(1), (float)scale, cur_stream());
}

// ckv bf16 [T, >= 576] rows, q bf16 [T, H, head] contiguous with the rotary values of a head at rope_offset
void mla_prepare(const Tensor& ckv, const Tensor& q, int64_t rope_offset, const Tensor& positions, const Tensor& slots, const Tensor& inv_freq,
                 double attn_factor, const Tensor& norm_w, double eps, Tensor cache, Tensor q_pe) {
  TORCH_CHECK(rows_bf16(ckv) && ckv.size(1) >= 576, "ckv: bf16 rows of at least 576 values");
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.dim() == 3 && q.is_contiguous() && rope_offset + 64 <= q.size(2) &&
                  q.size(0) == ckv.size(0), "q: contiguous bf16 [T, H, head]");
  TORCH_CHECK(inv_freq.scalar_type() == at::kFloat && inv_freq.is_contiguous() && inv_freq.numel() == 32, "inv_freq: fp32 [32]");
  TORCH_CHECK(norm_w.scalar_type() == at::kBFloat16 && norm_w.is_contiguous() && norm_w.numel() == 512, "norm_w: bf16 [512]");
  TORCH_CHECK(cache.scalar_type() == at::kBFloat16 && cache.is_contiguous() && cache.dim() == 3 && cache.size(2) == 576, "cache: bf16 [blocks, block_size, 576]");
  TORCH_CHECK(q_pe.scalar_type() == at::kBFloat16 && q_pe.is_contiguous() && q_pe.dim() == 3 && q_pe.size(0) == q.size(0) &&
                  q_pe.size(1) == q.size(1) && q_pe.size(2) == 64, "q_pe: contiguous bf16 [T, H, 64]");
  TORCH_CHECK(positions.scalar_type() == at::kInt && slots.scalar_type() == at::kInt && positions.is_contiguous() && slots.is_contiguous() &&
                  positions.numel() >= q.size(0) && slots.numel() >= q.size(0), "positions, slots: int32 [T]");
  c10::cuda::CUDAGuard guard(q.device());
  fllm::mla_prepare_bf16(ckv.data_ptr(), ckv.stride(0), q.data_ptr(), q.stride(0), (int)q.stride(1), (int)rope_offset, positions.data_ptr<int>(),
                         slots.data_ptr<int>(), inv_freq.data_ptr<float>(), (float)attn_factor, norm_w.data_ptr(), (float)eps, cache.data_ptr(),
                         q_pe.data_ptr(), (int)q.size(0), (int)q.size(1), cur_stream());
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(fllm_b200, m) {
  m.def("causal_conv1d(Tensor x, Tensor w, Tensor? bias, Tensor(a!) state, Tensor q_starts, Tensor seq_state, Tensor positions, Tensor(b!) y, bool act, int max_q_len) -> ()",
        &causal_conv1d);
  m.def("mamba2_scan(Tensor x, Tensor dt, Tensor Bm, Tensor Cm, Tensor A, Tensor? D, Tensor? dt_bias, Tensor(a!) state, Tensor q_starts, "
        "Tensor seq_state, Tensor positions, Tensor(b!) y, int H, int P, int G, int N, float dt_min, float dt_max, int seg_len, int segs, "
        "Tensor? seg_scratch, int skip_from) -> ()",
        &mamba2_scan);
  m.def("mamba1_scan(Tensor x, Tensor dt, Tensor Bm, Tensor Cm, Tensor? z, Tensor A, Tensor? D, Tensor? dt_bias, Tensor(a!) state, "
        "Tensor q_starts, Tensor seq_state, Tensor positions, Tensor(b!) y, int seg_len, int segs, Tensor? seg_scratch) -> ()",
        &mamba1_scan);
  m.def("matrix_state_scan(int kind, Tensor r, Tensor k, Tensor v, Tensor? a, Tensor? b, Tensor? w, Tensor? u, Tensor? beta, Tensor(a!) state, "
        "Tensor q_starts, Tensor seq_state, Tensor positions, Tensor(b!) y, int H, int DK, int DV, int kv_ratio, bool l2norm, float q_scale, "
        "Tensor? gate_raw, Tensor? gate_A, Tensor? gate_dt_bias) -> ()",
        &matrix_state_scan);
  m.def("attention_mla(Tensor q_abs, Tensor q_pe, Tensor cache, Tensor block_tables, Tensor row_seq, Tensor positions, Tensor(a!) out, "
        "bool head_major, float scale, int splits, Tensor? workspace) -> ()", &attention_mla);
  m.def("attention_mla_splits(int tokens, int H, int max_kv_len) -> int", &attention_mla_splits);
  m.def("attention_mla_workspace_bytes(int tokens, int H, int splits) -> int", &attention_mla_workspace_bytes);
  m.def("mla_prepare(Tensor ckv, Tensor q, int rope_offset, Tensor positions, Tensor slots, Tensor inv_freq, float attn_factor, Tensor norm_w, "
        "float eps, Tensor(a!) cache, Tensor(b!) q_pe) -> ()", &mla_prepare);
  m.def("gated_rmsnorm(Tensor x, Tensor? z, Tensor w, Tensor(a!) y, int group_size, float eps, bool norm_before_gate) -> ()", &gated_rmsnorm);
}
