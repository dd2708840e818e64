// CPU decoder for packed GGUF weights: the batch-1 engine of the tiny-Llama
// configuration and the oracle of the GPU packed-weight kernels.
//
// Projections run as integer dots of packed weights against activations quantised
// to Q8_K per 256 values (the scheme of the reference's CPU path,
// rust/engine/src/cpu_kquant.rs:1-10); other weight types are expanded block by
// block. The KV cache is paged, f16, [layer][k|v][block][kv_head][block_size][head_dim].
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "quant.h"

struct CpuConfig {
  int n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab;
  int block_size, num_blocks;
  int rope_style;        // 0 rotate-half, 1 interleaved pairs
  int tie_embeddings;
  float eps, rope_theta;
};

struct Mat {
  int type = -1;
  const uint8_t* data = nullptr;
  int64_t rows = 0, cols = 0, row_bytes = 0;
};

struct CpuModel {
  CpuConfig cfg;
  std::map<std::string, Mat> t;
  std::vector<uint16_t> kv;          // f16
  std::vector<float> inv_freq;
  const Mat& get(const std::string& n) const {
    auto it = t.find(n);
    if (it == t.end()) { static Mat none; return none; }
    return it->second;
  }
};

static void rmsnorm(const float* x, const Mat& w, float eps, int n, float* y) {
  float ss = 0;
  for (int i = 0; i < n; ++i) ss += x[i] * x[i];
  const float inv = 1.f / sqrtf(ss / n + eps);
  const float* wf = reinterpret_cast<const float*>(w.data);
  for (int i = 0; i < n; ++i) y[i] = x[i] * inv * wf[i];
}

// Y[tok][row] = W[row] . X[tok] for n_tok activation rows
static void matmul(const Mat& W, const float* X, int n_tok, float* Y) {
  const int64_t K = W.cols, N = W.rows;
  if (W.type == FLLM_Q4_K || W.type == FLLM_Q6_K) {
    const int64_t nb = K / QK_K;
    std::vector<BlockQ8K> xq((size_t)n_tok * nb);
    for (int t = 0; t < n_tok; ++t) quantize_row_q8_K(X + (size_t)t * K, xq.data() + (size_t)t * nb, K);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
      const uint8_t* wr = W.data + r * W.row_bytes;
      for (int t = 0; t < n_tok; ++t) {
        const BlockQ8K* a = xq.data() + (size_t)t * nb;
        Y[(size_t)t * N + r] = W.type == FLLM_Q4_K ? dot_q4_K_q8_K((const BlockQ4K*)wr, a, nb)
                                                    : dot_q6_K_q8_K((const BlockQ6K*)wr, a, nb);
      }
    }
    return;
  }
#pragma omp parallel
  {
    std::vector<float> row(K);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
      fllm_dequantize(W.type, W.data + r * W.row_bytes, row.data(), 1, K);
      for (int t = 0; t < n_tok; ++t) {
        const float* x = X + (size_t)t * K;
        float acc = 0;
        for (int64_t k = 0; k < K; ++k) acc += row[k] * x[k];
        Y[(size_t)t * N + r] = acc;
      }
    }
  }
}

static void rope(float* v, int head_dim, int pos, const std::vector<float>& inv_freq, int style) {
  const int half = head_dim / 2;
  for (int i = 0; i < half; ++i) {
    const float a = pos * inv_freq[i], c = cosf(a), s = sinf(a);
    const int i0 = style == 0 ? i : 2 * i, i1 = style == 0 ? i + half : 2 * i + 1;
    const float x = v[i0], y = v[i1];
    v[i0] = x * c - y * s;
    v[i1] = y * c + x * s;
  }
}

FLLM_API void* fllm_cpu_create(const CpuConfig* cfg) {
  auto* m = new CpuModel();
  m->cfg = *cfg;
  const size_t kv_elems = (size_t)cfg->n_layers * 2 * cfg->num_blocks * cfg->n_kv_heads * cfg->block_size * cfg->head_dim;
  m->kv.assign(kv_elems, 0);
  m->inv_freq.resize(cfg->head_dim / 2);
  for (int i = 0; i < cfg->head_dim / 2; ++i) m->inv_freq[i] = powf(cfg->rope_theta, -2.f * i / cfg->head_dim);
  return m;
}

FLLM_API void fllm_cpu_destroy(void* h) { delete static_cast<CpuModel*>(h); }

// The tensor memory is borrowed: the caller keeps the (mmap'ed) file alive.
FLLM_API int fllm_cpu_set_tensor(void* h, const char* name, int type, const void* data, int64_t rows, int64_t cols) {
  auto* m = static_cast<CpuModel*>(h);
  const int64_t rb = fllm_row_bytes(type, cols);
  if (rb < 0) return -1;
  Mat t;
  t.type = type; t.data = static_cast<const uint8_t*>(data); t.rows = rows; t.cols = cols; t.row_bytes = rb;
  m->t[name] = t;
  return 0;
}

// Feeds n tokens at positions pos0.. of one sequence whose KV blocks are `table`; writes the
// logits of the last token to logits[vocab]. Returns 0 on success.
FLLM_API int fllm_cpu_forward(void* h, const int* tokens, int n, int pos0, const int* table, float* logits) {
  auto* m = static_cast<CpuModel*>(h);
  const CpuConfig& c = m->cfg;
  const int H = c.hidden, D = c.head_dim, HQ = c.n_heads, HKV = c.n_kv_heads, G = HQ / HKV;
  const Mat& emb = m->get("token_embd.weight");
  if (emb.type < 0) return -1;
  std::vector<float> x((size_t)n * H), hbuf((size_t)n * H), q((size_t)n * HQ * D), k((size_t)n * HKV * D),
      v((size_t)n * HKV * D), att((size_t)n * HQ * D), proj((size_t)n * H), gate((size_t)n * c.ffn),
      up((size_t)n * c.ffn);
  for (int t = 0; t < n; ++t)
    fllm_dequantize(emb.type, emb.data + (size_t)tokens[t] * emb.row_bytes, x.data() + (size_t)t * H, 1, H);
  const size_t blk_elems = (size_t)HKV * c.block_size * D;
  for (int l = 0; l < c.n_layers; ++l) {
    const std::string p = "blk." + std::to_string(l) + ".";
    for (int t = 0; t < n; ++t) rmsnorm(x.data() + (size_t)t * H, m->get(p + "attn_norm.weight"), c.eps, H, hbuf.data() + (size_t)t * H);
    matmul(m->get(p + "attn_q.weight"), hbuf.data(), n, q.data());
    matmul(m->get(p + "attn_k.weight"), hbuf.data(), n, k.data());
    matmul(m->get(p + "attn_v.weight"), hbuf.data(), n, v.data());
    uint16_t* kc = m->kv.data() + ((size_t)l * 2 + 0) * c.num_blocks * blk_elems;
    uint16_t* vc = m->kv.data() + ((size_t)l * 2 + 1) * c.num_blocks * blk_elems;
    for (int t = 0; t < n; ++t) {
      const int pos = pos0 + t, blk = table[pos / c.block_size], off = pos % c.block_size;
      for (int hh = 0; hh < HQ; ++hh) rope(q.data() + ((size_t)t * HQ + hh) * D, D, pos, m->inv_freq, c.rope_style);
      for (int hh = 0; hh < HKV; ++hh) {
        float* kr = k.data() + ((size_t)t * HKV + hh) * D;
        rope(kr, D, pos, m->inv_freq, c.rope_style);
        uint16_t* kd = kc + (size_t)blk * blk_elems + ((size_t)hh * c.block_size + off) * D;
        uint16_t* vd = vc + (size_t)blk * blk_elems + ((size_t)hh * c.block_size + off) * D;
        const float* vr = v.data() + ((size_t)t * HKV + hh) * D;
        for (int d = 0; d < D; ++d) { kd[d] = fllm_fp32_to_fp16(kr[d]); vd[d] = fllm_fp32_to_fp16(vr[d]); }
      }
    }
    const float scale = 1.f / sqrtf((float)D);
#pragma omp parallel for collapse(2) schedule(static)
    for (int t = 0; t < n; ++t) {
      for (int hh = 0; hh < HQ; ++hh) {
        const int kvh = hh / G, len = pos0 + t + 1;
        const float* qr = q.data() + ((size_t)t * HQ + hh) * D;
        std::vector<float> sc(len);
        float mx = -INFINITY;
        for (int j = 0; j < len; ++j) {
          const uint16_t* kr = kc + (size_t)table[j / c.block_size] * blk_elems + ((size_t)kvh * c.block_size + j % c.block_size) * D;
          float a = 0;
          for (int d = 0; d < D; ++d) a += qr[d] * fllm_fp16_to_fp32(kr[d]);
          sc[j] = a * scale;
          mx = std::max(mx, sc[j]);
        }
        float den = 0;
        for (int j = 0; j < len; ++j) { sc[j] = expf(sc[j] - mx); den += sc[j]; }
        float* o = att.data() + ((size_t)t * HQ + hh) * D;
        for (int d = 0; d < D; ++d) o[d] = 0;
        for (int j = 0; j < len; ++j) {
          const uint16_t* vr = vc + (size_t)table[j / c.block_size] * blk_elems + ((size_t)kvh * c.block_size + j % c.block_size) * D;
          const float w = sc[j] / den;
          for (int d = 0; d < D; ++d) o[d] += w * fllm_fp16_to_fp32(vr[d]);
        }
      }
    }
    matmul(m->get(p + "attn_output.weight"), att.data(), n, proj.data());
    for (size_t i = 0; i < (size_t)n * H; ++i) x[i] += proj[i];
    for (int t = 0; t < n; ++t) rmsnorm(x.data() + (size_t)t * H, m->get(p + "ffn_norm.weight"), c.eps, H, hbuf.data() + (size_t)t * H);
    matmul(m->get(p + "ffn_gate.weight"), hbuf.data(), n, gate.data());
    matmul(m->get(p + "ffn_up.weight"), hbuf.data(), n, up.data());
    for (size_t i = 0; i < (size_t)n * c.ffn; ++i) gate[i] = gate[i] / (1.f + expf(-gate[i])) * up[i];
    matmul(m->get(p + "ffn_down.weight"), gate.data(), n, proj.data());
    for (size_t i = 0; i < (size_t)n * H; ++i) x[i] += proj[i];
  }
  rmsnorm(x.data() + (size_t)(n - 1) * H, m->get("output_norm.weight"), c.eps, H, hbuf.data());
  const Mat& head = c.tie_embeddings || m->get("output.weight").type < 0 ? emb : m->get("output.weight");
  matmul(head, hbuf.data(), 1, logits);
  return 0;
}

// Greedy generation: prompt pass, then n_out single-token steps. Returns tokens generated.
FLLM_API int fllm_cpu_generate(void* h, const int* prompt, int n_prompt, int n_out, const int* table, int* out) {
  auto* m = static_cast<CpuModel*>(h);
  std::vector<float> logits(m->cfg.vocab);
  if (fllm_cpu_forward(h, prompt, n_prompt, 0, table, logits.data())) return -1;
  int pos = n_prompt;
  for (int i = 0; i < n_out; ++i) {
    int best = 0;
    for (int j = 1; j < m->cfg.vocab; ++j)
      if (logits[j] > logits[best]) best = j;
    out[i] = best;
    if (i + 1 == n_out) break;
    if (fllm_cpu_forward(h, &best, 1, pos, table, logits.data())) return -1;
    ++pos;
  }
  return n_out;
}
