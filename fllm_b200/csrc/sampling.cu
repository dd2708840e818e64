// Device sampler: one CTA per logit row.
//
//   argmax_rows      greedy token (+ optional value) per row
//   sample_rows      penalties / logit bias (sparse lists prepared by the host),
//                    temperature, top-k, min-p, top-p, then a Gumbel-max draw whose
//                    noise is Philox-4x32-10 keyed by (seed, draw counter, token id),
//                    so a row's outcome does not depend on batch composition
//   spec_verify      speculative-decoding acceptance: greedy chain match, or the
//                    exact accept / residual-resample rule on full distributions
//
// Thresholds for top-k / top-p are found by bisection on the order-preserving
// 32-bit key of the float logit instead of sorting the vocabulary.
// Semantics follow rust/engine/cuda/sampling.cu:182-423 (sample_rows_kernel),
// :430-457 (spec_verify_kernel) and rust/engine/src/speculative.rs:103 (verify_chain).
#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

constexpr int kSampThreads = 1024;

__device__ __forceinline__ float ld_logit(const __nv_bfloat16* p, int i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ float ld_logit(const float* p, int i) { return p[i]; }
__device__ __forceinline__ void st_logit(__nv_bfloat16* p, int i, float v) { p[i] = __float2bfloat16(v); }
__device__ __forceinline__ void st_logit(float* p, int i, float v) { p[i] = v; }

// order-preserving map float -> uint32
__device__ __forceinline__ uint32_t fkey(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float fkey_inv(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

// uniform in (0,1) from (seed, draw, index)
__device__ __forceinline__ float philox_uniform(unsigned long long seed, uint32_t draw, uint32_t idx) {
  uint32_t c[4] = {idx, draw, 0x9E3779B9u, 0xBB67AE85u};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return ((float)(c[0] >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__device__ ArgMax block_argmax(ArgMax a, ArgMax* sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) sm[warp] = a;
  __syncthreads();
  if (warp == 0) {
    ArgMax b = lane < nw ? sm[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax c;
      c.v = __shfl_xor_sync(0xffffffffu, b.v, o);
      c.i = __shfl_xor_sync(0xffffffffu, b.i, o);
      b = better(b, c);
    }
    if (lane == 0) sm[0] = b;
  }
  __syncthreads();
  return sm[0];
}

__device__ float block_sum(float v, float* sm) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float b = lane < nw ? sm[lane] : 0.f;
    b = warp_sum(b);
    if (lane == 0) sm[0] = b;
  }
  __syncthreads();
  return sm[0];
}

template <typename T>
__global__ void __launch_bounds__(kSampThreads)
argmax_rows_kernel(const T* __restrict__ logits, long long ld, int vocab, int* __restrict__ out_ids,
                   float* __restrict__ out_vals, int id_offset) {
  __shared__ ArgMax sm[32];
  const T* row = logits + (size_t)blockIdx.x * ld;
  ArgMax a{-INFINITY, 0x7fffffff};
  int i0 = 0;
  if constexpr (sizeof(T) == 2) {
    // 16-byte loads (8 logits) when the row allows it; a strict '>' inside a vector and `better`
    // across threads keep the lowest index among equal maxima
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      const int nvec = vocab >> 3;
      const uint4* rv = reinterpret_cast<const uint4*>(row);
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        const uint4 u = rv[v];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
        float best = -INFINITY;
        int bi = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(w[j]);
          if (f.x > best) { best = f.x; bi = 2 * j; }
          if (f.y > best) { best = f.y; bi = 2 * j + 1; }
        }
        a = better(a, ArgMax{best, 8 * v + bi});
      }
      i0 = nvec << 3;
    }
  }
  for (int i = i0 + threadIdx.x; i < vocab; i += blockDim.x) a = better(a, ArgMax{ld_logit(row, i), i});
  a = block_argmax(a, sm);
  if (threadIdx.x == 0) {
    out_ids[blockIdx.x] = a.i + id_offset;
    if (out_vals) out_vals[blockIdx.x] = a.v;
  }
}

void argmax_rows(const void* logits, int is_fp32, long long ld, int rows, int vocab, int* out_ids,
                 float* out_vals, int id_offset, cudaStream_t s) {
  if (rows <= 0) return;
  if (is_fp32)
    argmax_rows_kernel<float><<<rows, kSampThreads, 0, s>>>((const float*)logits, ld, vocab, out_ids,
                                                           out_vals, id_offset);
  else
    argmax_rows_kernel<__nv_bfloat16><<<rows, kSampThreads, 0, s>>>(
        (const __nv_bfloat16*)logits, ld, vocab, out_ids, out_vals, id_offset);
  cuda_check(cudaGetLastError(), "argmax_rows_kernel");
}

// The same reduction with every row cut over `parts` CTAs (a decode batch has far fewer rows than the GPU
// has SMs, and a 150 k-entry row is 300 KB): each CTA reduces a slice, parks (value, index) and bumps the
// row's counter; the CTA that arrives last combines the slices and re-zeroes the counter. `better` makes the
// result independent of the arrival order. out_pairs (optional) receives (value, float(id)) per row, the
// message a vocabulary-parallel head exchanges.
template <typename T>
__global__ void __launch_bounds__(kSampThreads)
argmax_rows_split_kernel(const T* __restrict__ logits, long long ld, int vocab, int parts, int* __restrict__ out_ids,
                         float* __restrict__ out_vals, float* __restrict__ out_pairs, int id_offset,
                         float2* __restrict__ part, unsigned int* __restrict__ counters) {
  __shared__ ArgMax sm[32];
  __shared__ int is_last;
  const int r = blockIdx.x, pi = blockIdx.y;
  const T* row = logits + (size_t)r * ld;
  const int chunk = (((vocab + parts - 1) / parts) + 7) & ~7;
  const int lo = min(vocab, pi * chunk), hi = min(vocab, lo + chunk);
  ArgMax a{-INFINITY, 0x7fffffff};
  int i0 = lo;
  if constexpr (sizeof(T) == 2) {
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      const int v0 = lo >> 3, v1 = hi >> 3;
      const uint4* rv = reinterpret_cast<const uint4*>(row);
      for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
        const uint4 u = rv[v];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
        float best = -INFINITY;
        int bi = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(w[j]);
          if (f.x > best) { best = f.x; bi = 2 * j; }
          if (f.y > best) { best = f.y; bi = 2 * j + 1; }
        }
        a = better(a, ArgMax{best, 8 * v + bi});
      }
      i0 = max(lo, v1 << 3);
    }
  }
  for (int i = i0 + threadIdx.x; i < hi; i += blockDim.x) a = better(a, ArgMax{ld_logit(row, i), i});
  a = block_argmax(a, sm);
  if (threadIdx.x == 0) {
    part[(size_t)r * parts + pi] = make_float2(a.v, __int_as_float(a.i));
    __threadfence();
    const unsigned int old = atomicAdd(counters + r, 1u);
    is_last = old == (unsigned int)(parts - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (threadIdx.x < 32) {
    ArgMax b{-INFINITY, 0x7fffffff};
    for (int j = threadIdx.x; j < parts; j += 32) {
      const float2 pv = __ldcg(part + (size_t)r * parts + j);
      b = better(b, ArgMax{pv.x, __float_as_int(pv.y)});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax c;
      c.v = __shfl_xor_sync(0xffffffffu, b.v, o);
      c.i = __shfl_xor_sync(0xffffffffu, b.i, o);
      b = better(b, c);
    }
    if (threadIdx.x == 0) {
      out_ids[r] = b.i + id_offset;
      if (out_vals) out_vals[r] = b.v;
      if (out_pairs) { out_pairs[2 * r] = b.v; out_pairs[2 * r + 1] = (float)(b.i + id_offset); }
      counters[r] = 0;
    }
  }
}

// scratch layout: [kArgmaxMaxRows row counters, zero between launches][rows * parts (value, index) pairs]. The counter
// block has a fixed size so that calls with different row counts never park pairs where another call counts.
constexpr int kArgmaxMaxRows = 1024;
size_t argmax_split_scratch_bytes(int rows, int parts) { return (size_t)kArgmaxMaxRows * 4 + (size_t)rows * parts * 8; }

void argmax_rows_split(const void* logits, int is_fp32, long long ld, int rows, int vocab, int* out_ids, float* out_vals,
                       float* out_pairs, int id_offset, void* scratch, size_t scratch_bytes, cudaStream_t s) {
  if (rows <= 0) return;
  if (rows > kArgmaxMaxRows) throw std::runtime_error("argmax_rows_split: at most 1024 rows");
  int parts = max(1, min(32, (2 * sm_count() + rows - 1) / rows));
  parts = min(parts, max(1, vocab / 2048));
  if (argmax_split_scratch_bytes(rows, parts) > scratch_bytes)
    throw std::runtime_error("argmax_rows_split: scratch too small");
  auto* counters = reinterpret_cast<unsigned int*>(scratch);                       // zero between launches
  auto* part = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(scratch) + (size_t)kArgmaxMaxRows * 4);
  dim3 grid(rows, parts);
  if (is_fp32)
    argmax_rows_split_kernel<float><<<grid, kSampThreads, 0, s>>>((const float*)logits, ld, vocab, parts, out_ids, out_vals,
                                                                 out_pairs, id_offset, part, counters);
  else
    argmax_rows_split_kernel<__nv_bfloat16><<<grid, kSampThreads, 0, s>>>((const __nv_bfloat16*)logits, ld, vocab, parts,
                                                                         out_ids, out_vals, out_pairs, id_offset, part,
                                                                         counters);
  cuda_check(cudaGetLastError(), "argmax_rows_split_kernel");
}

// Vocabulary-parallel greedy token: pairs[rank][row] = (best local value, its global id as a float) gathered from
// every rank; the winner per row is the highest value, the lowest rank (= lowest id) among equals.
__global__ void argmax_pairs_select_kernel(const float2* __restrict__ pairs, int ranks, int rows, int* __restrict__ out_ids) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float best = -INFINITY;
  int id = 0;
  for (int k = 0; k < ranks; ++k) {
    const float2 pv = pairs[(size_t)k * rows + r];
    if (pv.x > best || k == 0) { best = pv.x; id = (int)pv.y; }
  }
  out_ids[r] = id;
}

void argmax_pairs_select(const float* pairs, int ranks, int rows, int* out_ids, cudaStream_t s) {
  if (rows <= 0) return;
  argmax_pairs_select_kernel<<<(rows + 127) / 128, 128, 0, s>>>(reinterpret_cast<const float2*>(pairs), ranks, rows, out_ids);
  cuda_check(cudaGetLastError(), "argmax_pairs_select_kernel");
}

// ---------------------------------------------------------------------------- full sampler
template <typename T>
__global__ void __launch_bounds__(kSampThreads)
sample_rows_kernel(T* __restrict__ logits, long long ld, int vocab, const SampleRow* __restrict__ prm,
                   const int* __restrict__ pen_ids, const int* __restrict__ pen_counts, int pen_stride,
                   const int* __restrict__ bias_ids, const float* __restrict__ bias_vals,
                   int bias_stride, const uint32_t* __restrict__ allow_mask, int mask_words,
                   int* __restrict__ out_ids, float* __restrict__ out_logprobs) {
  __shared__ ArgMax sm_a[32];
  __shared__ float sm_f[32];
  __shared__ float sm_scalar[2];
  const int r = blockIdx.x;
  T* row = logits + (size_t)r * ld;
  const SampleRow p = prm[r];

  // sparse edits: penalties on tokens already seen, then logit bias
  if (pen_ids) {
    for (int i = threadIdx.x; i < pen_stride; i += blockDim.x) {
      const int id = pen_ids[(size_t)r * pen_stride + i];
      if (id < 0 || id >= vocab) continue;
      const int cnt = pen_counts[(size_t)r * pen_stride + i];
      float v = ld_logit(row, id);
      if (p.repetition_penalty != 1.f) v = v > 0.f ? v / p.repetition_penalty : v * p.repetition_penalty;
      if (cnt > 0) v -= p.presence_penalty + p.frequency_penalty * (float)cnt;
      st_logit(row, id, v);
    }
  }
  __syncthreads();
  if (bias_ids) {
    for (int i = threadIdx.x; i < bias_stride; i += blockDim.x) {
      const int id = bias_ids[(size_t)r * bias_stride + i];
      if (id < 0 || id >= vocab) continue;
      st_logit(row, id, ld_logit(row, id) + bias_vals[(size_t)r * bias_stride + i]);
    }
  }
  __threadfence_block();
  __syncthreads();
  const uint32_t* mask = allow_mask ? allow_mask + (size_t)r * mask_words : nullptr;
  auto allowed = [&](int i) { return !mask || ((mask[i >> 5] >> (i & 31)) & 1u); };

  // pass 1: max (for stability and greedy) and log-sum-exp of the unscaled logits
  ArgMax a{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x)
    if (allowed(i)) a = better(a, ArgMax{ld_logit(row, i), i});
  a = block_argmax(a, sm_a);
  const float vmax = a.v;
  const bool greedy = p.temperature <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / p.temperature;
  float se = 0.f, se_t = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    if (!allowed(i)) continue;
    const float d = ld_logit(row, i) - vmax;
    se += __expf(d);
    se_t += __expf(d * inv_t);
  }
  se = block_sum(se, sm_f);
  se_t = block_sum(se_t, sm_f);

  int chosen = a.i;
  if (!greedy) {
    // threshold in logit space: keep tokens with logit >= thr
    float thr = -INFINITY;
    if (p.min_p > 0.f) thr = fmaxf(thr, vmax + p.temperature * __logf(p.min_p));
    if (p.top_k > 0 && p.top_k < vocab) {
      // largest key with count(logit >= key) >= k
      uint32_t lo = 0, hi = fkey(vmax);
      while (lo < hi) {
        const uint32_t mid = lo + (hi - lo + 1) / 2;
        const float t = fkey_inv(mid);
        float c = 0.f;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x)
          if (allowed(i) && ld_logit(row, i) >= t) c += 1.f;
        c = block_sum(c, sm_f);
        if (c >= (float)p.top_k) lo = mid; else hi = mid - 1;
      }
      thr = fmaxf(thr, fkey_inv(lo));
    }
    if (p.top_p > 0.f && p.top_p < 1.f) {
      // largest key whose kept probability mass (after the other filters) is >= top_p
      float kept = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = ld_logit(row, i);
        if (allowed(i) && v >= thr) kept += __expf((v - vmax) * inv_t);
      }
      kept = block_sum(kept, sm_f);
      const float need = p.top_p * kept;
      uint32_t lo = fkey(thr == -INFINITY ? -3.0e38f : thr), hi = fkey(vmax);
      while (lo < hi) {
        const uint32_t mid = lo + (hi - lo + 1) / 2;
        const float t = fkey_inv(mid);
        float mass = 0.f;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
          const float v = ld_logit(row, i);
          if (allowed(i) && v >= t) mass += __expf((v - vmax) * inv_t);
        }
        mass = block_sum(mass, sm_f);
        if (mass >= need) lo = mid; else hi = mid - 1;
      }
      thr = fmaxf(thr, fkey_inv(lo));
    }
    // Gumbel-max over the kept set
    ArgMax g{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = ld_logit(row, i);
      if (!allowed(i) || v < thr) continue;
      const float u = philox_uniform(p.seed, p.draw, (uint32_t)i);
      const float gum = -__logf(-__logf(u));
      g = better(g, ArgMax{(v - vmax) * inv_t + gum, i});
    }
    g = block_argmax(g, sm_a);
    chosen = g.i;
  }
  if (threadIdx.x == 0) {
    out_ids[r] = chosen;
    if (out_logprobs) out_logprobs[r] = (ld_logit(row, chosen) - vmax) - __logf(se);
  }
  (void)sm_scalar;
  (void)se_t;
}

void sample_rows(void* logits, int is_fp32, long long ld, int rows, int vocab, const SampleRow* prm,
                 const int* pen_ids, const int* pen_counts, int pen_stride, const int* bias_ids,
                 const float* bias_vals, int bias_stride, const uint32_t* allow_mask, int mask_words,
                 int* out_ids, float* out_logprobs, cudaStream_t s) {
  if (rows <= 0) return;
  if (is_fp32)
    sample_rows_kernel<float><<<rows, kSampThreads, 0, s>>>(
        (float*)logits, ld, vocab, prm, pen_ids, pen_counts, pen_stride, bias_ids, bias_vals,
        bias_stride, allow_mask, mask_words, out_ids, out_logprobs);
  else
    sample_rows_kernel<__nv_bfloat16><<<rows, kSampThreads, 0, s>>>(
        (__nv_bfloat16*)logits, ld, vocab, prm, pen_ids, pen_counts, pen_stride, bias_ids, bias_vals,
        bias_stride, allow_mask, mask_words, out_ids, out_logprobs);
  cuda_check(cudaGetLastError(), "sample_rows_kernel");
}

// ---------------------------------------------------------------------------- speculative verify
// Greedy chain: target_ids[b][0..k] are the target's argmax tokens for the k+1 verify rows of
// sequence b (row i scores the token after draft i-1). Accept drafts while they match; the
// token at the first mismatch (or the bonus token after k matches) is emitted as well.
//
// The verify rows of sequence b start at row_start[b] of the target arrays when row_start is given
// (a ragged step: sequences carry different numbers of drafts), else at b * (k + 1).
__global__ void spec_verify_greedy_kernel(const int* __restrict__ draft_ids,
                                          const int* __restrict__ target_ids, int batch, int k,
                                          const int* __restrict__ row_start,
                                          const int* __restrict__ n_draft, int* __restrict__ n_accept,
                                          int* __restrict__ out_tokens) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int nd = n_draft ? min(n_draft[b], k) : k;
  if (nd < 0) return;
  const int* tgt = target_ids + (row_start ? (size_t)row_start[b] : (size_t)b * (k + 1));
  int acc = 0;
  while (acc < nd && draft_ids[(size_t)b * k + acc] == tgt[acc]) {
    out_tokens[(size_t)b * (k + 1) + acc] = draft_ids[(size_t)b * k + acc];
    ++acc;
  }
  out_tokens[(size_t)b * (k + 1) + acc] = tgt[acc];
  n_accept[b] = acc;
}

void spec_verify_greedy(const int* draft_ids, const int* target_ids, int batch, int k,
                        const int* row_start, const int* n_draft, int* n_accept, int* out_tokens,
                        cudaStream_t s) {
  if (batch <= 0) return;
  spec_verify_greedy_kernel<<<(batch + 63) / 64, 64, 0, s>>>(draft_ids, target_ids, batch, k, row_start,
                                                            n_draft, n_accept, out_tokens);
  cuda_check(cudaGetLastError(), "spec_verify_greedy_kernel");
}

// Exact rule on full distributions. One CTA per sequence. For draft position i with token x:
// accept with probability min(1, p(x)/q(x)); at the first rejection draw from
// normalise(max(0, p - q)); after nd acceptances draw the bonus token from p of row nd.
// p = softmax(target_logits / T), q = softmax(draft_logits / T). Without draft logits (drafts that
// come from a lookup, not from a model) q is the point mass on the draft token: it is accepted with
// probability p(x), and the residual is p with x removed. row_start as in the greedy kernel.
template <typename T>
__global__ void __launch_bounds__(kSampThreads)
spec_verify_sampled_kernel(const T* __restrict__ target_logits, long long ld_t,
                           const T* __restrict__ draft_logits, long long ld_d, int vocab,
                           const int* __restrict__ draft_ids, int k, const int* __restrict__ row_start,
                           const int* __restrict__ n_draft,
                           const SampleRow* __restrict__ prm, int* __restrict__ n_accept,
                           int* __restrict__ out_tokens) {
  __shared__ ArgMax sm_a[32];
  __shared__ float sm_f[32];
  const int b = blockIdx.x;
  const SampleRow p = prm[b];
  const int nd = n_draft ? min(n_draft[b], k) : k;
  const float inv_t = p.temperature > 0.f ? 1.f / p.temperature : 1.f;
  const size_t row0 = row_start ? (size_t)row_start[b] : (size_t)b * (k + 1);
  int acc = 0;
  int final_tok = -1;
  for (int i = 0; i <= nd; ++i) {
    const T* trow = target_logits + (row0 + i) * ld_t;
    // softmax statistics of the target row
    ArgMax a{-INFINITY, 0x7fffffff};
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) a = better(a, ArgMax{ld_logit(trow, j), j});
    a = block_argmax(a, sm_a);
    float zt = 0.f;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) zt += __expf((ld_logit(trow, j) - a.v) * inv_t);
    zt = block_sum(zt, sm_f);
    if (i == nd) {
      // bonus token from p
      if (p.temperature <= 0.f) { final_tok = a.i; break; }
      ArgMax g{-INFINITY, 0x7fffffff};
      for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        const float u = philox_uniform(p.seed, p.draw + 2 * i + 1, (uint32_t)j);
        g = better(g, ArgMax{(ld_logit(trow, j) - a.v) * inv_t - __logf(-__logf(u)), j});
      }
      g = block_argmax(g, sm_a);
      final_tok = g.i;
      break;
    }
    const T* drow = draft_logits ? draft_logits + ((size_t)b * k + i) * ld_d : nullptr;
    ArgMax ad{0.f, 0};
    float zd = 1.f;
    if (drow) {
      ad = ArgMax{-INFINITY, 0x7fffffff};
      for (int j = threadIdx.x; j < vocab; j += blockDim.x) ad = better(ad, ArgMax{ld_logit(drow, j), j});
      ad = block_argmax(ad, sm_a);
      zd = 0.f;
      for (int j = threadIdx.x; j < vocab; j += blockDim.x) zd += __expf((ld_logit(drow, j) - ad.v) * inv_t);
      zd = block_sum(zd, sm_f);
    }
    const int x = draft_ids[(size_t)b * k + i];
    bool accept;
    if (p.temperature <= 0.f) {
      accept = (x == a.i);
    } else {
      const float px = __expf((ld_logit(trow, x) - a.v) * inv_t) / zt;
      const float qx = drow ? __expf((ld_logit(drow, x) - ad.v) * inv_t) / zd : 1.f;
      const float u = philox_uniform(p.seed, p.draw + 2 * i, 0xffffffffu);
      accept = qx <= 0.f ? true : (u < fminf(1.f, px / qx));
    }
    if (accept) {
      if (threadIdx.x == 0) out_tokens[(size_t)b * (k + 1) + acc] = x;
      ++acc;
      continue;
    }
    if (p.temperature <= 0.f) { final_tok = a.i; break; }
    // residual distribution max(0, p - q), sampled with Gumbel-max on its log
    ArgMax g{-INFINITY, 0x7fffffff};
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
      const float pj = __expf((ld_logit(trow, j) - a.v) * inv_t) / zt;
      const float qj = drow ? __expf((ld_logit(drow, j) - ad.v) * inv_t) / zd : (j == x ? 1.f : 0.f);
      const float rj = pj - qj;
      if (rj <= 0.f) continue;
      const float u = philox_uniform(p.seed, p.draw + 2 * i + 1, (uint32_t)j);
      g = better(g, ArgMax{__logf(rj) - __logf(-__logf(u)), j});
    }
    g = block_argmax(g, sm_a);
    final_tok = g.i == 0x7fffffff ? a.i : g.i;
    break;
  }
  if (threadIdx.x == 0) {
    out_tokens[(size_t)b * (k + 1) + acc] = final_tok;
    n_accept[b] = acc;
  }
}

void spec_verify_sampled(const void* target_logits, long long ld_t, const void* draft_logits,
                         long long ld_d, int is_fp32, int vocab, const int* draft_ids, int batch,
                         int k, const int* row_start, const int* n_draft, const SampleRow* prm,
                         int* n_accept, int* out_tokens, cudaStream_t s) {
  if (batch <= 0) return;
  if (is_fp32)
    spec_verify_sampled_kernel<float><<<batch, kSampThreads, 0, s>>>(
        (const float*)target_logits, ld_t, (const float*)draft_logits, ld_d, vocab, draft_ids, k,
        row_start, n_draft, prm, n_accept, out_tokens);
  else
    spec_verify_sampled_kernel<__nv_bfloat16><<<batch, kSampThreads, 0, s>>>(
        (const __nv_bfloat16*)target_logits, ld_t, (const __nv_bfloat16*)draft_logits, ld_d, vocab,
        draft_ids, k, row_start, n_draft, prm, n_accept, out_tokens);
  cuda_check(cudaGetLastError(), "spec_verify_sampled_kernel");
}

}  // namespace fllm
