// Generic paged attention: one CTA per (query row, query head), four warps that
// walk the visible keys with an online softmax and merge at the end. Handles any
// ragged mix of prefill and decode rows, GQA, sliding windows, attention sinks and
// logit soft-capping. This is the always-correct path and the oracle for the
// tensor-core kernels; its role matches rust/engine/cuda/attention.cu:41-115.
//
// Tree attention (speculative draft trees, rust/engine/cuda/attn_tree.cu:33): the rows of a sequence are the
// nodes of a draft tree whose keys / values sit behind the committed context in slot order. Row t then sees
// token j if j < tree_base[t] (context) or bit (j - tree_base[t]) of tree_mask[t] is set (its ancestors and
// itself): the M x M mask of a tree of at most 64 nodes is one 64-bit word per row.
//
// KV cache layout: [block][kv_head][block_size][head_dim], bf16 or e4m3 bytes (fp8 KV cache: values are
// stored unscaled, e4m3 covers +-448; the reference's counterpart is rust/engine/cuda/kv_quant.cu).
#include <cuda_fp8.h>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

__device__ __forceinline__ float kv_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float kv_to_float(uint8_t v) {
  __nv_fp8_e4m3 f;
  f.__x = v;
  return static_cast<float>(f);
}

template <int D, typename KV>
__global__ void __launch_bounds__(128)
attn_generic_kernel(const __nv_bfloat16* __restrict__ q, long long ldq,
                    const KV* __restrict__ k_cache,
                    const KV* __restrict__ v_cache, const int* __restrict__ block_tables,
                    int max_blocks, const int* __restrict__ row_seq,
                    const int* __restrict__ positions, __nv_bfloat16* __restrict__ out,
                    long long ldo, int hq, int hkv, int block_size, float scale, int window,
                    const float* __restrict__ sinks, float softcap,
                    const unsigned long long* __restrict__ tree_mask, const int* __restrict__ tree_base) {
  constexpr int EPL = D / 32;
  const int h = blockIdx.x;
  const int t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = h / (hq / hkv);
  const int seq = row_seq[t];
  const int pos = positions[t];
  const int kv_len = pos + 1;
  const int kv_begin = (window > 0 && kv_len > window) ? kv_len - window : 0;
  const int* table = block_tables + (size_t)seq * max_blocks;
  const unsigned long long tmask = tree_mask ? tree_mask[t] : ~0ull;
  const int tbase = tree_mask ? tree_base[t] : kv_len;
  auto visible = [&](int j) -> bool {
    if (j >= kv_len) return false;
    if (j < tbase) return true;
    const int b = j - tbase;
    return b < 64 && ((tmask >> b) & 1ull);
  };

  float qv[EPL];
  {
    const __nv_bfloat16* qp = q + (size_t)t * ldq + (size_t)h * D + lane * EPL;
#pragma unroll
    for (int j = 0; j < EPL; ++j) qv[j] = __bfloat162float(qp[j]) * scale;
  }
  float m = -INFINITY, l = 0.f;
  float acc[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) acc[j] = 0.f;

  constexpr int UN = 4;
  for (int base = kv_begin + warp * UN; base < kv_len; base += 4 * UN) {
    float s[UN];
    float vv[UN][EPL];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int j = base + u;
      s[u] = 0.f;
      if (visible(j)) {
        const int blk = table[j / block_size];
        const size_t off = (((size_t)blk * hkv + kvh) * block_size + (j % block_size)) * D + lane * EPL;
        const KV* kp = k_cache + off;
        const KV* vp = v_cache + off;
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          s[u] += qv[e] * kv_to_float(kp[e]);
          vv[u][e] = kv_to_float(vp[e]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < EPL; ++e) vv[u][e] = 0.f;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int u = 0; u < UN; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      if (visible(base + u)) {
        float sc = s[u];
        if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
        const float mn = fmaxf(m, sc);
        const float corr = __expf(m - mn);
        const float p = __expf(sc - mn);
        l = l * corr + p;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] = acc[e] * corr + p * vv[u][e];
        m = mn;
      }
    }
  }

  __shared__ float sm_m[4], sm_l[4];
  __shared__ float sm_acc[4][D];
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
  for (int e = 0; e < EPL; ++e) sm_acc[warp][lane * EPL + e] = acc[e];
  __syncthreads();
  if (warp == 0) {
    float mm = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
    const float sink = sinks ? sinks[h] : -INFINITY;
    if (sinks) mm = fmaxf(mm, sink);
    float ll = sinks ? __expf(sink - mm) : 0.f;
    float o[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[e] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = sm_m[w] == -INFINITY ? 0.f : __expf(sm_m[w] - mm);
      ll += sm_l[w] * c;
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[e] += sm_acc[w][lane * EPL + e] * c;
    }
    const float inv = ll > 0.f ? 1.f / ll : 0.f;
    __nv_bfloat16* op = out + (size_t)t * ldo + (size_t)h * D + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) op[e] = __float2bfloat16(o[e] * inv);
  }
}

void attention_generic_bf16(const void* q, long long ldq, const void* k_cache, const void* v_cache,
                            const int* block_tables, int max_blocks, const int* row_seq,
                            const int* positions, void* out, long long ldo, int tokens, int hq,
                            int hkv, int head_dim, int block_size, float scale, int window,
                            const float* sinks, float softcap, cudaStream_t s, int kv_fp8,
                            const unsigned long long* tree_mask, const int* tree_base) {
  if (tokens <= 0) return;
  dim3 grid(hq, tokens);
#define FLLM_ATT(DD)                                                                           \
  do {                                                                                         \
    if (kv_fp8)                                                                                \
      attn_generic_kernel<DD, uint8_t><<<grid, 128, 0, s>>>(                                   \
          (const __nv_bfloat16*)q, ldq, (const uint8_t*)k_cache, (const uint8_t*)v_cache, block_tables, max_blocks, \
          row_seq, positions, (__nv_bfloat16*)out, ldo, hq, hkv, block_size, scale, window, sinks, softcap, tree_mask, tree_base); \
    else                                                                                       \
      attn_generic_kernel<DD, __nv_bfloat16><<<grid, 128, 0, s>>>(                             \
          (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_tables, \
          max_blocks, row_seq, positions, (__nv_bfloat16*)out, ldo, hq, hkv, block_size, scale, window, sinks, \
          softcap, tree_mask, tree_base);                                                      \
  } while (0)
  switch (head_dim) {
    case 64: FLLM_ATT(64); break;
    case 128: FLLM_ATT(128); break;
    case 256: FLLM_ATT(256); break;
    default: throw std::runtime_error("attention_generic_bf16: head_dim must be 64, 128 or 256");
  }
#undef FLLM_ATT
  cuda_check(cudaGetLastError(), "attn_generic_kernel");
}

}  // namespace fllm
