// Mixture-of-experts routing and data movement around the grouped tcgen05 GEMM:
//
//   moe_route_kernel    one warp per token: top-k over the router logits, weights = softmax over
//                       the selected logits (gpt-oss) or softmax over all experts renormalised
//                       over the selection (Mixtral / Qwen-MoE);
//   moe_align_kernel    one CTA: count rows per expert, lay the experts' row segments out back to
//                       back, each padded to the token-tile width, and emit the tile list
//                       (expert, first row) that the grouped GEMM walks; sizes stay on the device
//                       so the whole layer can live in a CUDA graph;
//   moe_gather_kernel   permuted activations xp[row] = x[token(row)] (zero rows for padding);
//   moe_combine_kernel  out[token] = sum_j weight[token, j] * y[row(token, j)] in slot order, so
//                       the result does not depend on scheduling.
//
// Reference counterparts: rust/engine/cuda/moe.cu:40-150 (moe_route2), :159-205 (moe_align),
// :533-597 (combine2). The reference routes on the host inside a device group
// (rust/engine/src/rust_decoder.rs:7621-7729); here nothing leaves the device.
#include <algorithm>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

__global__ void moe_route_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, const __nv_bfloat16* __restrict__ bias,
                                 int tokens, int experts, int k, int softmax_all, int* __restrict__ ids,
                                 float* __restrict__ weights) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  constexpr int MAXPL = 8;                      // up to 256 experts
  float v[MAXPL];
#pragma unroll
  for (int i = 0; i < MAXPL; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < experts ? __bfloat162float(logits[(size_t)t * ld + e]) + (bias ? __bfloat162float(bias[e]) : 0.f) : -INFINITY;
  }
  float denom_all = 0.f, vmax = -INFINITY;
  if (softmax_all) {
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) vmax = fmaxf(vmax, v[i]);
    vmax = warp_max(vmax);
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) denom_all += v[i] == -INFINITY ? 0.f : __expf(v[i] - vmax);
    denom_all = warp_sum(denom_all);
  }
  float sel_v[8];
  int sel_e[8];
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best || (v[i] == best && e < best_e)) { best = v[i]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    sel_v[j] = best;
    sel_e[j] = best_e;
    if ((best_e & 31) == lane) v[best_e >> 5] = -INFINITY;    // remove the winner
  }
  if (lane == 0) {
    float w[8], sum = 0.f;
    for (int j = 0; j < k; ++j) {
      w[j] = softmax_all ? __expf(sel_v[j] - vmax) / denom_all : __expf(sel_v[j] - sel_v[0]);
      sum += w[j];
    }
    for (int j = 0; j < k; ++j) {
      ids[(size_t)t * k + j] = sel_e[j];
      weights[(size_t)t * k + j] = w[j] / sum;
    }
  }
}

// Routers that weigh experts by their score: score = softmax over all experts (score_kind 1) or sigmoid (2) of the logit; the
// k experts with the largest score + select_bias are taken (the bias only steers the choice: DeepSeek-V3, GLM-4.5, ERNIE 4.5);
// weights = the scores of the chosen experts, renormalised on request, times `scale`. One warp per token, up to 256 experts.
__global__ void moe_route_scored_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, const float* __restrict__ select_bias,
                                        int tokens, int experts, int k, int score_kind, int renorm, float scale, int* __restrict__ ids,
                                        float* __restrict__ weights) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  constexpr int MAXPL = 8;
  float sc[MAXPL], ch[MAXPL];
  float vmax = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAXPL; ++i) {
    const int e = lane + 32 * i;
    sc[i] = e < experts ? __bfloat162float(logits[(size_t)t * ld + e]) : -INFINITY;
    vmax = fmaxf(vmax, sc[i]);
  }
  if (score_kind == 1) {
    vmax = warp_max(vmax);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) {
      sc[i] = sc[i] == -INFINITY ? 0.f : __expf(sc[i] - vmax);
      den += sc[i];
    }
    den = warp_sum(den);
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) sc[i] /= den;
  } else {
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) sc[i] = sc[i] == -INFINITY ? 0.f : 1.f / (1.f + __expf(-sc[i]));
  }
#pragma unroll
  for (int i = 0; i < MAXPL; ++i) {
    const int e = lane + 32 * i;
    ch[i] = e < experts ? sc[i] + (select_bias ? select_bias[e] : 0.f) : -INFINITY;
  }
  float sel_s[8];
  int sel_e[8];
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY, best_s = 0.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) {
      const int e = lane + 32 * i;
      if (ch[i] > best || (ch[i] == best && e < best_e)) { best = ch[i]; best_e = e; best_s = sc[i]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, best_s, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; best_s = os; }
    }
    sel_s[j] = best_s;
    sel_e[j] = best_e;
    if ((best_e & 31) == lane) ch[best_e >> 5] = -INFINITY;    // remove the winner
  }
  if (lane == 0) {
    float sum = 0.f;
    for (int j = 0; j < k; ++j) sum += sel_s[j];
    const float f = (renorm ? 1.f / (sum + 1e-20f) : 1.f) * scale;
    for (int j = 0; j < k; ++j) {
      ids[(size_t)t * k + j] = sel_e[j];
      weights[(size_t)t * k + j] = sel_s[j] * f;
    }
  }
}

void moe_route_scored(const void* logits, long long ld, const float* select_bias, int tokens, int experts, int k, int score_kind,
                      int renorm, float scale, int* ids, float* weights, cudaStream_t s) {
  if (tokens <= 0) return;
  if (experts > 256 || k > 8 || (score_kind != 1 && score_kind != 2)) throw std::runtime_error("moe_route_scored: at most 256 experts, top-8, score kind 1 or 2");
  moe_route_scored_kernel<<<(tokens + 3) / 4, 128, 0, s>>>((const __nv_bfloat16*)logits, ld, select_bias, tokens, experts, k, score_kind,
                                                           renorm, scale, ids, weights);
  cuda_check(cudaGetLastError(), "moe_route_scored_kernel");
}

void moe_route(const void* logits, long long ld, const void* bias, int tokens, int experts, int k, int softmax_all,
               int* ids, float* weights, cudaStream_t s) {
  if (tokens <= 0) return;
  if (experts > 256 || k > 8) throw std::runtime_error("moe_route: at most 256 experts and top-8");
  moe_route_kernel<<<(tokens + 3) / 4, 128, 0, s>>>((const __nv_bfloat16*)logits, ld, (const __nv_bfloat16*)bias,
                                                     tokens, experts, k, softmax_all, ids, weights);
  cuda_check(cudaGetLastError(), "moe_route_kernel");
}

// Single CTA. expert_lo/expert_hi select the experts this rank holds; entries routed elsewhere get
// row -1. Outputs: row_of[tokens*k] (permuted row of each (token, slot) or -1), token_of[rows_cap]
// (token of each permuted row, -1 = padding), tile_expert / tile_row0 / num_tiles, total_rows.
__global__ void __launch_bounds__(1024) moe_align_kernel(const int* __restrict__ ids, int entries, int experts,
                                                         int expert_lo, int expert_hi, int bn, int k,
                                                         int* __restrict__ row_of, int* __restrict__ token_of,
                                                         int rows_cap, int* __restrict__ tile_expert,
                                                         int* __restrict__ tile_row0, int* __restrict__ num_tiles,
                                                         int max_tiles, int staged) {
  __shared__ int cnt[512], off[513], fill[512];
  extern __shared__ int ids_s[];              // the first `staged` ids: the per-expert scans below read them from here
  for (int e = threadIdx.x; e < 512; e += blockDim.x) { cnt[e] = 0; fill[e] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = ids[i];
    if (i < staged) ids_s[i] = e;
    if (e >= expert_lo && e < expert_hi) atomicAdd(&cnt[e - expert_lo], 1);
  }
  __syncthreads();
  const int local = expert_hi - expert_lo;
  if (threadIdx.x == 0) {
    int o = 0, nt = 0;
    for (int e = 0; e < local; ++e) {
      off[e] = o;
      const int padded = (cnt[e] + bn - 1) / bn * bn;
      for (int r = 0; r < padded && nt < max_tiles; r += bn) {
        tile_expert[nt] = e;
        tile_row0[nt] = o + r;
        ++nt;
      }
      o += padded;
    }
    off[local] = o;
    num_tiles[0] = nt;
    num_tiles[1] = o;                         // total permuted rows (incl. padding)
  }
  __syncthreads();
  for (int i = threadIdx.x; i < rows_cap; i += blockDim.x) token_of[i] = -1;
  __syncthreads();
  // Deterministic placement: entries of an expert keep their (token, slot) order. The entries are taken 1024 at a time,
  // one per thread; the warps of a round go one after the other, and inside a warp the lanes that drew the same expert
  // rank themselves with a match mask, so no thread ever scans the list.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int base = 0; base < entries; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const int e = i < entries ? (i < staged ? ids_s[i] : ids[i]) - expert_lo : -1;
    const bool valid = e >= 0 && e < local;
    const int warps = min((int)(blockDim.x >> 5), (entries - base + 31) >> 5);
    for (int w = 0; w < warps; ++w) {
      if (warp == w) {
        const unsigned same = __match_any_sync(0xffffffffu, valid ? e : -1 - lane);      // other lanes with this expert
        if (valid) {
          const int pos = off[e] + fill[e] + __popc(same & ((1u << lane) - 1u));
          row_of[i] = pos;
          if (pos < rows_cap) token_of[pos] = i / k;
        }
        __syncwarp();
        if (valid && lane == __ffs(same) - 1) fill[e] += __popc(same);
      }
      __syncthreads();
    }
    if (i < entries && !valid) row_of[i] = -1;
  }
}

void moe_align(const int* ids, int tokens, int k, int experts, int expert_lo, int expert_hi, int bn, int* row_of,
               int* token_of, int rows_cap, int* tile_expert, int* tile_row0, int* num_tiles, int max_tiles,
               cudaStream_t s) {
  if (expert_hi - expert_lo > 512) throw std::runtime_error("moe_align: at most 512 local experts");
  const int staged = std::min(tokens * k, 10240);              // 40 KiB of dynamic shared memory at most
  moe_align_kernel<<<1, 1024, (size_t)staged * sizeof(int), s>>>(ids, tokens * k, experts, expert_lo, expert_hi, bn, k, row_of, token_of,
                                                                 rows_cap, tile_expert, tile_row0, num_tiles, max_tiles, staged);
  cuda_check(cudaGetLastError(), "moe_align_kernel");
}

__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ token_of,
                                  __nv_bfloat16* __restrict__ xp, int hidden) {
  const int row = blockIdx.x;
  const int t = token_of[row];
  uint4* dst = reinterpret_cast<uint4*>(xp + (size_t)row * hidden);
  if (t < 0) {
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * ldx);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

void moe_gather(const void* x, long long ldx, const int* token_of, void* xp, int rows_cap, int hidden, cudaStream_t s) {
  if (rows_cap <= 0) return;
  moe_gather_kernel<<<rows_cap, 128, 0, s>>>((const __nv_bfloat16*)x, ldx, token_of, (__nv_bfloat16*)xp, hidden);
  cuda_check(cudaGetLastError(), "moe_gather_kernel");
}

__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, long long ldy, const int* __restrict__ row_of,
                                   const float* __restrict__ weights, int k, __nv_bfloat16* __restrict__ out,
                                   long long ldo, int hidden) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int row = row_of[(size_t)t * k + j];
      if (row < 0) continue;                                  // expert lives on another rank
      const float w = weights[(size_t)t * k + j];
      const uint4 v = reinterpret_cast<const uint4*>(y + (size_t)row * ldy)[i];
      const uint32_t* vw = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16x2(vw[q]);
        acc[2 * q] += w * f.x;
        acc[2 * q + 1] += w * f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + (size_t)t * ldo)[i] = o;
  }
}

void moe_combine(const void* y, long long ldy, const int* row_of, const float* weights, int tokens, int k, void* out,
                 long long ldo, int hidden, cudaStream_t s) {
  if (tokens <= 0) return;
  moe_combine_kernel<<<tokens, 128, 0, s>>>((const __nv_bfloat16*)y, ldy, row_of, weights, k, (__nv_bfloat16*)out, ldo,
                                            hidden);
  cuda_check(cudaGetLastError(), "moe_combine_kernel");
}

}  // namespace fllm
