// Multi-head latent attention over the compressed cache (DeepSeek-V2 / V3 family). A token stores one row of
// 576 values: the normalised KV latent (512) followed by the rotated shared key part (64). With the key
// up-projection absorbed into the query and the value up-projection applied after the softmax, every head is a
// query of width 576 against that one row per token, and its output is a weighted sum of the 512-wide latents:
// multi-query attention whose values are a prefix of its keys. The reference's counterparts are
// rust/engine/cuda/mla_latent.cu and mla_decode.cu (absorbed query, 576-wide cache).
//
// One CTA per (query row, group of HG heads); its four warps take every fourth key, keep an online softmax per
// head and are merged through shared memory. A key row is fetched once per warp and used by all HG heads, so the
// cache traffic out of L2 is 1 / HG of a kernel with one head per CTA. Lane l owns key elements [18 l, 18 l + 18)
// for the dot products and latent columns [16 l, 16 l + 16) for the output.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <stdexcept>

#include "fllm_ops.h"

namespace fllm {
namespace {
using bf16 = __nv_bfloat16;
constexpr int kLatent = 512, kRope = 64, kRow = kLatent + kRope;

template <int HG>
__global__ void __launch_bounds__(128) mla_attn_kernel(const bf16* __restrict__ q, long long ldq, const bf16* __restrict__ cache,
                                                       const int* __restrict__ block_tables, int max_blocks,
                                                       const int* __restrict__ row_seq, const int* __restrict__ positions,
                                                       bf16* __restrict__ out, long long ldo, int H, int block_size, float scale) {
  constexpr int EK = kRow / 32, EV = kLatent / 32;      // 18 key elements and 16 latent columns per lane
  const int h0 = blockIdx.x * HG, t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_len = positions[t] + 1;
  const int* table = block_tables + (size_t)row_seq[t] * max_blocks;

  float qv[HG][EK];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    const int h = min(h0 + g, H - 1);                    // a ragged last group repeats the last head, unstored
    const __nv_bfloat162* qp = reinterpret_cast<const __nv_bfloat162*>(q + (size_t)t * ldq + (size_t)h * kRow + lane * EK);
#pragma unroll
    for (int j = 0; j < EK / 2; ++j) {
      const float2 f = __bfloat1622float2(qp[j]);
      qv[g][2 * j] = f.x * scale, qv[g][2 * j + 1] = f.y * scale;
    }
  }
  float m[HG], l[HG], acc[HG][EV];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    m[g] = -INFINITY, l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EV; ++e) acc[g][e] = 0.f;
  }
  for (int j = warp; j < kv_len; j += 4) {
    const bf16* row = cache + ((size_t)table[j / block_size] * block_size + (j % block_size)) * kRow;
    float kvv[EK], vv[EV];
    {
      const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(row + lane * EK);
#pragma unroll
      for (int e = 0; e < EK / 2; ++e) {
        const float2 f = __bfloat1622float2(kp[e]);
        kvv[2 * e] = f.x, kvv[2 * e + 1] = f.y;
      }
      const uint4* vp = reinterpret_cast<const uint4*>(row + lane * EV);
#pragma unroll
      for (int e = 0; e < EV / 8; ++e) {
        const uint4 raw = vp[e];
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(hh[i]);
          vv[8 * e + 2 * i] = f.x, vv[8 * e + 2 * i + 1] = f.y;
        }
      }
    }
    float s[HG];
#pragma unroll
    for (int g = 0; g < HG; ++g) {
      s[g] = 0.f;
#pragma unroll
      for (int e = 0; e < EK; ++e) s[g] = fmaf(qv[g][e], kvv[e], s[g]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int g = 0; g < HG; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
    }
#pragma unroll
    for (int g = 0; g < HG; ++g) {
      const float mn = fmaxf(m[g], s[g]);
      const float corr = __expf(m[g] - mn), p = __expf(s[g] - mn);
      l[g] = l[g] * corr + p;
#pragma unroll
      for (int e = 0; e < EV; ++e) acc[g][e] = fmaf(acc[g][e], corr, p * vv[e]);
      m[g] = mn;
    }
  }
  __shared__ float sm_m[4][HG], sm_l[4][HG];
  __shared__ float sm_acc[4][HG][kLatent];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    if (lane == 0) sm_m[warp][g] = m[g], sm_l[warp][g] = l[g];
#pragma unroll
    for (int e = 0; e < EV; ++e) sm_acc[warp][g][lane * EV + e] = acc[g][e];
  }
  __syncthreads();
  // warp w merges heads w, w + 4, ... of the group
  for (int g = warp; g < HG; g += 4) {
    if (h0 + g >= H) break;
    const float mm = fmaxf(fmaxf(sm_m[0][g], sm_m[1][g]), fmaxf(sm_m[2][g], sm_m[3][g]));
    float ll = 0.f, o[EV];
#pragma unroll
    for (int e = 0; e < EV; ++e) o[e] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = sm_m[w][g] == -INFINITY ? 0.f : __expf(sm_m[w][g] - mm);
      ll = fmaf(sm_l[w][g], c, ll);
#pragma unroll
      for (int e = 0; e < EV; ++e) o[e] = fmaf(sm_acc[w][g][lane * EV + e], c, o[e]);
    }
    const float inv = ll > 0.f ? 1.f / ll : 0.f;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * ldo + (size_t)(h0 + g) * kLatent + lane * EV);
#pragma unroll
    for (int e = 0; e < EV / 2; ++e) op[e] = __floats2bfloat162_rn(o[2 * e] * inv, o[2 * e + 1] * inv);
  }
}
}  // namespace

// q [tokens][H][576] (absorbed query | rotated query part), cache [blocks][block_size][576], out [tokens][H][512].
void attention_mla_bf16(const void* q, long long ldq, const void* cache, const int* block_tables, int max_blocks, const int* row_seq,
                        const int* positions, void* out, long long ldo, int tokens, int H, int block_size, float scale, cudaStream_t s) {
  if (tokens <= 0) return;
  if ((ldq & 1) || (ldo & 1) || (reinterpret_cast<uintptr_t>(cache) & 15))
    throw std::runtime_error("attention_mla_bf16: even leading dimensions and a 16-byte aligned cache are required");
  constexpr int HG = 4;
  mla_attn_kernel<HG><<<dim3((H + HG - 1) / HG, tokens), 128, 0, s>>>(static_cast<const bf16*>(q), ldq, static_cast<const bf16*>(cache),
                                                                     block_tables, max_blocks, row_seq, positions, static_cast<bf16*>(out),
                                                                     ldo, H, block_size, scale);
}

}  // namespace fllm
