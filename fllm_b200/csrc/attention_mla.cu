// Multi-head latent attention over the compressed cache (DeepSeek-V2 / V3 family). A token stores one row of
// 576 values: the normalised KV latent (512) followed by the rotated shared key part (64). With the key
// up-projection absorbed into the query and the value up-projection applied after the softmax, every head is a
// query of width 576 against that one row per token, and its output is a weighted sum of the 512-wide latents:
// multi-query attention whose values are a prefix of its keys. The reference's counterparts are
// rust/engine/cuda/mla_latent.cu and mla_decode.cu (absorbed query, 576-wide cache).
//
// One CTA per (query row, group of HG heads); its NW warps take every NW-th key, keep an online softmax per
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

template <int HG, int NW>
__global__ void __launch_bounds__(NW * 32) mla_attn_kernel(const bf16* __restrict__ q_abs, long long qa_t, long long qa_h,
                                                           const bf16* __restrict__ q_pe, const bf16* __restrict__ cache,
                                                           const int* __restrict__ block_tables, int max_blocks,
                                                           const int* __restrict__ row_seq, const int* __restrict__ positions,
                                                           bf16* __restrict__ out, long long o_t, long long o_h, int H, int block_size,
                                                           float scale) {
  constexpr int EK = kRow / 32, EV = kLatent / 32;      // 18 key elements and 16 latent columns per lane
  const int h0 = blockIdx.x * HG, t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_len = positions[t] + 1;
  const int* table = block_tables + (size_t)row_seq[t] * max_blocks;

  float qv[HG][EK];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    const int h = min(h0 + g, H - 1);                    // a ragged last group repeats the last head, unstored
    // element e of the 576-wide query: the absorbed part below 512, the rotated part above (pairs never straddle)
    const bf16* qa = q_abs + (size_t)t * qa_t + (size_t)h * qa_h;
    const bf16* qr = q_pe + ((size_t)t * H + h) * kRope;
#pragma unroll
    for (int j = 0; j < EK / 2; ++j) {
      const int e = lane * EK + 2 * j;
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(e < kLatent ? qa + e : qr + (e - kLatent)));
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
  for (int j = warp; j < kv_len; j += NW) {
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
  __shared__ float sm_m[NW][HG], sm_l[NW][HG];
  __shared__ float sm_acc[NW][HG][kLatent];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    if (lane == 0) sm_m[warp][g] = m[g], sm_l[warp][g] = l[g];
#pragma unroll
    for (int e = 0; e < EV; ++e) sm_acc[warp][g][lane * EV + e] = acc[g][e];
  }
  __syncthreads();
  // warp w merges heads w, w + NW, ... of the group
  for (int g = warp; g < HG; g += NW) {
    if (h0 + g >= H) break;
    float mm = sm_m[0][g];
#pragma unroll
    for (int w = 1; w < NW; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, o[EV];
#pragma unroll
    for (int e = 0; e < EV; ++e) o[e] = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float c = sm_m[w][g] == -INFINITY ? 0.f : __expf(sm_m[w][g] - mm);
      ll = fmaf(sm_l[w][g], c, ll);
#pragma unroll
      for (int e = 0; e < EV; ++e) o[e] = fmaf(sm_acc[w][g][lane * EV + e], c, o[e]);
    }
    const float inv = ll > 0.f ? 1.f / ll : 0.f;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * o_t + (size_t)(h0 + g) * o_h + lane * EV);
#pragma unroll
    for (int e = 0; e < EV / 2; ++e) op[e] = __floats2bfloat162_rn(o[2 * e] * inv, o[2 * e + 1] * inv);
  }
}

// Per token: RMSNorm of the 512 latent values and rotation of the 64 shared key values into the token's cache row
// (skipped for padding rows, slot < 0), and rotation of every head's 64 query values into q_pe [T][H][64]. Pairs are
// neighbours (x[2i], x[2i+1]); cos / sin carry the YaRN attention factor.
__global__ void __launch_bounds__(128) mla_prepare_kernel(const bf16* __restrict__ ckv, long long ldc, const bf16* __restrict__ q, long long ldq,
                                                          int q_head_stride, int q_rope_offset, const int* __restrict__ positions,
                                                          const int* __restrict__ slots, const float* __restrict__ inv_freq, float attn_factor,
                                                          const bf16* __restrict__ norm_w, float eps, bf16* __restrict__ cache,
                                                          bf16* __restrict__ q_pe, int H) {
  const int t = blockIdx.x, tid = threadIdx.x;
  const float pos = (float)positions[t];
  const int slot = slots[t];
  const bf16* row = ckv + (size_t)t * ldc;
  // latent: four values per thread
  float v[4], ss = 0.f;
  {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(row + tid * 4);
    const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
    ss = a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
  }
  __shared__ float part[4];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) part[tid >> 5] = ss;
  __syncthreads();
  const float inv = rsqrtf((part[0] + part[1] + part[2] + part[3]) / kLatent + eps);
  if (slot >= 0) {
    bf16* dst = cache + (size_t)slot * kRow;
    __nv_bfloat162* d = reinterpret_cast<__nv_bfloat162*>(dst + tid * 4);
    const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(norm_w + tid * 4);
    const float2 w0 = __bfloat1622float2(w[0]), w1 = __bfloat1622float2(w[1]);
    d[0] = __floats2bfloat162_rn(v[0] * inv * w0.x, v[1] * inv * w0.y);
    d[1] = __floats2bfloat162_rn(v[2] * inv * w1.x, v[3] * inv * w1.y);
    if (tid < kRope / 2) {
      float sn, cs;
      sincosf(pos * inv_freq[tid], &sn, &cs);
      sn *= attn_factor, cs *= attn_factor;
      const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + kLatent + 2 * tid));
      *reinterpret_cast<__nv_bfloat162*>(dst + kLatent + 2 * tid) = __floats2bfloat162_rn(x.x * cs - x.y * sn, x.x * sn + x.y * cs);
    }
  }
  for (int i = tid; i < H * (kRope / 2); i += 128) {
    const int h = i / (kRope / 2), f = i % (kRope / 2);
    float sn, cs;
    sincosf(pos * inv_freq[f], &sn, &cs);
    sn *= attn_factor, cs *= attn_factor;
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q + (size_t)t * ldq + (size_t)h * q_head_stride + q_rope_offset + 2 * f));
    *reinterpret_cast<__nv_bfloat162*>(q_pe + ((size_t)t * H + h) * kRope + 2 * f) = __floats2bfloat162_rn(x.x * cs - x.y * sn, x.x * sn + x.y * cs);
  }
}
}  // namespace

// q_abs: absorbed query part, element (t, h, e) at q_abs[t * qa_t + h * qa_h + e] (e < 512); q_pe [tokens][H][64] rotated
// query part; cache [blocks][block_size][576]; out element (t, h, e) at out[t * o_t + h * o_h + e].
void attention_mla_bf16(const void* q_abs, long long qa_t, long long qa_h, const void* q_pe, const void* cache, const int* block_tables,
                        int max_blocks, const int* row_seq, const int* positions, void* out, long long o_t, long long o_h, int tokens,
                        int H, int block_size, float scale, cudaStream_t s) {
  if (tokens <= 0) return;
  if ((qa_t & 1) || (qa_h & 1) || (o_t & 1) || (o_h & 1) || (reinterpret_cast<uintptr_t>(cache) & 15) ||
      (reinterpret_cast<uintptr_t>(q_abs) & 3) || (reinterpret_cast<uintptr_t>(q_pe) & 3) || (reinterpret_cast<uintptr_t>(out) & 3))
    throw std::runtime_error("attention_mla_bf16: even strides, 4-byte aligned queries / output and a 16-byte aligned cache are required");
  // Few rows (decode): two heads per CTA and eight warps over the keys, so that a step fills the machine and a warp
  // walks an eighth of the context; many rows (prefill): four heads per CTA, which quarters the cache traffic out of L2.
  const bf16* qa = static_cast<const bf16*>(q_abs);
  const bf16* qr = static_cast<const bf16*>(q_pe);
  const bf16* cp = static_cast<const bf16*>(cache);
  bf16* op = static_cast<bf16*>(out);
  if ((long long)((H + 3) / 4) * tokens < 2 * 148) {
    mla_attn_kernel<2, 8><<<dim3((H + 1) / 2, tokens), 256, 0, s>>>(qa, qa_t, qa_h, qr, cp, block_tables, max_blocks, row_seq, positions, op,
                                                                   o_t, o_h, H, block_size, scale);
  } else {
    mla_attn_kernel<4, 4><<<dim3((H + 3) / 4, tokens), 128, 0, s>>>(qa, qa_t, qa_h, qr, cp, block_tables, max_blocks, row_seq, positions, op,
                                                                   o_t, o_h, H, block_size, scale);
  }
}

// ckv [tokens][>= 576] (latent | shared key part, leading dimension ldc); q [tokens][H][head] with the 64 rotary values of a
// head at q_rope_offset; cache rows are addressed by slot (block * block_size + offset; negative = no write).
void mla_prepare_bf16(const void* ckv, long long ldc, const void* q, long long ldq, int q_head_stride, int q_rope_offset,
                      const int* positions, const int* slots, const float* inv_freq, float attn_factor, const void* norm_w, float eps,
                      void* cache, void* q_pe, int tokens, int H, cudaStream_t s) {
  if (tokens <= 0) return;
  if ((ldc & 1) || (ldq & 1) || (q_head_stride & 1) || (q_rope_offset & 1) || (reinterpret_cast<uintptr_t>(ckv) & 3) ||
      (reinterpret_cast<uintptr_t>(q) & 3) || (reinterpret_cast<uintptr_t>(cache) & 3) || (reinterpret_cast<uintptr_t>(norm_w) & 3))
    throw std::runtime_error("mla_prepare_bf16: even strides and 4-byte aligned tensors are required");
  mla_prepare_kernel<<<tokens, 128, 0, s>>>(static_cast<const bf16*>(ckv), ldc, static_cast<const bf16*>(q), ldq, q_head_stride, q_rope_offset,
                                            positions, slots, inv_freq, attn_factor, static_cast<const bf16*>(norm_w), eps,
                                            static_cast<bf16*>(cache), static_cast<bf16*>(q_pe), H);
}

}  // namespace fllm
