// Memory-bound bf16 kernels of the decoder: embedding gather, RMSNorm with fused
// residual add, per-head QK-RMSNorm + RoPE + paged KV write, SwiGLU variants.
// All of them move 16 bytes per thread per access and keep reductions in fp32.
//
// Reference counterparts: rust/engine/cuda/elementwise.cu:271-293 (rms_norm_*),
// :470-530 (rope_kv_f16_kernel), rust/engine/cuda/fused.cu:68 (add_rms_norm_kernel),
// rust/engine/cuda/act_narrow.cu (bf16 activation pipeline). There the activation
// dtype is a run-time switch; here bf16 is the only activation dtype.
#include <cuda_fp8.h>

#include <algorithm>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

// ---------------------------------------------------------------------------- embedding
__global__ void embed_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                             __nv_bfloat16* __restrict__ out, int hidden, int vocab, float scale) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    uint4 v = src[i];
    if (scale != 1.f) {
      uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(w[j]);
        w[j] = pack_bf16x2(f.x * scale, f.y * scale);
      }
    }
    dst[i] = v;
  }
}

void embed_bf16(const int* ids, const void* table, void* out, int tokens, int hidden, int vocab,
                float scale, cudaStream_t s) {
  if (tokens <= 0) return;
  embed_kernel<<<tokens, 256, 0, s>>>(ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out,
                                      hidden, vocab, scale);
  cuda_check(cudaGetLastError(), "embed_kernel");
}

// ---------------------------------------------------------------------------- RMSNorm
// One CTA per row. y = x_new * rsqrt(mean(x_new^2) + eps) * w, where
// x_new = residual + delta when `delta` is given (and residual is updated in place).
// `w_offset` = 1 for Gemma-style (1 + w) weights.
template <int VEC_ITERS>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(__nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ delta,
               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int hidden,
               long long ld_res, long long ld_delta, long long ld_y, float eps, float w_offset) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  __nv_bfloat16* xr = residual + (size_t)row * ld_res;
  const __nv_bfloat16* dr = delta ? delta + (size_t)row * ld_delta : nullptr;
  const int nvec = hidden / 8;
  float vals[VEC_ITERS][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < VEC_ITERS; ++it) {
    const int i = threadIdx.x + it * 256;
    if (i < nvec) {
      uint4 v = reinterpret_cast<const uint4*>(xr)[i];
      const uint32_t* vw = reinterpret_cast<const uint32_t*>(&v);
      uint4 d = make_uint4(0, 0, 0, 0);
      if (dr) d = reinterpret_cast<const uint4*>(dr)[i];
      const uint32_t* dw = reinterpret_cast<const uint32_t*>(&d);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 a = unpack_bf16x2(vw[j]);
        if (dr) {
          float2 b = unpack_bf16x2(dw[j]);
          // the updated residual is stored as bf16, so normalise the rounded value
          const uint32_t packed = pack_bf16x2(a.x + b.x, a.y + b.y);
          a = unpack_bf16x2(packed);
        }
        vals[it][2 * j] = a.x;
        vals[it][2 * j + 1] = a.y;
        ss += a.x * a.x + a.y * a.y;
      }
      if (dr) {
        uint4 o;
        o.x = pack_bf16x2(vals[it][0], vals[it][1]);
        o.y = pack_bf16x2(vals[it][2], vals[it][3]);
        o.z = pack_bf16x2(vals[it][4], vals[it][5]);
        o.w = pack_bf16x2(vals[it][6], vals[it][7]);
        reinterpret_cast<uint4*>(xr)[i] = o;
      }
    }
  }
  __shared__ float red[8];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)hidden + eps);
  __nv_bfloat16* yr = y + (size_t)row * ld_y;
#pragma unroll
  for (int it = 0; it < VEC_ITERS; ++it) {
    const int i = threadIdx.x + it * 256;
    if (i < nvec) {
      const uint4 wv = reinterpret_cast<const uint4*>(w)[i];
      const uint32_t* ww = reinterpret_cast<const uint32_t*>(&wv);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 g = unpack_bf16x2(ww[j]);
        o[j] = pack_bf16x2(vals[it][2 * j] * inv * (g.x + w_offset),
                           vals[it][2 * j + 1] * inv * (g.y + w_offset));
      }
      reinterpret_cast<uint4*>(yr)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

void rmsnorm_bf16(void* residual, long long ld_res, const void* delta, long long ld_delta,
                  const void* w, void* y, long long ld_y, int rows, int hidden, float eps,
                  float w_offset, cudaStream_t s) {
  if (rows <= 0) return;
  if (hidden % 8 || hidden > 8 * 256 * 8)
    throw std::runtime_error("rmsnorm_bf16: hidden must be a multiple of 8 and at most 16384");
  const int iters = (hidden / 8 + 255) / 256;
  auto* r = (__nv_bfloat16*)residual;
  auto* d = (const __nv_bfloat16*)delta;
  auto* ww = (const __nv_bfloat16*)w;
  auto* yy = (__nv_bfloat16*)y;
#define FLLM_RMS(IT)                                                                          \
  launch_pdl(rmsnorm_kernel<IT>, dim3(rows), dim3(256), 0, s, r, d, ww, yy, hidden, ld_res, ld_delta, ld_y, eps, \
             w_offset)
  switch (iters) {
    case 1: FLLM_RMS(1); break;
    case 2: FLLM_RMS(2); break;
    case 3: FLLM_RMS(3); break;
    case 4: FLLM_RMS(4); break;
    default: FLLM_RMS(8); break;
  }
#undef FLLM_RMS
  cuda_check(cudaGetLastError(), "rmsnorm_kernel");
}

// Split-K reduction + bias + residual add + RMSNorm in one pass. The projection before the norm left
// fp32 partial sums [splits][rows][hidden]; one CTA per row with a thread per four columns keeps as many
// loads in flight as the stand-alone reduction kernel did. Rounding points are those of the two-kernel
// path (delta -> bf16, updated residual -> bf16), so both paths give the same bits.
template <int ITERS>
__global__ void __launch_bounds__(1024)
rmsnorm_splitk_kernel(__nv_bfloat16* __restrict__ residual, long long ld_res, const float* __restrict__ ws,
                      int splits, int rows, const __nv_bfloat16* __restrict__ bias,
                      const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, long long ld_y,
                      int hidden, float eps, float w_offset) {
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const int nvec = hidden / 4;
  __nv_bfloat16* xr = residual + (size_t)row * ld_res;
  // The norm weights are static: fetch them before the wait. The residual is NOT: programmatic launches
  // chain (a kernel may start while the predecessor of its predecessor still runs), so everything an
  // earlier kernel of the step wrote is read only after griddepcontrol.wait.
  uint2 xv[ITERS], wv[ITERS];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (i < nvec) wv[it] = reinterpret_cast<const uint2*>(w)[i];
  }
  pdl_wait();
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (i < nvec) xv[it] = reinterpret_cast<const uint2*>(xr)[i];
  }
  const size_t plane = (size_t)rows * hidden;
  float vals[ITERS][4];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (i < nvec) {
      const float* src = ws + (size_t)row * hidden + 4 * i;
      float4 acc = __ldcg(reinterpret_cast<const float4*>(src));
#pragma unroll 4
      for (int sp = 1; sp < splits; ++sp) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + sp * plane));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      if (bias) {
        const uint2 bb = reinterpret_cast<const uint2*>(bias)[i];
        const float2 b0 = unpack_bf16x2(bb.x), b1 = unpack_bf16x2(bb.y);
        acc.x += b0.x; acc.y += b0.y; acc.z += b1.x; acc.w += b1.y;
      }
      const float2 d0 = unpack_bf16x2(pack_bf16x2(acc.x, acc.y)), d1 = unpack_bf16x2(pack_bf16x2(acc.z, acc.w));
      const float2 x0 = unpack_bf16x2(xv[it].x), x1 = unpack_bf16x2(xv[it].y);
      uint2 o;
      o.x = pack_bf16x2(x0.x + d0.x, x0.y + d0.y);
      o.y = pack_bf16x2(x1.x + d1.x, x1.y + d1.y);
      reinterpret_cast<uint2*>(xr)[i] = o;
      const float2 n0 = unpack_bf16x2(o.x), n1 = unpack_bf16x2(o.y);
      vals[it][0] = n0.x; vals[it][1] = n0.y; vals[it][2] = n1.x; vals[it][3] = n1.y;
      ss += n0.x * n0.x + n0.y * n0.y + n1.x * n1.x + n1.y * n1.y;
    }
  }
  __shared__ float red[32];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  const int nw = blockDim.x >> 5;
  for (int i = 0; i < nw; ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)hidden + eps);
  __nv_bfloat16* yr = y + (size_t)row * ld_y;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (i < nvec) {
      const float2 g0 = unpack_bf16x2(wv[it].x), g1 = unpack_bf16x2(wv[it].y);
      uint2 o;
      o.x = pack_bf16x2(vals[it][0] * inv * (g0.x + w_offset), vals[it][1] * inv * (g0.y + w_offset));
      o.y = pack_bf16x2(vals[it][2] * inv * (g1.x + w_offset), vals[it][3] * inv * (g1.y + w_offset));
      reinterpret_cast<uint2*>(yr)[i] = o;
    }
  }
}

void rmsnorm_splitk_bf16(void* residual, long long ld_res, const float* partials, int splits, const void* bias,
                         const void* w, void* y, long long ld_y, int rows, int hidden, float eps, float w_offset,
                         cudaStream_t s) {
  if (rows <= 0) return;
  if (hidden % 4 || hidden > 16384 || (ld_res & 3) || (ld_y & 3) || splits < 1)
    throw std::runtime_error("rmsnorm_splitk_bf16: hidden must be a multiple of 4 and at most 16384");
  const int nvec = hidden / 4;
  const int threads = min(1024, (nvec + 31) / 32 * 32);
  const int iters = (nvec + threads - 1) / threads;
  auto* r = (__nv_bfloat16*)residual;
  auto* b = (const __nv_bfloat16*)bias;
  auto* ww = (const __nv_bfloat16*)w;
  auto* yy = (__nv_bfloat16*)y;
#define FLLM_RMS_SK(IT)                                                                                       \
  launch_pdl(rmsnorm_splitk_kernel<IT>, dim3(rows), dim3(threads), 0, s, r, ld_res, partials, splits, rows, b, ww, yy, \
             ld_y, hidden, eps, w_offset)
  switch (iters) {
    case 1: FLLM_RMS_SK(1); break;
    case 2: FLLM_RMS_SK(2); break;
    case 3: FLLM_RMS_SK(3); break;
    default: FLLM_RMS_SK(4); break;
  }
#undef FLLM_RMS_SK
  cuda_check(cudaGetLastError(), "rmsnorm_splitk_kernel");
}

// ---------------------------------------------------------------------------- RoPE + QK-norm + KV write
// One warp per (token, head). Heads [0, hq) are query heads (rotated in place),
// [hq, hq+hkv) key heads (normalised, rotated, written to the paged cache),
// [hq+hkv, hq+2hkv) value heads (copied to the cache).
// Cache layout: [block][kv_head][block_size][head_dim] (a head's page is contiguous).
// rope_style: 0 = rotate-half ("neox": pairs (i, i + rot/2)), 1 = interleaved pairs (2i, 2i+1).
template <int D>
__global__ void __launch_bounds__(128)
rope_kv_kernel(__nv_bfloat16* __restrict__ qkv, long long ld_qkv, const int* __restrict__ positions,
               const int* __restrict__ slots, const float* __restrict__ inv_freq,
               const __nv_bfloat16* __restrict__ q_norm_w, const __nv_bfloat16* __restrict__ k_norm_w,
               __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int tokens,
               int hq, int hkv, int block_size, int rot_dim, int rope_style, float eps,
               float attn_factor, int kv_fp8, const float* __restrict__ ws, int splits,
               const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ q_out, long long ld_q) {
  // ws != null: the projection left fp32 split-K partials [splits][tokens][heads * D] (bias not added);
  // this kernel adds them, rounds to bf16 like the reduction kernel would, and writes the rotated query
  // heads to q_out (the key / value heads only go to the cache).
  constexpr int EPL = D / 32;  // elements per lane
  pdl_launch_dependents();
  pdl_wait();
  const int heads = hq + 2 * hkv;
  const long long gw = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (gw >= (long long)tokens * heads) return;
  const int t = (int)(gw / heads);
  const int h = (int)(gw - (long long)t * heads);
  const int lane = threadIdx.x & 31;
  __nv_bfloat16* src = qkv ? qkv + (size_t)t * ld_qkv + (size_t)h * D : nullptr;
  const int slot = slots ? slots[t] : -1;
  const size_t width = (size_t)heads * D;
  const size_t plane = (size_t)tokens * width;
  const float* wsrc = ws ? ws + (size_t)t * width + (size_t)h * D : nullptr;
  // element e of this head as the bf16 value the unfused path would have stored
  auto ld_elem = [&](int e) -> float {
    if (!ws) return __bfloat162float(src[e]);
    float a = __ldcg(wsrc + e);
    for (int sp = 1; sp < splits; ++sp) a += __ldcg(wsrc + sp * plane + e);
    if (bias) a += __bfloat162float(bias[h * D + e]);
    return __bfloat162float(__float2bfloat16(a));
  };

  if (h >= hq + hkv) {  // value head: straight copy
    if (slot < 0) return;
    const int kvh = h - hq - hkv;
    const int blk = slot / block_size, off = slot - blk * block_size;
    __nv_bfloat16* dst = v_cache + (((size_t)blk * hkv + kvh) * block_size + off) * D;
    if (kv_fp8) {                  // e4m3 cache: one byte per value, same [block][head][slot][dim] order
      uint8_t* d8 = reinterpret_cast<uint8_t*>(v_cache) + (((size_t)blk * hkv + kvh) * block_size + off) * D;
      for (int i = lane; i < D / 2; i += 32) {
        const float2 f = ws ? make_float2(ld_elem(2 * i), ld_elem(2 * i + 1))
                            : unpack_bf16x2(reinterpret_cast<const uint32_t*>(src)[i]);
        reinterpret_cast<uint16_t*>(d8)[i] = (uint16_t)__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
      }
      return;
    }
    if (ws) {
      float a[EPL];            // pairs (2i, 2i+1), i = lane + 32 * (j / 2): every load of a split is independent
#pragma unroll
      for (int j = 0; j < EPL; ++j) a[j] = __ldcg(wsrc + 2 * (lane + 32 * (j / 2)) + (j & 1));
#pragma unroll 4
      for (int sp = 1; sp < splits; ++sp) {
#pragma unroll
        for (int j = 0; j < EPL; ++j) a[j] += __ldcg(wsrc + sp * plane + 2 * (lane + 32 * (j / 2)) + (j & 1));
      }
#pragma unroll
      for (int j = 0; j < EPL; j += 2) {
        const int e = 2 * (lane + 32 * (j / 2));
        if (bias) { a[j] += __bfloat162float(bias[h * D + e]); a[j + 1] += __bfloat162float(bias[h * D + e + 1]); }
        reinterpret_cast<uint32_t*>(dst)[lane + 32 * (j / 2)] = pack_bf16x2(a[j], a[j + 1]);
      }
      return;
    }
    if (EPL == 4) {
      reinterpret_cast<uint2*>(dst)[lane] = reinterpret_cast<const uint2*>(src)[lane];
    } else {
      for (int i = lane; i < D / 2; i += 32)
        reinterpret_cast<uint32_t*>(dst)[i] = reinterpret_cast<const uint32_t*>(src)[i];
    }
    return;
  }

  // Load the head with lanes striding so that lane l owns elements {l + 32*j}: the
  // rotate-half partner of element i (i + rot/2) then sits in the same lane whenever
  // rot/2 is a multiple of 32, and in lane l for the interleaved style we use pairs.
  float v[EPL];
  int eidx[EPL];               // element index of v[j] within the head
#pragma unroll
  for (int j = 0; j < EPL; ++j)
    eidx[j] = rope_style == 0 ? lane + 32 * j : 2 * (lane + 32 * (j / 2)) + (j & 1);
  if (ws) {
    // all EPL loads of a split are independent; four splits are in flight at a time
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = __ldcg(wsrc + eidx[j]);
#pragma unroll 4
    for (int sp = 1; sp < splits; ++sp) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) v[j] += __ldcg(wsrc + sp * plane + eidx[j]);
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      if (bias) v[j] += __bfloat162float(bias[h * D + eidx[j]]);
      v[j] = __bfloat162float(__float2bfloat16(v[j]));
    }
  } else if (rope_style == 0) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = __bfloat162float(src[lane + 32 * j]);
  } else {
#pragma unroll
    for (int j = 0; j < EPL; j += 2) {
      float2 f = unpack_bf16x2(reinterpret_cast<const uint32_t*>(src)[lane + 32 * (j / 2)]);
      v[j] = f.x;
      v[j + 1] = f.y;
    }
  }
  const bool is_q = h < hq;
  const __nv_bfloat16* nw = is_q ? q_norm_w : k_norm_w;
  if (nw) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) ss += v[j] * v[j];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)D + eps);
    if (rope_style == 0) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        // round through bf16 like an unfused norm would
        v[j] = __bfloat162float(__float2bfloat16(v[j] * inv * __bfloat162float(nw[lane + 32 * j])));
      }
    } else {
#pragma unroll
      for (int j = 0; j < EPL; j += 2) {
        const int e = 2 * (lane + 32 * (j / 2));
        v[j] = __bfloat162float(__float2bfloat16(v[j] * inv * __bfloat162float(nw[e])));
        v[j + 1] = __bfloat162float(__float2bfloat16(v[j + 1] * inv * __bfloat162float(nw[e + 1])));
      }
    }
  }
  const float pos = (float)positions[t];
  const int half = rot_dim / 2;
  if (rope_style == 0) {
    // element index e = lane + 32*j ; partner e + half when e < half
    if (half % 32 == 0) {
      const int jh = half / 32;
#pragma unroll
      for (int j = 0; j < EPL / 2; ++j) {
        if (j < jh) {
          const int e = lane + 32 * j;
          float sn, cs;
          sincosf(pos * inv_freq[e], &sn, &cs);
          sn *= attn_factor;
          cs *= attn_factor;
          const float a = v[j], b = v[j + jh];
          v[j] = a * cs - b * sn;
          v[j + jh] = b * cs + a * sn;
        }
      }
    } else {
      // partner lives in another lane (half = 16, head_dim 32 or partial rotary): shuffle
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const int e = lane + 32 * j;
        const int pe = e < half ? e + half : e - half;
        const float other = __shfl_sync(0xffffffffu, v[j], pe & 31);  // same j only when half<32
        if (e < rot_dim && half < 32) {
          float sn, cs;
          sincosf(pos * inv_freq[e < half ? e : e - half], &sn, &cs);
          sn *= attn_factor;
          cs *= attn_factor;
          v[j] = e < half ? v[j] * cs - other * sn : v[j] * cs + other * sn;
        }
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < EPL; j += 2) {
      const int pair = lane + 32 * (j / 2);
      if (2 * pair < rot_dim) {
        float sn, cs;
        sincosf(pos * inv_freq[pair], &sn, &cs);
        sn *= attn_factor;
        cs *= attn_factor;
        const float a = v[j], b = v[j + 1];
        v[j] = a * cs - b * sn;
        v[j + 1] = b * cs + a * sn;
      }
    }
  }
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out ? q_out + (size_t)t * ld_q + (size_t)h * D : src;
  } else {
    if (slot < 0) return;
    const int kvh = h - hq;
    const int blk = slot / block_size, off = slot - blk * block_size;
    dst = k_cache + (((size_t)blk * hkv + kvh) * block_size + off) * D;
    if (kv_fp8) {
      uint8_t* d8 = reinterpret_cast<uint8_t*>(k_cache) + (((size_t)blk * hkv + kvh) * block_size + off) * D;
      if (rope_style == 0) {
#pragma unroll
        for (int j = 0; j < EPL; ++j) d8[lane + 32 * j] = (uint8_t)__nv_cvt_float_to_fp8(v[j], __NV_SATFINITE, __NV_E4M3);
      } else {
#pragma unroll
        for (int j = 0; j < EPL; j += 2)
          reinterpret_cast<uint16_t*>(d8)[lane + 32 * (j / 2)] =
              (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(v[j], v[j + 1]), __NV_SATFINITE, __NV_E4M3);
      }
      return;
    }
  }
  if (rope_style == 0) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) dst[lane + 32 * j] = __float2bfloat16(v[j]);
  } else {
#pragma unroll
    for (int j = 0; j < EPL; j += 2)
      reinterpret_cast<uint32_t*>(dst)[lane + 32 * (j / 2)] = pack_bf16x2(v[j], v[j + 1]);
  }
}

void rope_qknorm_kvwrite_bf16(void* qkv, long long ld_qkv, const int* positions, const int* slots,
                              const float* inv_freq, const void* q_norm_w, const void* k_norm_w,
                              void* k_cache, void* v_cache, int tokens, int hq, int hkv,
                              int head_dim, int block_size, int rot_dim, int rope_style, float eps,
                              float attn_factor, cudaStream_t s, int kv_fp8, const float* partials, int splits,
                              const void* bias, void* q_out, long long ld_q) {
  if (tokens <= 0) return;
  if (!qkv && !(partials && q_out)) throw std::runtime_error("rope_qknorm_kvwrite_bf16: no source");
  const long long warps = (long long)tokens * (hq + 2 * hkv);
  const int blocks = (int)((warps + 3) / 4);
  auto* x = (__nv_bfloat16*)qkv;
  auto* qn = (const __nv_bfloat16*)q_norm_w;
  auto* kn = (const __nv_bfloat16*)k_norm_w;
  auto* kc = (__nv_bfloat16*)k_cache;
  auto* vc = (__nv_bfloat16*)v_cache;
#define FLLM_ROPE(DD)                                                                            \
  launch_pdl(rope_kv_kernel<DD>, dim3(blocks), dim3(128), 0, s, x, ld_qkv, positions, slots, inv_freq, qn, kn, kc, \
             vc, tokens, hq, hkv, block_size, rot_dim, rope_style, eps, attn_factor, kv_fp8, partials, splits,    \
             (const __nv_bfloat16*)bias, (__nv_bfloat16*)q_out, ld_q)
  switch (head_dim) {
    case 64: FLLM_ROPE(64); break;
    case 128: FLLM_ROPE(128); break;
    case 256: FLLM_ROPE(256); break;
    default: throw std::runtime_error("rope_qknorm_kvwrite_bf16: head_dim must be 64, 128 or 256");
  }
#undef FLLM_ROPE
  cuda_check(cudaGetLastError(), "rope_kv_kernel");
}

// ---------------------------------------------------------------------------- GLU activations
// act_kind 0: silu(gate) * up with gate = x[:, :I], up = x[:, I:2I]
// act_kind 1: gelu_tanh(gate) * up (GeGLU)
// act_kind 2: gpt-oss clamped SwiGLU on interleaved columns (gate = x[2i], up = x[2i+1]):
//             g = min(g, limit); u = clamp(u, -limit, limit); out = g * sigmoid(alpha g) * (u + 1)
// layout: 0 = the kind's natural one (halves; pairs for kind 2), 16 = blocks of 16 gate columns followed
// by the 16 up columns of the same features (the order the GEMM's gated epilogue wants its weight rows in).
// ws != null: x is not read; the columns are the sums of fp32 split-K partials [splits][rows][2 * inter]
// (+ bias), rounded to bf16 like the reduction kernel would have stored them.
__global__ void glu_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                           __nv_bfloat16* __restrict__ out, long long ldo, int inter, int act_kind,
                           float alpha, float limit, int layout, const float* __restrict__ ws, int splits,
                           int rows, const __nv_bfloat16* __restrict__ bias) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y;
  const int i8 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i8 >= inter) return;
  const __nv_bfloat16* xr = x ? x + (size_t)row * ldx : nullptr;
  float g[8], u[8];
  if (ws || layout == 16) {
    // column of gate / up value j of this thread's 8 features
    auto col = [&](int j, bool up) -> int {
      const int f = i8 + j;
      if (layout == 16) return 32 * (f >> 4) + (f & 15) + (up ? 16 : 0);
      if (act_kind == 2) return 2 * f + (up ? 1 : 0);
      return f + (up ? inter : 0);
    };
    int cg[8], cu[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { cg[j] = col(j, false); cu[j] = col(j, true); }
    if (!ws) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { g[j] = __bfloat162float(xr[cg[j]]); u[j] = __bfloat162float(xr[cu[j]]); }
    } else {
      const size_t plane = (size_t)rows * 2 * inter;
      const float* src = ws + (size_t)row * 2 * inter;
#pragma unroll
      for (int j = 0; j < 8; ++j) { g[j] = __ldcg(src + cg[j]); u[j] = __ldcg(src + cu[j]); }
#pragma unroll 2
      for (int sp = 1; sp < splits; ++sp) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { g[j] += __ldcg(src + sp * plane + cg[j]); u[j] += __ldcg(src + sp * plane + cu[j]); }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (bias) { g[j] += __bfloat162float(bias[cg[j]]); u[j] += __bfloat162float(bias[cu[j]]); }
        g[j] = __bfloat162float(__float2bfloat16(g[j]));
        u[j] = __bfloat162float(__float2bfloat16(u[j]));
      }
    }
  } else if (act_kind == 2) {
    const uint4 a = *reinterpret_cast<const uint4*>(xr + 2 * i8);
    const uint4 b = *reinterpret_cast<const uint4*>(xr + 2 * i8 + 8);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float2 f = unpack_bf16x2(w[j]);
      g[j] = f.x;
      u[j] = f.y;
    }
  } else {
    const uint4 a = *reinterpret_cast<const uint4*>(xr + i8);
    const uint4 b = *reinterpret_cast<const uint4*>(xr + inter + i8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
    const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16x2(aw[j]);
      float2 h = unpack_bf16x2(bw[j]);
      g[2 * j] = f.x; g[2 * j + 1] = f.y;
      u[2 * j] = h.x; u[2 * j + 1] = h.y;
    }
  }
  float o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (act_kind == 0) {
      o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    } else if (act_kind == 1) {
      const float c = 0.7978845608028654f * (g[j] + 0.044715f * g[j] * g[j] * g[j]);
      o[j] = 0.5f * g[j] * (1.f + tanhf(c)) * u[j];
    } else {
      const float gg = fminf(g[j], limit);
      const float uu = fminf(fmaxf(u[j], -limit), limit);
      o[j] = gg / (1.f + __expf(-alpha * gg)) * (uu + 1.f);
    }
  }
  uint4 r;
  r.x = pack_bf16x2(o[0], o[1]);
  r.y = pack_bf16x2(o[2], o[3]);
  r.z = pack_bf16x2(o[4], o[5]);
  r.w = pack_bf16x2(o[6], o[7]);
  *reinterpret_cast<uint4*>(out + (size_t)row * ldo + i8) = r;
}

void glu_bf16(const void* x, long long ldx, void* out, long long ldo, int rows, int inter,
              int act_kind, float alpha, float limit, cudaStream_t s, int layout, const float* partials, int splits,
              const void* bias) {
  if (rows <= 0) return;
  if (inter % 8) throw std::runtime_error("glu_bf16: intermediate size must be a multiple of 8");
  if (layout == 16 && inter % 16) throw std::runtime_error("glu_bf16: the blocked layout needs a multiple of 16 features");
  dim3 grid((inter / 8 + 127) / 128, rows);
  launch_pdl(glu_kernel, grid, dim3(128), 0, s, (const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)out, ldo, inter,
             act_kind, alpha, limit, layout, partials, splits, rows, (const __nv_bfloat16*)bias);
  cuda_check(cudaGetLastError(), "glu_kernel");
}

// ---------------------------------------------------------------------------- row gather (logit rows)
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                   const int* __restrict__ rows, __nv_bfloat16* __restrict__ out,
                                   int hidden) {
  const int r = rows[blockIdx.x];
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)r * ldx);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

void gather_rows_bf16(const void* x, long long ldx, const int* rows, void* out, int n_rows,
                      int hidden, cudaStream_t s) {
  if (n_rows <= 0) return;
  gather_rows_kernel<<<n_rows, 128, 0, s>>>((const __nv_bfloat16*)x, ldx, rows,
                                            (__nv_bfloat16*)out, hidden);
  cuda_check(cudaGetLastError(), "gather_rows_kernel");
}

// ---- logit soft-cap: x = cap * tanh(x / cap), in place over bf16 rows (Gemma-2 final logits; the reference keeps it with
// its small architecture ops in rust/engine/cuda/arch_ops.cu) -------------------------------------------------------
__global__ void softcap_rows_kernel(__nv_bfloat16* __restrict__ x, long long ldx, int cols, float cap, float inv_cap) {
  __nv_bfloat16* row = x + (size_t)blockIdx.y * ldx;
  for (int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2; c < cols; c += gridDim.x * blockDim.x * 2) {
    if (c + 1 < cols) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + c));
      *reinterpret_cast<__nv_bfloat162*>(row + c) = __floats2bfloat162_rn(cap * tanhf(v.x * inv_cap), cap * tanhf(v.y * inv_cap));
    } else {
      row[c] = __float2bfloat16(cap * tanhf(__bfloat162float(row[c]) * inv_cap));
    }
  }
}

void softcap_rows_bf16(void* x, long long ldx, int rows, int cols, float cap, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return;
  if ((ldx & 1) || (reinterpret_cast<uintptr_t>(x) & 3)) throw std::runtime_error("softcap_rows_bf16: even leading dimension, 4-byte aligned rows");
  const int bx = std::min((cols / 2 + 255) / 256, 64);
  softcap_rows_kernel<<<dim3(std::max(bx, 1), rows), 256, 0, s>>>((__nv_bfloat16*)x, ldx, cols, cap, 1.f / cap);
  cuda_check(cudaGetLastError(), "softcap_rows_kernel");
}

// ---- LayerNorm with the residual update in front (GPT-NeoX / Phi / StarCoder2 / Cohere / Nemotron blocks): x += delta (in place, when
// delta is given), y = (x - mean) * rstd * (w + w_offset) + b. One CTA per row, the row kept in registers between the passes
// (up to 16384 columns), two-pass variance. -----------------------------------------------------------------------------
__global__ void __launch_bounds__(256) add_layernorm_kernel(__nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ delta,
                                                            long long ldd, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                                                            __nv_bfloat16* __restrict__ y, long long ldy, int cols, float eps, float w_offset) {
  constexpr int KEEP = 32;                                  // pairs per thread: 256 * 32 * 2 columns
  const int row = blockIdx.x, pairs = cols / 2;
  __nv_bfloat162* xr = reinterpret_cast<__nv_bfloat162*>(x + (size_t)row * ldx);
  const __nv_bfloat162* dr = delta ? reinterpret_cast<const __nv_bfloat162*>(delta + (size_t)row * ldd) : nullptr;
  float2 v[KEEP];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int p = threadIdx.x + i * 256;
    v[i] = make_float2(0.f, 0.f);
    if (p < pairs) {
      v[i] = __bfloat1622float2(xr[p]);
      if (dr) {
        const float2 d = __bfloat1622float2(dr[p]);
        const __nv_bfloat162 r = __floats2bfloat162_rn(v[i].x + d.x, v[i].y + d.y);     // the stored residual is what gets normalised
        xr[p] = r;
        v[i] = __bfloat1622float2(r);
      }
      sum += v[i].x + v[i].y;
    }
  }
  __shared__ float part[8];
  __shared__ float stat[2];
  sum = warp_sum(sum);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += part[i];
    stat[0] = t / cols;
  }
  __syncthreads();
  const float mean = stat[0];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int p = threadIdx.x + i * 256;
    if (p < pairs) sq += (v[i].x - mean) * (v[i].x - mean) + (v[i].y - mean) * (v[i].y - mean);
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += part[i];
    stat[1] = rsqrtf(t / cols + eps);
  }
  __syncthreads();
  const float rstd = stat[1];
  __nv_bfloat162* yr = reinterpret_cast<__nv_bfloat162*>(y + (size_t)row * ldy);
  const __nv_bfloat162* wr = reinterpret_cast<const __nv_bfloat162*>(w);
  const __nv_bfloat162* br = b ? reinterpret_cast<const __nv_bfloat162*>(b) : nullptr;
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int p = threadIdx.x + i * 256;
    if (p < pairs) {
      const float2 ww = __bfloat1622float2(wr[p]);
      const float2 bb = br ? __bfloat1622float2(br[p]) : make_float2(0.f, 0.f);
      yr[p] = __floats2bfloat162_rn((v[i].x - mean) * rstd * (ww.x + w_offset) + bb.x, (v[i].y - mean) * rstd * (ww.y + w_offset) + bb.y);
    }
  }
}

void add_layernorm_bf16(void* x, long long ldx, const void* delta, long long ldd, const void* w, const void* b, void* y, long long ldy,
                        int rows, int cols, float eps, float w_offset, cudaStream_t s) {
  if (rows <= 0) return;
  if ((cols & 1) || cols > 16384 || (ldx & 1) || (ldd & 1) || (ldy & 1))
    throw std::runtime_error("add_layernorm_bf16: an even width of at most 16384 and even leading dimensions are required");
  add_layernorm_kernel<<<rows, 256, 0, s>>>((__nv_bfloat16*)x, ldx, (const __nv_bfloat16*)delta, ldd, (const __nv_bfloat16*)w,
                                            (const __nv_bfloat16*)b, (__nv_bfloat16*)y, ldy, cols, eps, w_offset);
  cuda_check(cudaGetLastError(), "add_layernorm_kernel");
}

// ---- activation of a plain MLP, in place over bf16 rows: 0 gelu (erf), 1 gelu (tanh), 2 squared relu, 3 silu, 4 relu -------------
__global__ void act_rows_kernel(__nv_bfloat16* __restrict__ x, long long ldx, int cols, int kind) {
  __nv_bfloat16* row = x + (size_t)blockIdx.y * ldx;
  for (int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2; c < cols; c += gridDim.x * blockDim.x * 2) {
    float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + c));
    float* f = &v.x;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float t = f[i];
      float r;
      if (kind == 0) r = 0.5f * t * (1.f + erff(t * 0.70710678118654752f));
      else if (kind == 1) r = 0.5f * t * (1.f + tanhf(0.7978845608028654f * (t + 0.044715f * t * t * t)));
      else if (kind == 2) r = t > 0.f ? t * t : 0.f;
      else if (kind == 3) r = t / (1.f + __expf(-t));
      else r = fmaxf(t, 0.f);
      f[i] = r;
    }
    *reinterpret_cast<__nv_bfloat162*>(row + c) = __floats2bfloat162_rn(v.x, v.y);
  }
}

void act_rows_bf16(void* x, long long ldx, int rows, int cols, int kind, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return;
  if ((cols & 1) || (ldx & 1) || (reinterpret_cast<uintptr_t>(x) & 3) || kind < 0 || kind > 4)
    throw std::runtime_error("act_rows_bf16: an even width and leading dimension, 4-byte aligned rows, kind 0..4");
  const int bx = std::max(1, std::min((cols / 2 + 255) / 256, 64));
  act_rows_kernel<<<dim3(bx, rows), 256, 0, s>>>((__nv_bfloat16*)x, ldx, cols, kind);
  cuda_check(cudaGetLastError(), "act_rows_kernel");
}

}  // namespace fllm
