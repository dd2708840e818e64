// GGUF Q5_K / Q6_K / Q8_0 weights in their planar device forms x a handful of tokens (T <= 4) on dp4a, and
// their expansion to bf16 for longer steps. The planes (ops/intk.py) hold exactly the bits of the file format:
//
//   5 (Q5_K)  low nibbles [N][K/2] (nibble j of a word = value [0 2 4 6 1 3 5 7][j]), fifth bits uint32 [N][K/32]
//             (nibble g = the four values nibble mask g of the block delivers), (scale, min) bytes [N][K/32][2],
//             (d, dmin) fp16 [N][K/256][2]:                       w = d * scale * q - dmin * min
//   6 (Q6_K)  low nibbles, two high-bit planes uint32 [N][K/32][2], int8 scales [N][K/16], d fp16 [N][K/256]:
//                                                                  w = d * scale * (q - 32)
//   8 (Q8_0)  int8 codes [N][K], d fp16 [N][K/32]:                 w = d * q
//
// Activations are quantised to int8 per 32 values inside the kernel (sums per 16 values kept for the Q6_K
// offset). A lane owns one 32-value block per step, a warp four or eight rows at a time; CTAs are persistent.
// Reference counterparts: rust/engine/cuda/qgemm5k.cu:17, qgemm6k.cu:23, qgemm8.cu, mmvq.cu:173.
#include <cuda_fp16.h>

#include <algorithm>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

constexpr int kWkThreads = 256;
constexpr int kWkMaxT = 4;
__host__ __device__ constexpr int wk_rows_per_warp(int T) { return T <= 2 ? 8 : 4; }

// bit i of a nibble -> bit 0 of byte i
__device__ __forceinline__ uint32_t spread4(uint32_t nib) { return (nib * 0x00204081u) & 0x01010101u; }

template <int T, int FMT>
__global__ void __launch_bounds__(kWkThreads)
gemv_wk_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const uint8_t* __restrict__ codes,
               const uint32_t* __restrict__ high, const uint8_t* __restrict__ sub, const __half* __restrict__ sup,
               const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, long long ldy, int N, int K) {
  extern __shared__ __align__(16) uint8_t wk_smem[];
  const int nblk = K / 32;
  int8_t* xq = reinterpret_cast<int8_t*>(wk_smem);                                // [T][K]
  float4* xs = reinterpret_cast<float4*>(wk_smem + (size_t)T * K);                // [T][K/32] {d, d*sum(first 16), d*sum(last 16), d*sum}
  pdl_launch_dependents();
  pdl_wait();
  for (int i = threadIdx.x; i < T * nblk; i += kWkThreads) {
    const int t = i / nblk, b = i - t * nblk;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * ldx + b * 32);
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 r = src[j];
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(w[e]);
        v[j * 8 + e * 2] = f.x;
        v[j * 8 + e * 2 + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
    const float d = amax / 127.f;
    const float inv = amax > 0.f ? 127.f / amax : 0.f;
    int sum_lo = 0, sum_hi = 0;
    uint32_t out[8];
#pragma unroll
    for (int g8 = 0; g8 < 4; ++g8) {
      int q[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        q[e] = __float2int_rn(v[g8 * 8 + e] * inv);
        if (g8 < 2) sum_lo += q[e]; else sum_hi += q[e];
      }
      if constexpr (FMT != 8) {          // the order the two nibble masks deliver: [0 4 1 5] and [2 6 3 7]
        out[g8 * 2] = (q[0] & 0xFF) | ((q[4] & 0xFF) << 8) | ((q[1] & 0xFF) << 16) | ((uint32_t)(q[5] & 0xFF) << 24);
        out[g8 * 2 + 1] = (q[2] & 0xFF) | ((q[6] & 0xFF) << 8) | ((q[3] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
      } else {
        out[g8 * 2] = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
        out[g8 * 2 + 1] = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(xq + (size_t)t * K + b * 32);
    dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
    dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
    xs[i] = make_float4(d, d * (float)sum_lo, d * (float)sum_hi, d * (float)(sum_lo + sum_hi));
  }
  __syncthreads();

  constexpr int R = wk_rows_per_warp(T);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kiters = (nblk + 31) / 32;
  const int n_groups = (N + R - 1) / R;
  const int warps_total = gridDim.x * (kWkThreads / 32);
  const int gwarp = blockIdx.x * (kWkThreads / 32) + warp;
  for (int grp = gwarp; grp < n_groups; grp += warps_total) {
    const int row0 = grp * R;
    float acc[R][T];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
    for (int ki = 0; ki < kiters; ++ki) {
      const int b = ki * 32 + lane;
      if (b >= nblk) continue;
      // this block's operands of every row first (independent loads), then the arithmetic
      uint4 c0[R], c1[R];
      uint32_t h0[R], h1[R], sc[R];
      float s0[R], s1[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const size_t row = (size_t)min(row0 + r, N - 1);
        h0[r] = h1[r] = 0;
        s1[r] = 0.f;
        if constexpr (FMT == 8) {
          const uint4* cp = reinterpret_cast<const uint4*>(codes + row * K + b * 32);
          c0[r] = cp[0];
          c1[r] = cp[1];
          sc[r] = 0;
          s0[r] = __half2float(sup[row * nblk + b]);
        } else if constexpr (FMT == 5) {
          c0[r] = *reinterpret_cast<const uint4*>(codes + row * (K / 2) + b * 16);
          h0[r] = high[row * nblk + b];
          sc[r] = reinterpret_cast<const uint16_t*>(sub)[row * nblk + b];
          const __half2 dd = reinterpret_cast<const __half2*>(sup)[row * (K / 256) + (b >> 3)];
          s0[r] = __low2float(dd);
          s1[r] = __high2float(dd);
        } else {
          c0[r] = *reinterpret_cast<const uint4*>(codes + row * (K / 2) + b * 16);
          const uint2 hh = reinterpret_cast<const uint2*>(high)[row * nblk + b];
          h0[r] = hh.x;
          h1[r] = hh.y;
          sc[r] = reinterpret_cast<const uint16_t*>(sub)[row * nblk + b];            // two int8 scales (values 0-15, 16-31)
          s0[r] = __half2float(sup[row * (K / 256) + (b >> 3)]);
        }
      }
      uint4 a0[T], a1[T];
      float4 sx[T];
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const uint4* ap = reinterpret_cast<const uint4*>(xq + (size_t)t * K + b * 32);
        a0[t] = ap[0];
        a1[t] = ap[1];
        sx[t] = xs[t * nblk + b];
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t cw[4] = {c0[r].x, c0[r].y, c0[r].z, c0[r].w};
        // int8 x 4 operands in the order of the activation words: q8[2j + h] for word j, nibble mask h
        uint32_t q8[8];
        if constexpr (FMT == 8) {
          q8[0] = c0[r].x; q8[1] = c0[r].y; q8[2] = c0[r].z; q8[3] = c0[r].w;
          q8[4] = c1[r].x; q8[5] = c1[r].y; q8[6] = c1[r].z; q8[7] = c1[r].w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int g = 2 * j + h;
              uint32_t q = (cw[j] >> (4 * h)) & 0x0F0F0F0Fu;
              q |= spread4((h0[r] >> (4 * g)) & 0xFu) << 4;
              if constexpr (FMT == 6) q |= spread4((h1[r] >> (4 * g)) & 0xFu) << 5;
              q8[g] = q;
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const uint32_t av[8] = {a0[t].x, a0[t].y, a0[t].z, a0[t].w, a1[t].x, a1[t].y, a1[t].z, a1[t].w};
          int i_lo = 0, i_hi = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            i_lo = __dp4a((int)q8[j], (int)av[j], i_lo);
            i_hi = __dp4a((int)q8[4 + j], (int)av[4 + j], i_hi);
          }
          if constexpr (FMT == 8) {
            acc[r][t] += s0[r] * sx[t].x * (float)(i_lo + i_hi);
          } else if constexpr (FMT == 5) {
            const float scale = (float)(sc[r] & 0xFFu), mn = (float)(sc[r] >> 8);
            acc[r][t] += s0[r] * scale * sx[t].x * (float)(i_lo + i_hi) - s1[r] * mn * sx[t].w;
          } else {
            const float sl = (float)(int)(int8_t)(sc[r] & 0xFFu), sh = (float)(int)(int8_t)(sc[r] >> 8);
            acc[r][t] += s0[r] * (sl * (sx[t].x * (float)i_lo - 32.f * sx[t].y) + sh * (sx[t].x * (float)i_hi - 32.f * sx[t].z));
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const float v = warp_sum(acc[r][t]);
        const int row = row0 + r;
        if (lane == 0 && row < N) y[(size_t)t * ldy + row] = __float2bfloat16(v + (bias ? __bfloat162float(bias[row]) : 0.f));
      }
  }
}

// Expand to bf16 [N][K]: one thread per 8 values (one word of low nibbles, or 8 int8 codes).
__global__ void wk_dequant_kernel(const uint8_t* __restrict__ codes, const uint32_t* __restrict__ high,
                                  const uint8_t* __restrict__ sub, const __half* __restrict__ sup, int fmt,
                                  __nv_bfloat16* __restrict__ out, long long n_groups8, int K) {
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n_groups8) return;
  const long long e0 = g * 8;
  const long long row = e0 / K;
  const int k = (int)(e0 - row * K);
  const int nblk = K / 32, b = k / 32, j = (k & 31) >> 3;            // block of 32, word within the block
  float v[8];
  if (fmt == 8) {
    const uint2 c = *reinterpret_cast<const uint2*>(codes + e0);
    const float d = __half2float(sup[row * nblk + b]);
    const uint32_t w[2] = {c.x, c.y};
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = d * (float)(int)(int8_t)((w[i >> 2] >> (8 * (i & 3))) & 0xFF);
  } else {
    const uint32_t cw = reinterpret_cast<const uint32_t*>(codes)[g];
    const uint32_t h0 = high[(row * nblk + b) * (fmt == 6 ? 2 : 1)];
    const uint32_t h1 = fmt == 6 ? high[(row * nblk + b) * 2 + 1] : 0u;
    int q[8];
    constexpr int order[2][4] = {{0, 4, 1, 5}, {2, 6, 3, 7}};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int grp = 2 * j + h;
      uint32_t q4 = (cw >> (4 * h)) & 0x0F0F0F0Fu;
      q4 |= spread4((h0 >> (4 * grp)) & 0xFu) << 4;
      q4 |= spread4((h1 >> (4 * grp)) & 0xFu) << 5;
#pragma unroll
      for (int i = 0; i < 4; ++i) q[order[h][i]] = (int)((q4 >> (8 * i)) & 0xFF);
    }
    if (fmt == 5) {
      const uint32_t sm = reinterpret_cast<const uint16_t*>(sub)[row * nblk + b];
      const __half2 dd = reinterpret_cast<const __half2*>(sup)[row * (K / 256) + (b >> 3)];
      const float s = __low2float(dd) * (float)(sm & 0xFF), m = __high2float(dd) * (float)(sm >> 8);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = s * (float)q[i] - m;
    } else {
      const int8_t sc = reinterpret_cast<const int8_t*>(sub)[row * (K / 16) + (k >> 4)];
      const float s = __half2float(sup[row * (K / 256) + (b >> 3)]) * (float)sc;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = s * (float)(q[i] - 32);
    }
  }
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(out + e0) = o;
}

void wk_dequant_bf16(const void* codes, const void* high, const void* sub, const void* sup, int fmt, void* out,
                     long long rows, int K, cudaStream_t s) {
  if (fmt != 5 && fmt != 6 && fmt != 8) throw std::runtime_error("wk_dequant: fmt must be 5 (Q5_K), 6 (Q6_K) or 8 (Q8_0)");
  if (K % (fmt == 8 ? 32 : 256)) throw std::runtime_error("wk_dequant: K must be a multiple of 256 (32 for Q8_0)");
  const long long groups = rows * K / 8;
  if (groups <= 0) return;
  wk_dequant_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, s>>>((const uint8_t*)codes, (const uint32_t*)high,
                                                                     (const uint8_t*)sub, (const __half*)sup, fmt,
                                                                     (__nv_bfloat16*)out, groups, K);
  cuda_check(cudaGetLastError(), "wk_dequant_kernel");
}

template <int T, int FMT>
static void launch_wk(const void* x, long long ldx, const void* codes, const void* high, const void* sub, const void* sup,
                      const void* bias, void* y, long long ldy, int N, int K, cudaStream_t s) {
  const size_t smem = (size_t)T * K + (size_t)T * (K / 32) * sizeof(float4);
  static bool configured[kMaxDevices] = {};
  if (first_call_on_device(configured))
    cuda_check(cudaFuncSetAttribute(gemv_wk_kernel<T, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024),
               "cudaFuncSetAttribute(gemv_wk_kernel)");
  int per_sm = 1;
  cuda_check(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_wk_kernel<T, FMT>, kWkThreads, smem), "gemv_wk occupancy");
  const int resident = sm_count() * std::max(per_sm, 1);
  const int rows_per_cta = (kWkThreads / 32) * wk_rows_per_warp(T);
  const int row_blocks = (N + rows_per_cta - 1) / rows_per_cta;
  const int rounds = (row_blocks + resident - 1) / resident;
  const int ctas = (row_blocks + rounds - 1) / rounds;
  launch_pdl(gemv_wk_kernel<T, FMT>, dim3(ctas), dim3(kWkThreads), smem, s, (const __nv_bfloat16*)x, ldx,
             (const uint8_t*)codes, (const uint32_t*)high, (const uint8_t*)sub, (const __half*)sup,
             (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, ldy, N, K);
}

template <int FMT>
static void launch_wk_t(int T, const void* x, long long ldx, const void* codes, const void* high, const void* sub,
                        const void* sup, const void* bias, void* y, long long ldy, int N, int K, cudaStream_t s) {
  switch (T) {
    case 1: launch_wk<1, FMT>(x, ldx, codes, high, sub, sup, bias, y, ldy, N, K, s); break;
    case 2: launch_wk<2, FMT>(x, ldx, codes, high, sub, sup, bias, y, ldy, N, K, s); break;
    case 3: launch_wk<3, FMT>(x, ldx, codes, high, sub, sup, bias, y, ldy, N, K, s); break;
    default: launch_wk<4, FMT>(x, ldx, codes, high, sub, sup, bias, y, ldy, N, K, s); break;
  }
}

bool gemv_wk_supported(int T, int K, int fmt) {
  return T >= 1 && T <= kWkMaxT && (fmt == 5 || fmt == 6 || fmt == 8) && K % (fmt == 8 ? 32 : 256) == 0 &&
         (size_t)T * K + (size_t)T * (K / 32) * 16 <= 200 * 1024;
}

// y[T][N] = x[T][K] * dequant(planes)^T (+ bias) for T <= 4.
int gemv_wk(const void* x, long long ldx, const void* codes, const void* high, const void* sub, const void* sup, int fmt,
            const void* bias, void* y, long long ldy, int T, int N, int K, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (!gemv_wk_supported(T, K, fmt)) throw std::runtime_error("gemv_wk: at most 4 tokens, fmt 5 / 6 / 8, K a multiple of 256 (32 for Q8_0)");
  if ((ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(codes) & 15))
    throw std::runtime_error("gemv_wk: activations and codes must be 16-byte aligned");
  if (fmt == 5) launch_wk_t<5>(T, x, ldx, codes, high, sub, sup, bias, y, ldy, N, K, stream);
  else if (fmt == 6) launch_wk_t<6>(T, x, ldx, codes, high, sub, sup, bias, y, ldy, N, K, stream);
  else launch_wk_t<8>(T, x, ldx, codes, high, sub, sup, bias, y, ldy, N, K, stream);
  return 1;
}

}  // namespace fllm
