// Packed 4-bit weights x a handful of tokens (T <= 4): integer dot products on the CUDA cores.
//
// A single-stream decode step multiplies every weight by one token. Tensor-core tiles are empty at that
// shape (one useful column of 16), so the packed tcgen05 GEMM of gemm_w4a16.cu spends its time expanding
// codes nobody multiplies. Here the weights stay 4-bit all the way into the arithmetic: the activations are
// quantised to int8 (one fp32 scale per 32 values, in shared memory, by every CTA for itself), a lane loads
// 16 bytes = one 32-value block of codes, splits the nibbles with two masks and feeds them to dp4a; the
// block's integer sum is scaled once. The kernel is bound by the bytes of weight it reads.
//
// Formats (the device forms of gemm_w4a16.cu):
//   2 INT4G  unsigned codes, nibble j of a word holds value [0 2 4 6 1 3 5 7][j], {bf16 scale, bf16 min} per 32:
//            y += s * dx * sum(q * qx) - m * dx * sum(qx)          (GGUF Q4_K / Q4_0 / Q4_1, AWQ / GPTQ)
//   1 MXFP4  e2m1 codes in index order + e8m0 scale per 32; 0 NVFP4: + e4m3 scale per 16 and a tensor scale.
//            e2m1 magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6} are doubled into int8 by a byte-permute table.
//
// One warp owns eight (one or two tokens) or four output rows at a time (as many independent 16-byte loads per lane,
// and the next group's already in flight); CTAs are persistent (at most three per SM), so the activations are quantised once per CTA.
// Reference counterparts: rust/engine/cuda/mmvq.cu:50,173,375 (dp4a GEMV on q8_1 activations),
// rust/engine/cuda/gemv2.cu.
#include <cuda_fp8.h>

#include <algorithm>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

constexpr int kGvThreads = 256;
constexpr int kGvMaxT = 4;
// rows a warp multiplies at a time: its loads in flight per item. One or two tokens leave registers for eight.
__host__ __device__ constexpr int gv_rows_per_warp(int T) { return T <= 2 ? 8 : 4; }

__device__ __forceinline__ uint32_t gv_prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

// four e2m1 codes (16 bits, index order) -> four int8 of twice their value
__device__ __forceinline__ uint32_t e2m1x4_to_s8(uint32_t h) {
  constexpr uint32_t P_LO = 0x03020100u, P_HI = 0x0C080604u;       //  0  1  2  3 |  4  6  8  12
  constexpr uint32_t N_LO = 0xFDFEFF00u, N_HI = 0xF4F8FAFCu;       // -0 -1 -2 -3 | -4 -6 -8 -12
  const uint32_t sel = h & 0x7777u;
  const uint32_t pos = gv_prmt(P_LO, P_HI, sel);
  const uint32_t neg = gv_prmt(N_LO, N_HI, sel);
  const uint32_t sg = gv_prmt(h, h << 4, 0x9D8Cu);                  // byte i = 0xFF where code i has its sign bit set
  return (pos & ~sg) | (neg & sg);
}

template <int T, int FMT>
__global__ void __launch_bounds__(kGvThreads)
gemv_w4_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const uint8_t* __restrict__ codes,
               const uint8_t* __restrict__ scales, float alpha, const __nv_bfloat16* __restrict__ bias,
               __nv_bfloat16* __restrict__ y, long long ldy, int N, int K) {
  extern __shared__ __align__(16) uint8_t gv_smem[];
  const int nblk = K / 32;
  int8_t* xq = reinterpret_cast<int8_t*>(gv_smem);                               // [T][K]
  float2* xs = reinterpret_cast<float2*>(gv_smem + (size_t)T * K);               // [T][K/32] {d, d * sum(q)}
  pdl_launch_dependents();
  pdl_wait();
  // ---- quantise the activations: one thread per 32-value block
  for (int i = threadIdx.x; i < T * nblk; i += kGvThreads) {
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
    int sum = 0;
    uint32_t out[8];
#pragma unroll
    for (int g8 = 0; g8 < 4; ++g8) {                                              // groups of 8 values = 2 words
      int q[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        q[e] = __float2int_rn(v[g8 * 8 + e] * inv);
        sum += q[e];
      }
      if constexpr (FMT == 2) {          // the order the two nibble masks deliver: [0 4 1 5] and [2 6 3 7]
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
    xs[i] = make_float2(d, d * (float)sum);
  }
  __syncthreads();

  constexpr int kGvRowsPerWarp = gv_rows_per_warp(T);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Persistent CTAs: the activations are quantised once per CTA, then every warp walks (row group, K slice)
  // items with the next item's codes already in flight while the current one is multiplied.
  const int kiters = (nblk + 31) / 32;                                 // K slices of 32 blocks per row group
  const int n_groups = (N + kGvRowsPerWarp - 1) / kGvRowsPerWarp;      // row groups of kGvRowsPerWarp rows
  const int warps_total = gridDim.x * (kGvThreads / 32);
  const int gwarp = blockIdx.x * (kGvThreads / 32) + warp;
  const long long items = (long long)((n_groups - gwarp + warps_total - 1) / warps_total) * kiters;   // this warp's items
  if (gwarp >= n_groups) return;

  auto item_row0 = [&](long long it) { return (int)((gwarp + (it / kiters) * warps_total) * kGvRowsPerWarp); };
  auto load_item = [&](long long it, uint4 (&w)[kGvRowsPerWarp], uint32_t (&sc)[kGvRowsPerWarp]) {
    const int row0 = item_row0(it);
    const int b = (int)(it % kiters) * 32 + lane;
#pragma unroll
    for (int r = 0; r < kGvRowsPerWarp; ++r) {
      const int row = min(row0 + r, N - 1);
      w[r] = make_uint4(0, 0, 0, 0);
      sc[r] = 0;
      if (b < nblk) {
        w[r] = *reinterpret_cast<const uint4*>(codes + (size_t)row * (K / 2) + b * 16);
        if constexpr (FMT == 2) sc[r] = reinterpret_cast<const uint32_t*>(scales)[(size_t)row * nblk + b];
        else if constexpr (FMT == 1) sc[r] = scales[(size_t)row * nblk + b];
        else sc[r] = reinterpret_cast<const uint16_t*>(scales)[(size_t)row * nblk + b];
      }
    }
  };

  float acc[kGvRowsPerWarp][T];
#pragma unroll
  for (int r = 0; r < kGvRowsPerWarp; ++r)
#pragma unroll
    for (int t = 0; t < T; ++t) acc[r][t] = 0.f;

  uint4 w[kGvRowsPerWarp], wn[kGvRowsPerWarp];
  uint32_t sc[kGvRowsPerWarp], scn[kGvRowsPerWarp];
  load_item(0, w, sc);
  for (long long it = 0; it < items; ++it) {
    if (it + 1 < items) load_item(it + 1, wn, scn);
    const int row0 = item_row0(it);
    const int b = (int)(it % kiters) * 32 + lane;
    if (b < nblk) {
      uint4 a0[T], a1[T];
      float2 sx[T];
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const uint4* ap = reinterpret_cast<const uint4*>(xq + (size_t)t * K + b * 32);
        a0[t] = ap[0];
        a1[t] = ap[1];
        sx[t] = xs[t * nblk + b];
      }
#pragma unroll
      for (int r = 0; r < kGvRowsPerWarp; ++r) {
        const uint32_t cw[4] = {w[r].x, w[r].y, w[r].z, w[r].w};
        if constexpr (FMT == 2) {
          const float2 smf = unpack_bf16x2(sc[r]);                                  // {scale, min}
#pragma unroll
          for (int t = 0; t < T; ++t) {
            const uint32_t av[8] = {a0[t].x, a0[t].y, a0[t].z, a0[t].w, a1[t].x, a1[t].y, a1[t].z, a1[t].w};
            int isum = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              isum = __dp4a((int)(cw[j] & 0x0F0F0F0Fu), (int)av[2 * j], isum);
              isum = __dp4a((int)((cw[j] >> 4) & 0x0F0F0F0Fu), (int)av[2 * j + 1], isum);
            }
            acc[r][t] += smf.x * (sx[t].x * (float)isum) - smf.y * sx[t].y;
          }
        } else {
          // index order: the low half-word of a code word holds values 0..3, the high half-word 4..7
          uint32_t q8[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            q8[2 * j] = e2m1x4_to_s8(cw[j] & 0xFFFFu);
            q8[2 * j + 1] = e2m1x4_to_s8(cw[j] >> 16);
          }
          float s_lo, s_hi;                                                          // scales of values 0..15 and 16..31, halved (codes were doubled)
          if constexpr (FMT == 1) {
            const uint32_t e = sc[r];
            s_lo = s_hi = e ? __uint_as_float(e << 23) * 0.5f : 0.f;
          } else {
            const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)sc[r], __NV_E4M3);
            const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&h2));
            s_lo = f2.x * 0.5f;
            s_hi = f2.y * 0.5f;
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
            acc[r][t] += sx[t].x * (s_lo * (float)i_lo + s_hi * (float)i_hi);
          }
        }
      }
    }
    if ((it + 1) % kiters == 0) {                                      // last K slice of this row group: reduce and store
#pragma unroll
      for (int r = 0; r < kGvRowsPerWarp; ++r)
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const float v = warp_sum(acc[r][t]);
          const int row = row0 + r;
          if (lane == 0 && row < N)
            y[(size_t)t * ldy + row] = __float2bfloat16(v * alpha + (bias ? __bfloat162float(bias[row]) : 0.f));
          acc[r][t] = 0.f;
        }
    }
#pragma unroll
    for (int r = 0; r < kGvRowsPerWarp; ++r) {
      w[r] = wn[r];
      sc[r] = scn[r];
    }
  }
}

template <int T, int FMT>
static void launch_gemv(const void* x, long long ldx, const void* codes, const void* scales, float alpha, const void* bias,
                        void* y, long long ldy, int N, int K, cudaStream_t s) {
  const size_t smem = (size_t)T * K + (size_t)T * (K / 32) * sizeof(float2);
  static bool configured[kMaxDevices] = {};
  if (first_call_on_device(configured))
    cuda_check(cudaFuncSetAttribute(gemv_w4_kernel<T, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024),
               "cudaFuncSetAttribute(gemv_w4_kernel)");
  int per_sm = 1;
  cuda_check(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_w4_kernel<T, FMT>, kGvThreads, smem), "gemv_w4 occupancy");
  const int resident = sm_count() * std::max(per_sm, 1);
  // equal work per CTA: as many rounds of row blocks as the resident CTAs need, then the fewest CTAs for that many rounds
  const int rows_per_cta = (kGvThreads / 32) * gv_rows_per_warp(T);
  const int row_blocks = (N + rows_per_cta - 1) / rows_per_cta;
  const int rounds = (row_blocks + resident - 1) / resident;
  const int ctas = (row_blocks + rounds - 1) / rounds;
  launch_pdl(gemv_w4_kernel<T, FMT>, dim3(ctas), dim3(kGvThreads), smem, s,
             (const __nv_bfloat16*)x, ldx, (const uint8_t*)codes, (const uint8_t*)scales, alpha, (const __nv_bfloat16*)bias,
             (__nv_bfloat16*)y, ldy, N, K);
}

template <int FMT>
static void launch_gemv_t(int T, const void* x, long long ldx, const void* codes, const void* scales, float alpha,
                          const void* bias, void* y, long long ldy, int N, int K, cudaStream_t s) {
  switch (T) {
    case 1: launch_gemv<1, FMT>(x, ldx, codes, scales, alpha, bias, y, ldy, N, K, s); break;
    case 2: launch_gemv<2, FMT>(x, ldx, codes, scales, alpha, bias, y, ldy, N, K, s); break;
    case 3: launch_gemv<3, FMT>(x, ldx, codes, scales, alpha, bias, y, ldy, N, K, s); break;
    default: launch_gemv<4, FMT>(x, ldx, codes, scales, alpha, bias, y, ldy, N, K, s); break;
  }
}

bool gemv_w4_supported(int T, int K) {
  return T >= 1 && T <= kGvMaxT && K % 32 == 0 && (size_t)T * K + (size_t)T * (K / 32) * 8 <= 160 * 1024;
}

// y[T][N] = x[T][K] * dequant(codes, scales)^T * alpha (+ bias) for T <= 4; formats as in linear_w4a16.
int gemv_w4(const void* x, long long ldx, const void* codes, const void* scales, int fmt, float alpha, const void* bias,
            void* y, long long ldy, int T, int N, int K, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (!gemv_w4_supported(T, K)) throw std::runtime_error("gemv_w4: at most 4 tokens, K a multiple of 32 that fits shared memory");
  if ((ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(codes) & 15))
    throw std::runtime_error("gemv_w4: activations and codes must be 16-byte aligned");
  switch (fmt) {
    case 0: launch_gemv_t<0>(T, x, ldx, codes, scales, alpha, bias, y, ldy, N, K, stream); break;
    case 1: launch_gemv_t<1>(T, x, ldx, codes, scales, alpha, bias, y, ldy, N, K, stream); break;
    case 2: launch_gemv_t<2>(T, x, ldx, codes, scales, alpha, bias, y, ldy, N, K, stream); break;
    default: throw std::runtime_error("gemv_w4: fmt must be 0 (NVFP4), 1 (MXFP4) or 2 (INT4G)");
  }
  return 1;
}

}  // namespace fllm
