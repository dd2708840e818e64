// Block-scaled MX GEMM on the fifth-generation tensor cores (tcgen05.mma kind::mxf8f6f4.block_scale):
//
//   y[T][N] = alpha * sum_k (xq[t][k] * 2^(sx[t][k/32] - 127)) * (wq[n][k] * 2^(sw[n][k/32] - 127))  (+ bias)
//
//   weights      MXFP8: e4m3 bytes [N][K], or MXFP4: e2m1 codes, two per byte [N][K/2] (low nibble = even k),
//                with one e8m0 (power-of-two) scale per 32 values
//   activations  e4m3 [T][K] + one e8m0 scale per token per 32 values, produced from bf16 by quant_mx_kernel
//
// The scales never touch the ALUs: they are copied from shared memory into tensor memory (tcgen05.cp) and
// the MMA applies them to every 32-deep slice of the dot product, so a packed 4-bit weight goes from HBM to
// the tensor core without an expansion stage (TMA's 16U4_ALIGN16B type spreads 16 codes over 16 bytes of
// shared memory, the form the instruction reads). That is what makes a 4-bit weight cost 4.25 bits of HBM
// traffic and nothing else.
//
// Scale factors travel in 512-byte atoms that cover 128 rows x 128 values of K (4 scales per row):
//   byte (r % 32) * 16 + (r / 32) * 4 + j   holds the scale of row r, K slice j
// which is the order in which tcgen05.cp (32 rows x 128 bits, replicated over the four lane quarters) lays
// them into four tensor-memory columns: row r -> lane r % 32, column r / 32, byte j. The instruction
// descriptor names the byte (the K slice) each of the four MMAs of a stage uses. Weight atoms are built at
// load time ([N / 128][K / 128][512]); the activation quantiser writes atoms per token tile.
//
// Orientation: weights are the A operand (M = 128 output features per tile), tokens the B operand
// (N = 16 ... 128 per tile), for decode and prefill alike; results are stored transposed. Few feature
// tiles split K over grid.z (fp32 partial sums + a reduce kernel). Warp roles and TMA staging follow
// gemm_fp8.cu; every wait is bounded and reports through the status word.
//
// A third kind runs NVFP4 on both sides (kind::mxf4nvf4.block_scale.block16): packed e2m1 codes for weights and
// activations (256 values of K per 128-byte row, so a stage carries twice the K of the 8-bit kinds), one e4m3
// scale per 16 values (four per row per MMA of K = 64: a whole atom per MMA), the weight's tensor scale and a
// per-token activation scale applied in the epilogue. The activation quantiser (quant_nvfp4_kernel) derives the
// token scale from the token's largest magnitude, so no calibration pass is needed.
//
// Two more kinds share the tile loop without block scales: e4m3 x e4m3 (kind::f8f6f4) and int8 x int8 (kind::i8,
// int32 accumulators) with one scale per output feature and one per token, applied in the epilogue. They are the
// W8A8 forms of per-channel FP8 and SmoothQuant-style INT8 checkpoints (dynamic per-token activation scales,
// quant_rows_8bit_kernel).
//
// Reference counterparts: rust/engine/cuda/nvfp4.cu:132-307 (mma.sync block-scaled FP4 for GeForce
// Blackwell; the data-centre parts fall back to W4A16 Marlin there), rust/engine/cuda/mxfp4_moe.cu.
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <algorithm>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

constexpr int MX_BM = 128;
constexpr int kMxThreads = 192;
constexpr int kMxAtomBytes = 512;

struct MxArgs {
  int M, N, K;                   // M = output features, N = tokens
  int m_tiles, n_tiles, k_blocks;
  int k_splits, kb_per_split;
  float* ws;                     // [k_splits][N][M] fp32 when k_splits > 1
  long long ldc;
  __nv_bfloat16* out;
  const uint8_t* sfa;            // [m_tiles][k_blocks][512]
  const uint8_t* sfb;            // [n_tiles][k_blocks][512]
  float alpha;
  const float* tok_scale;        // [N] per-token factor (NVFP4 and row-scaled activations), or null
  const float* feat_scale;       // [M] per-feature factor (row-scaled 8-bit weights), or null
  const __nv_bfloat16* bias;
  int* status;
};

// KIND: 0 = e4m3 weights, 1 = packed e2m1 weights unpacked by TMA (both kind::mxf8f6f4, e8m0 scales per 32,
// 128 values of K per stage), 2 = packed e2m1 on both sides (kind::mxf4nvf4, e4m3 scales per 16, 256 per stage).
// 3 = e4m3 x e4m3 and 4 = int8 x int8 without block scales (one scale per feature and per token, in the epilogue).
constexpr int kMxKindE4M3 = 0, kMxKindE2M1A8 = 1, kMxKindNvf4 = 2, kMxKindRowF8 = 3, kMxKindRowI8 = 4;
__host__ __device__ constexpr bool mx_kind_has_sf(int kind) { return kind <= kMxKindNvf4; }

template <int BN, int KIND>
struct MxSmem {
  static constexpr int kABytes = MX_BM * 128;                   // 128-byte rows in shared memory for every kind
  static constexpr int kBBytes = BN * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStageK = KIND == kMxKindNvf4 ? 256 : 128;
  static constexpr int kAtoms = KIND == kMxKindNvf4 ? 4 : (mx_kind_has_sf(KIND) ? 1 : 0);   // scale atoms per operand per stage
  // two CTAs per SM when BN <= 64: the NVFP4 stage carries 4 KB of scale atoms, so three stages fit twice
  static constexpr int kStages = BN <= 64 ? (KIND == kMxKindNvf4 ? 3 : 4) : 6;
  static constexpr int kAccCols = BN < 32 ? 32 : BN;
  static constexpr int kSfCols = kAtoms ? 2 * 8 * kAtoms : 0;   // two buffers of (A, B) x 4 columns per atom
  static constexpr int kTmemCols = kAccCols + kSfCols <= 64 ? 64 : (kAccCols + kSfCols <= 128 ? 128 : 256);
  static constexpr int kSfBytes = kStages * 2 * kAtoms * kMxAtomBytes;
  static constexpr int kTotal = kStages * kStageBytes + kSfBytes + 256 + 1024;
  static_assert(4 * 32 * 32 * 2 <= kABytes, "the epilogue staging reuses the first weight stage");
  static_assert(kAccCols + kSfCols <= 256, "tensor memory columns");
  static_assert(BN > 64 || 2 * (kTotal + 1024) <= 227 * 1024, "two CTAs per SM");
};

// Shared-memory descriptor of one scale-factor atom for tcgen05.cp: K-major, no swizzle, 8-row x 16-byte
// core matrices 128 bytes apart along the rows; a single core matrix along K.
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(128 >> 4) << 32;                 // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                          // descriptor version 1 (sm_100)
  return d;                                        // layout type 0: no swizzle
}

__device__ __forceinline__ void tc_cp_sf(uint32_t tmem_dst, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(sdesc) : "memory");
}

// Instruction descriptor of the block-scaled kinds: fp32 accumulate, K-major operands. kind::mxf8f6f4 formats:
// 0 e4m3, 1 e5m2, 5 e2m1; kind::mxf4nvf4: 1 e2m1. Bit 23: the scales are e8m0 (set) or e4m3 (clear). The
// scale-factor ids (bits 29-30 for A, 4-5 for B) are OR-ed in per MMA.
__host__ __device__ constexpr uint32_t make_idesc_mx(int M, int N, int a_fmt, int b_fmt, int e8m0) {
  return ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)e8m0 << 23) |
         ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void tc_mma_mx(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

__device__ __forceinline__ void tc_mma_nvf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

// int8 x int8 -> int32 accumulators; idesc: D format S32 (2 at bits 4-5), signed operands (format 1)
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__host__ __device__ constexpr uint32_t make_idesc_i8(int M, int N) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

template <int BN, int KIND>
__global__ void __launch_bounds__(kMxThreads, BN <= 64 ? 2 : 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const MxArgs p) {
  using S = MxSmem<BN, KIND>;
  constexpr int SF_STAGE = 2 * S::kAtoms * kMxAtomBytes;      // bytes of scale factors per stage (A atoms, then B atoms)
  constexpr int STAGES = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * S::kABytes;
  uint8_t* sSF = smem + STAGES * S::kStageBytes;            // per stage: A atom, B atom
  uint64_t* bars = reinterpret_cast<uint64_t*>(sSF + S::kSfBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_idx = blockIdx.x, m_idx = blockIdx.y;
  const int kb0 = blockIdx.z * p.kb_per_split;
  const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tma_a); tma_prefetch_desc(&tma_b); }
  if (warp == 1) { tmem_alloc(tmem_slot, S::kTmemCols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      pdl_wait();                                              // the activations come from the kernel before
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) break;
        // a 4-bit tile that TMA unpacks is counted by the bytes that leave global memory, not by the padded bytes it fills
        mbar_expect_tx(&full_bar[stage], (KIND == kMxKindE2M1A8 ? S::kABytes / 2 : S::kABytes) + S::kBBytes + SF_STAGE);
        // x coordinates are in elements of the tensor map: K values for the 8-bit and unpacking maps, bytes for packed codes
        const int xa = KIND == kMxKindNvf4 ? kb * 128 : kb * S::kStageK;
        tma_load_2d(sA + stage * S::kABytes, &tma_a, &full_bar[stage], xa, m_idx * MX_BM);
        tma_load_2d(sB + stage * S::kBBytes, &tma_b, &full_bar[stage], xa, n_idx * BN);
        if constexpr (SF_STAGE > 0) {
          bulk_load_1d(sSF + stage * SF_STAGE, p.sfa + ((size_t)m_idx * p.k_blocks + kb) * (SF_STAGE / 2), SF_STAGE / 2,
                       &full_bar[stage]);
          bulk_load_1d(sSF + stage * SF_STAGE + SF_STAGE / 2, p.sfb + ((size_t)n_idx * p.k_blocks + kb) * (SF_STAGE / 2),
                       SF_STAGE / 2, &full_bar[stage]);
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = KIND == kMxKindNvf4    ? make_idesc_mx(MX_BM, BN, 1, 1, 0)
                                 : KIND == kMxKindRowF8 ? make_idesc(MX_BM, BN, 0, 0)
                                 : KIND == kMxKindRowI8 ? make_idesc_i8(MX_BM, BN)
                                                        : make_idesc_mx(MX_BM, BN, KIND == kMxKindE2M1A8 ? 5 : 0, 0, 1);
      constexpr int SFC = 4 * S::kAtoms;                      // columns of one operand's scales per buffer
      const uint32_t tmem_sf = tmem_base + S::kAccCols;       // two buffers: A scales, then B scales
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t sf_cols = tmem_sf + ((kb - kb0) & 1) * 2 * SFC;
#pragma unroll
        for (int a = 0; a < 2 * S::kAtoms; ++a)
          tc_cp_sf(sf_cols + 4 * a, make_sf_desc(smem_u32(sSF + stage * SF_STAGE + a * kMxAtomBytes)));
        const uint64_t da = make_smem_desc_sw128(smem_u32(sA + stage * S::kABytes));
        const uint64_t db = make_smem_desc_sw128(smem_u32(sB + stage * S::kBBytes));
#pragma unroll
        for (int k = 0; k < 4; ++k) {                         // four MMAs of 32 bytes of K each
          const uint32_t acc = (kb > kb0 || k > 0) ? 1u : 0u;
          if constexpr (KIND == kMxKindRowF8)
            tc_mma_f8f6f4(tmem_base, da + 2 * k, db + 2 * k, idesc, acc);
          else if constexpr (KIND == kMxKindRowI8)
            tc_mma_i8(tmem_base, da + 2 * k, db + 2 * k, idesc, acc);
          else if constexpr (KIND == kMxKindNvf4)             // K = 64: a whole atom (four scales per row) per MMA
            tc_mma_nvf4(tmem_base, da + 2 * k, db + 2 * k, idesc, sf_cols + 4 * k, sf_cols + SFC + 4 * k, acc);
          else                                                // K = 32: byte k of the atom's columns
            tc_mma_mx(tmem_base, da + 2 * k, db + 2 * k, idesc | ((uint32_t)k << 29) | ((uint32_t)k << 4), sf_cols,
                      sf_cols + SFC, acc);
        }
        tc_commit(&empty_bar[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (ok) tc_commit(tfull_bar);
    }
  } else {
    const int q = warp & 3;
    const int e = warp - 2;
    if (kb1 > kb0 && mbar_wait(tfull_bar, 0, abort_flag)) {
      tc_fence_after_sync();
      const int m = m_idx * MX_BM + q * 32 + lane;
      const int n_base = n_idx * BN;
      const float bias_m = (p.bias && m < p.M) ? __bfloat162float(p.bias[m]) : 0.f;
      const float fs = (p.feat_scale && m < p.M) ? p.feat_scale[m] : 1.f;
      auto acc_f = [](uint32_t v) -> float {                   // the accumulator as a float (int32 for the int8 kind)
        if constexpr (KIND == kMxKindRowI8) return (float)(int)v;
        else return __uint_as_float(v);
      };
      const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
      __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(sA) + e * (32 * 32);
      constexpr int CH = BN < 32 ? 16 : 32;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += CH) {
        uint32_t r[CH];
        if constexpr (CH == 32) tmem_ld_32x32(t_lane + c0, r);
        else tmem_ld_32x16(t_lane + c0, r);
        tmem_ld_wait();
        if (p.k_splits > 1) {                                  // fp32 partial sums, lanes along features: coalesced
          float* wsp = p.ws + (size_t)blockIdx.z * p.N * p.M;
#pragma unroll
          for (int c = 0; c < CH; ++c)
            if (n_base + c0 + c < p.N && m < p.M) wsp[(size_t)(n_base + c0 + c) * p.M + m] = acc_f(r[c]) * fs;
          continue;
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const float ts = p.tok_scale ? p.tok_scale[min(n_base + c0 + c, p.N - 1)] : 1.f;
          stg[c * 32 + lane] = __float2bfloat16(acc_f(r[c]) * (p.alpha * ts * fs) + bias_m);
        }
        __syncwarp();
        const int f0 = 8 * (lane & 3);
        const int mm0 = m_idx * MX_BM + q * 32 + f0;
#pragma unroll
        for (int rnd = 0; rnd < CH / 8; ++rnd) {
          const int c = (lane >> 2) + 8 * rnd;
          const int n = n_base + c0 + c;
          if (n < p.N && mm0 < p.M)
            *reinterpret_cast<uint4*>(p.out + (size_t)n * p.ldc + mm0) = *reinterpret_cast<const uint4*>(stg + c * 32 + f0);
        }
        __syncwarp();
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tmem_base, S::kTmemCols); }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicCAS(p.status, FLLM_OK, FLLM_ERR_MBAR_TIMEOUT);
}

// out[n][m] = bf16(alpha * sum_s ws[s][n][m] + bias[m])
__global__ void mx_splitk_reduce_kernel(const float* __restrict__ ws, int splits, int rows, int cols, long long ldc,
                                        float alpha, const float* __restrict__ tok_scale,
                                        const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t n = (size_t)rows * cols;
  const size_t i4 = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 >= n) return;
  float4 acc = *reinterpret_cast<const float4*>(ws + i4);
  for (int s = 1; s < splits; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(ws + (size_t)s * n + i4);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  const int r = (int)(i4 / cols);
  const int c = (int)(i4 - (size_t)r * cols);
  float b[4] = {0.f, 0.f, 0.f, 0.f};
  if (bias) for (int i = 0; i < 4; ++i) b[i] = __bfloat162float(bias[c + i]);
  if (tok_scale) alpha *= tok_scale[r];
  uint2 o;
  o.x = pack_bf16x2(acc.x * alpha + b[0], acc.y * alpha + b[1]);
  o.y = pack_bf16x2(acc.z * alpha + b[2], acc.w * alpha + b[3]);
  *reinterpret_cast<uint2*>(out + (size_t)r * ldc + c) = o;
}

// x bf16 [T][K] -> e4m3 [T][K] + e8m0 scales per 32 values in atoms of `bn`-token tiles:
// sf[(t / bn) * (K / 128) + kb][512]. One warp per (token, 128-value block); eight lanes share a scale.
// The scale is the smallest power of two that brings the group's largest magnitude under 448. Rows past
// T inside the last tile get zero scales.
__global__ void quant_mx_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ xq,
                                uint8_t* __restrict__ sf, int tokens, int padded_tokens, int K, int bn) {
  pdl_launch_dependents();
  pdl_wait();
  const int kb_n = K / 128;
  const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= (long long)padded_tokens * kb_n) return;
  const int t = (int)(gw / kb_n), kb = (int)(gw - (long long)t * kb_n), lane = threadIdx.x & 31;
  const int r = t % bn;
  uint8_t* atom = sf + ((size_t)(t / bn) * kb_n + kb) * kMxAtomBytes + (r & 31) * 16 + (r >> 5) * 4;
  if (t >= tokens) {
    if ((lane & 7) == 0) atom[lane >> 3] = 0;
    return;
  }
  const uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)t * ldx + kb * 128 + lane * 4);
  const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  // smallest e with amax * 2^-e <= 448: e = ceil(log2(amax / 448)); frexp gives amax / 448 = f * 2^ex, f in [0.5, 1)
  int e = -127;
  if (amax > 0.f) {
    int ex;
    const float f = frexpf(amax / 448.f, &ex);          // the division is exact where the quotient is a power of two
    e = f == 0.5f ? ex - 1 : ex;
    e = max(-127, min(127, e));
  }
  const float inv = exp2f((float)-e);
  __nv_fp8x4_e4m3 q(make_float4(a.x * inv, a.y * inv, b.x * inv, b.y * inv));
  *reinterpret_cast<uint32_t*>(xq + (size_t)t * K + kb * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(&q);
  if ((lane & 7) == 0) atom[lane >> 3] = (uint8_t)(e + 127);
}

// x bf16 [T][K] -> packed e2m1 codes [T][K/2] + e4m3 scales per 16 values in atoms of `bn`-token tiles
// (sf[(t / bn) * (K / 64) + k64][512]) + one fp32 scale per token: value = code * block_scale * tok_scale.
// tok_scale = (largest magnitude of the token) / (6 * 448), so the block scales use the whole e4m3 range.
// One CTA per token; a thread owns 16-value groups g = tid, tid + 256, ... (at most 8: K <= 32768).
__global__ void __launch_bounds__(256)
quant_nvfp4_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ xq, uint8_t* __restrict__ sf,
                   float* __restrict__ tok_scale, int tokens, int K, int bn) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[8];
  const int t = blockIdx.x;
  const int groups = K / 16, k64_n = K / 64;
  const int r = t % bn;
  uint8_t* atoms = sf + (size_t)(t / bn) * k64_n * kMxAtomBytes + (r & 31) * 16 + (r >> 5) * 4;
  if (t >= tokens) {                                     // padding rows of the last tile: zero scales
    for (int g = threadIdx.x; g < groups; g += 256) atoms[(size_t)(g >> 2) * kMxAtomBytes + (g & 3)] = 0;
    return;
  }
  constexpr int MAXG = 8;
  uint4 v[MAXG][2];
  float gmax[MAXG];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < MAXG; ++i) {
    const int g = threadIdx.x + i * 256;
    gmax[i] = 0.f;
    if (g < groups) {
      const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * ldx + g * 16);
      v[i][0] = src[0];
      v[i][1] = src[1];
      const uint32_t* w = reinterpret_cast<const uint32_t*>(v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        gmax[i] = fmaxf(gmax[i], fmaxf(fabsf(f.x), fabsf(f.y)));
      }
      amax = fmaxf(amax, gmax[i]);
    }
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float ts = amax > 0.f ? amax / (6.f * 448.f) : 1.f;
  if (threadIdx.x == 0) tok_scale[t] = ts;
#pragma unroll
  for (int i = 0; i < MAXG; ++i) {
    const int g = threadIdx.x + i * 256;
    if (g >= groups) continue;
    const __nv_fp8_storage_t sb = __nv_cvt_float_to_fp8(gmax[i] / 6.f / ts, __NV_SATFINITE, __NV_E4M3);
    const float sbf = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3)));
    const float inv = sbf > 0.f ? 1.f / (sbf * ts) : 0.f;
    const uint32_t* w = reinterpret_cast<const uint32_t*>(v[i]);
    uint32_t out[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      const uint32_t c2 = __nv_cvt_float2_to_fp4x2(make_float2(f.x * inv, f.y * inv), __NV_E2M1, cudaRoundNearest);
      out[j >> 2] |= (c2 & 0xFFu) << (8 * (j & 3));
    }
    *reinterpret_cast<uint2*>(xq + (size_t)t * (K / 2) + g * 8) = make_uint2(out[0], out[1]);
    atoms[(size_t)(g >> 2) * kMxAtomBytes + (g & 3)] = sb;
  }
}

// x bf16 [T][K] -> 8-bit codes [T][K] with one scale per token (largest magnitude / 127 for int8, / 448 for e4m3).
// One CTA per token.
template <bool I8>
__global__ void __launch_bounds__(256)
quant_rows_8bit_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ xq, float* __restrict__ tok_scale,
                       int K) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[8];
  const int t = blockIdx.x;
  const __nv_bfloat16* row = x + (size_t)t * ldx;
  float amax = 0.f;
  for (int i = threadIdx.x * 8; i < K; i += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(w[e]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float qmax = I8 ? 127.f : 448.f;
  const float scale = amax > 0.f ? amax / qmax : 1.f;
  const float inv = 1.f / scale;
  if (threadIdx.x == 0) tok_scale[t] = scale;
  for (int i = threadIdx.x * 8; i < K; i += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[2] = {0u, 0u};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(w[e]);
      uint32_t two;
      if constexpr (I8) {
        const int a = max(-127, min(127, __float2int_rn(f.x * inv))), b = max(-127, min(127, __float2int_rn(f.y * inv)));
        two = (uint32_t)(a & 0xFF) | ((uint32_t)(b & 0xFF) << 8);
      } else {
        two = __nv_cvt_float2_to_fp8x2(make_float2(f.x * inv, f.y * inv), __NV_SATFINITE, __NV_E4M3);
      }
      o[e >> 1] |= two << (16 * (e & 1));
    }
    *reinterpret_cast<uint2*>(xq + (size_t)t * K + i) = make_uint2(o[0], o[1]);
  }
}

void quant_rows_8bit(const void* x, long long ldx, void* xq, float* tok_scale, int T, int K, int is_int8, cudaStream_t s) {
  if (T <= 0) return;
  if (K % 8 || (ldx & 7)) throw std::runtime_error("quant_rows_8bit: K and the row pitch must be multiples of 8");
  if (is_int8)
    launch_pdl(quant_rows_8bit_kernel<true>, dim3((unsigned)T), dim3(256), 0, s, (const __nv_bfloat16*)x, ldx, (uint8_t*)xq, tok_scale, K);
  else
    launch_pdl(quant_rows_8bit_kernel<false>, dim3((unsigned)T), dim3(256), 0, s, (const __nv_bfloat16*)x, ldx, (uint8_t*)xq, tok_scale, K);
}

int mx_token_tile(int T) { return T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : 128; }

// Bytes of the activation scale atoms for T tokens: one e8m0 per 32 values (kind 0 / 1) or one e4m3 per 16 (kind 2).
size_t mx_act_scale_bytes(int T, int K, int kind) {
  const int bn = mx_token_tile(T);
  return (size_t)((T + bn - 1) / bn) * (K / (kind == kMxKindNvf4 ? 64 : 128)) * kMxAtomBytes;
}

void quant_mx(const void* x, long long ldx, void* xq, void* sf, int T, int K, cudaStream_t s) {
  if (T <= 0) return;
  if (K % 128) throw std::runtime_error("quant_mx: K must be a multiple of 128");
  const int bn = mx_token_tile(T);
  const int padded = (T + bn - 1) / bn * bn;
  const long long groups = (long long)padded * (K / 128);
  launch_pdl(quant_mx_kernel, dim3((unsigned)((groups + 7) / 8)), dim3(256), 0, s, (const __nv_bfloat16*)x, ldx,
             (uint8_t*)xq, (uint8_t*)sf, T, padded, K, bn);
}

void quant_nvfp4(const void* x, long long ldx, void* xq, void* sf, float* tok_scale, int T, int K, cudaStream_t s) {
  if (T <= 0) return;
  if (K % 256 || K > 32768 || (ldx & 7)) throw std::runtime_error("quant_nvfp4: K must be a multiple of 256, at most 32768, rows 16-byte aligned");
  const int bn = mx_token_tile(T);
  const int padded = (T + bn - 1) / bn * bn;
  launch_pdl(quant_nvfp4_kernel, dim3((unsigned)padded), dim3(256), 0, s, (const __nv_bfloat16*)x, ldx, (uint8_t*)xq,
             (uint8_t*)sf, tok_scale, T, K, bn);
}

template <int BN, int KIND>
static void launch_mx(const CUtensorMap& ta, const CUtensorMap& tb, const MxArgs& a, cudaStream_t s) {
  using S = MxSmem<BN, KIND>;
  static bool configured[kMaxDevices] = {};
  if (first_call_on_device(configured)) {
    cuda_check(cudaFuncSetAttribute(gemm_mx_kernel<BN, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal),
               "cudaFuncSetAttribute(gemm_mx_kernel)");
  }
  launch_pdl(gemm_mx_kernel<BN, KIND>, dim3(a.n_tiles, a.m_tiles, a.k_splits), dim3(kMxThreads), (size_t)S::kTotal, s, ta, tb, a);
}

template <int KIND>
static void launch_mx_bn(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const MxArgs& a, cudaStream_t s) {
  switch (bn) {
    case 16: launch_mx<16, KIND>(ta, tb, a, s); break;
    case 32: launch_mx<32, KIND>(ta, tb, a, s); break;
    case 64: launch_mx<64, KIND>(ta, tb, a, s); break;
    default: launch_mx<128, KIND>(ta, tb, a, s); break;
  }
}

// y[T][N] = alpha * tok_scale[t] * dequant(xq, sfb) * dequant(wq, sfa)^T (+ bias).
// kind 0: e4m3 weights [N][K] x e4m3 activations [T][K]; kind 1: e2m1 weights [N][K/2] x e4m3 activations;
// kind 2: e2m1 weights [N][K/2] x e2m1 activations [T][K/2] with e4m3 scales per 16 (NVFP4);
// kind 3 / 4: e4m3 / int8 weights [N][K] x activations [T][K] with feat_scale[N] and tok_scale[T] (no scale atoms).
int linear_mx(const void* xq, const void* sfb, const void* wq, const void* sfa, int kind, float alpha,
              const float* tok_scale, const float* feat_scale, const void* bias, void* y, long long ldy, int T, int N, int K,
              void* workspace, size_t workspace_bytes, int* status, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (kind < 0 || kind > 4) throw std::runtime_error("linear_mx: kind must be 0 ... 4");
  if (mx_kind_has_sf(kind) ? (!sfa || !sfb) : (!feat_scale || !tok_scale))
    throw std::runtime_error("linear_mx: block-scaled kinds need scale atoms, row-scaled kinds need feature and token scales");
  const int stage_k = kind == kMxKindNvf4 ? 256 : 128;
  if (K % stage_k || N % 8 || (ldy & 7)) throw std::runtime_error("linear_mx: K % 128 (256 for NVFP4), N % 8 and 16-byte output rows required");
  if ((reinterpret_cast<uintptr_t>(wq) & 31) || (reinterpret_cast<uintptr_t>(xq) & 15) || (reinterpret_cast<uintptr_t>(sfa) & 15) ||
      (reinterpret_cast<uintptr_t>(sfb) & 15))
    throw std::runtime_error("linear_mx: operands must be 32-byte (weights) and 16-byte (scales) aligned");
  MxArgs a{};
  a.M = N; a.N = T; a.K = K;
  a.m_tiles = (N + MX_BM - 1) / MX_BM; a.k_blocks = K / stage_k;
  const int bn = mx_token_tile(T);
  a.n_tiles = (T + bn - 1) / bn;
  a.ldc = ldy; a.out = reinterpret_cast<__nv_bfloat16*>(y);
  a.sfa = reinterpret_cast<const uint8_t*>(sfa); a.sfb = reinterpret_cast<const uint8_t*>(sfb);
  a.alpha = alpha; a.tok_scale = tok_scale; a.feat_scale = feat_scale; a.bias = reinterpret_cast<const __nv_bfloat16*>(bias); a.status = status;
  // Few tiles cannot pull the whole HBM bandwidth: split K over grid.z until the machine is full.
  const int slots = sm_count() * (bn <= 64 ? 2 : 1);
  const int tiles = a.m_tiles * a.n_tiles;
  int splits = 1;
  if (tiles * 2 <= slots && a.k_blocks >= 8) splits = std::min(std::min(slots / tiles, a.k_blocks / 4), 8);
  while (splits > 1 && (!workspace || (size_t)splits * T * N * 4 > workspace_bytes)) --splits;
  a.kb_per_split = (a.k_blocks + splits - 1) / splits;
  a.k_splits = (a.k_blocks + a.kb_per_split - 1) / a.kb_per_split;
  a.ws = reinterpret_cast<float*>(workspace);
  CUtensorMap ta, tb;
  if (kind == kMxKindE2M1A8) ta = make_tmap_2d(wq, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 1, N, K, K / 2, MX_BM, 128, true);
  else if (kind == kMxKindNvf4) ta = make_tmap_2d(wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, K / 2, MX_BM, 128, true);
  else ta = make_tmap_2d(wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, MX_BM, 128, true);
  if (kind == kMxKindNvf4) tb = make_tmap_2d(xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, T, K / 2, K / 2, bn, 128, true);
  else tb = make_tmap_2d(xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, T, K, K, bn, 128, true);
  if (kind == kMxKindE4M3) launch_mx_bn<kMxKindE4M3>(bn, ta, tb, a, stream);
  else if (kind == kMxKindE2M1A8) launch_mx_bn<kMxKindE2M1A8>(bn, ta, tb, a, stream);
  else if (kind == kMxKindNvf4) launch_mx_bn<kMxKindNvf4>(bn, ta, tb, a, stream);
  else if (kind == kMxKindRowF8) launch_mx_bn<kMxKindRowF8>(bn, ta, tb, a, stream);
  else launch_mx_bn<kMxKindRowI8>(bn, ta, tb, a, stream);
  if (a.k_splits > 1) {
    const size_t n = (size_t)T * N;
    launch_pdl(mx_splitk_reduce_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, stream,
               (const float*)a.ws, a.k_splits, T, N, ldy, alpha, tok_scale, a.bias, a.out);
    return 2;
  }
  return 1;
}

}  // namespace fllm
