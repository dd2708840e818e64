// Block-scaled FP8 (e4m3) GEMM on tcgen05:  y = (x_q * sx) (w_q * sw)^T
//
//   weights      e4m3 [N][K] with one fp32 scale per 128 x 128 block  (sw[N/128][K/128])
//   activations  e4m3 [T][K] with one fp32 scale per token per 128 K  (sx[T][K/128]),
//                produced by quant_fp8_1x128_kernel from bf16 (dynamic, amax / 448)
//
// These scales do not map onto the hardware's 1x32 block-scaled MMA (that needs power-of-two
// scales per 32 values), so every 128-deep K block is multiplied unscaled into a fresh TMEM
// accumulator (tcgen05.mma kind::f8f6f4, four K=32 instructions) and the epilogue warps
// promote it: they read the partial sums out of TMEM, multiply by sx * sw of that K block and
// add them into fp32 registers. Two TMEM buffers alternate, so the tensor core works on K block
// i+1 while block i is being promoted. Warp roles, TMA staging (128-byte swizzle, one K block
// = one 128-byte row) and the swap-AB orientation for small token counts are those of
// gemm_bf16.cu.
//
// Reference counterparts: rust/engine/cuda/fp8_block.cu:94-312 (FP32 GEMV / FP16-expanded GEMM for
// block-wise FP8 weights), rust/engine/cuda/fp8_gemm.cu:44-78 (per-128-group activation quant).
// Unlike the reference (docs/multi-gpu.md:166) the format can be cut for tensor parallelism on
// 128-element boundaries.
#include <cuda_fp8.h>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

constexpr int F8_BM = 128;
constexpr int F8_BK = 128;      // e4m3 elements = bytes per swizzle row = scale block depth
constexpr int F8_UMMA_K = 32;
constexpr int kF8Threads = 192;

struct Fp8GemmArgs {
  int M, N, K;              // MMA orientation: D[M][N] = A[M][K] B[N][K]^T
  int m_tiles, n_tiles, k_blocks;
  int transposed;           // 1: A = weights (M = features), tokens in N; out[n * ldc + m]
  long long ldc;
  __nv_bfloat16* out;
  const float* sx;          // [tokens][k_blocks]
  const float* sw;          // [features / 128][k_blocks]
  const __nv_bfloat16* bias;
  int* status;
  int k_splits, kb_per_split;   // work items are (tile, split): few tiles cannot pull the whole HBM bandwidth otherwise
  float* ws;                    // [k_splits][tokens][features] fp32 partial sums when k_splits > 1
};

template <int BN>
struct Fp8Smem {
  static constexpr int kABytes = F8_BM * F8_BK;
  static constexpr int kBBytes = BN * F8_BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN <= 64 ? 80 * 1024 : 160 * 1024) / kStageBytes;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int kScaleFloats = 64 * BN;            // token scales of a swap-AB tile, up to 64 K blocks
  static constexpr int kTotal = kStages * kStageBytes + kScaleFloats * 4 + 256 + 1024;
};

template <int BN>
__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const Fp8GemmArgs p) {
  using S = Fp8Smem<BN>;
  constexpr int STAGES = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * S::kABytes;
  float* s_scale = reinterpret_cast<float*>(smem + STAGES * S::kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_scale + S::kScaleFloats);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 128); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tma_a); tma_prefetch_desc(&tma_b); }
  if (warp == 1) { tmem_alloc(tmem_slot, S::kTmemCols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles = p.m_tiles * p.n_tiles * p.k_splits;      // work items: the split is the fastest index

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < tiles && ok; w += gridDim.x) {
        const int split = w % p.k_splits, t = w / p.k_splits;
        const int n_idx = t / p.m_tiles, m_idx = t - n_idx * p.m_tiles;
        const int kb0 = split * p.kb_per_split, kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&full_bar[stage], S::kStageBytes);
          tma_load_2d(sA + stage * S::kABytes, &tma_a, &full_bar[stage], kb * F8_BK, m_idx * F8_BM);
          tma_load_2d(sB + stage * S::kBBytes, &tma_b, &full_bar[stage], kb * F8_BK, n_idx * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(F8_BM, BN, 0, 0);      // e4m3 x e4m3
      int stage = 0, buf = 0;
      uint32_t phase = 0, buf_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < tiles && ok; w += gridDim.x) {
        const int split = w % p.k_splits;
        const int kb0 = split * p.kb_per_split, kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          // each K block gets its own accumulator: wait until the epilogue drained this buffer
          if (!mbar_wait(&tempty_bar[buf], buf_phase ^ 1, abort_flag)) { ok = false; break; }
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t da = make_smem_desc_sw128(smem_u32(sA + stage * S::kABytes));
          const uint64_t db = make_smem_desc_sw128(smem_u32(sB + stage * S::kBBytes));
#pragma unroll
          for (int k = 0; k < F8_BK / F8_UMMA_K; ++k)
            tc_mma_f8f6f4(tmem_base + buf * BN, da + 2 * k, db + 2 * k, idesc, k > 0 ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
          tc_commit(&tfull_bar[buf]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          buf ^= 1;
          if (buf == 0) buf_phase ^= 1;
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int etid = (warp - 2) * 32 + lane;                        // 0..127 among epilogue threads
    int buf = 0;
    uint32_t buf_phase = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < tiles && ok; w += gridDim.x) {
      const int split = w % p.k_splits, t = w / p.k_splits;
      const int n_idx = t / p.m_tiles, m_idx = t - n_idx * p.m_tiles;
      const int kb0 = split * p.kb_per_split, kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
      const int m = m_idx * F8_BM + q * 32 + lane;
      const int n_base = n_idx * BN;
      if (p.transposed) {
        // token scales of the tile: s_scale[kb][c] = sx[n_base + c][kb]
        asm volatile("bar.sync 1, 128;" ::: "memory");              // previous tile finished reading
        for (int i = etid; i < (kb1 - kb0) * BN; i += 128) {
          const int kb = kb0 + i / BN, c = i % BN;
          const int tok = n_base + c;
          s_scale[i] = tok < p.N ? p.sx[(size_t)tok * p.k_blocks + kb] : 0.f;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      float acc[BN];
#pragma unroll
      for (int c = 0; c < BN; ++c) acc[c] = 0.f;
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        if (!mbar_wait(&tfull_bar[buf], buf_phase, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t t_row = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
        float row_scale;                                            // constant along the thread's row
        if (p.transposed) row_scale = p.sw[(size_t)m_idx * p.k_blocks + kb];          // 128 features = 1 block
        else row_scale = m < p.M ? p.sx[(size_t)m * p.k_blocks + kb] : 0.f;
        constexpr int CH = BN < 32 ? 16 : 32;
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += CH) {
          uint32_t r[32];
          if constexpr (CH == 32) {
            tmem_ld_32x32(t_row + c0, r);
          } else {
            uint32_t r16[16];
            tmem_ld_32x16(t_row + c0, r16);
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = r16[i];
          }
          tmem_ld_wait();
          if (p.transposed) {
#pragma unroll
            for (int c = 0; c < CH; ++c) acc[c0 + c] += __uint_as_float(r[c]) * (row_scale * s_scale[(kb - kb0) * BN + c0 + c]);
          } else {
#pragma unroll
            for (int c = 0; c < CH; ++c) {
              // columns are features: one weight scale per 128 columns
              const float cs = p.sw[(size_t)((n_base + c0 + c) >> 7) * p.k_blocks + kb];
              acc[c0 + c] += __uint_as_float(r[c]) * (row_scale * cs);
            }
          }
        }
        tc_fence_before_sync();
        mbar_arrive(&tempty_bar[buf]);
        buf ^= 1;
        if (buf == 0) buf_phase ^= 1;
      }
      if (!ok) break;
      // store
      if (p.k_splits > 1) {                                   // fp32 partial sums [split][token][feature]; bias in the reduction
        float* wsp = p.ws + (size_t)split * (p.transposed ? (size_t)p.N * p.M : (size_t)p.M * p.N);
        if (p.transposed) {                                   // lanes run along features: coalesced
#pragma unroll
          for (int c = 0; c < BN; ++c)
            if (n_base + c < p.N && m < p.M) wsp[(size_t)(n_base + c) * p.M + m] = acc[c];
        } else if (m < p.M) {
#pragma unroll
          for (int c = 0; c < BN; c += 4)
            if (n_base + c < p.N) *reinterpret_cast<float4*>(wsp + (size_t)m * p.N + n_base + c) = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
        }
      } else if (!p.transposed) {
        if (m < p.M) {
          __nv_bfloat16* dst = p.out + (size_t)m * p.ldc + n_base;
#pragma unroll
          for (int c = 0; c < BN; c += 8) {
            if (n_base + c < p.N) {
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = acc[c + i] + (p.bias ? __bfloat162float(p.bias[n_base + c + i]) : 0.f);
              uint4 o;
              o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(dst + c) = o;
            }
          }
        }
      } else {
        const float bias_m = (p.bias && m < p.M) ? __bfloat162float(p.bias[m]) : 0.f;
        const bool odd = lane & 1;
#pragma unroll
        for (int c = 0; c < BN; c += 2) {
          const float own0 = acc[c] + bias_m, own1 = acc[c + 1] + bias_m;
          const float recv = __shfl_xor_sync(0xffffffffu, odd ? own0 : own1, 1);
          const int n = n_base + c + (odd ? 1 : 0);
          const int mm = odd ? m - 1 : m;
          const uint32_t packed = odd ? pack_bf16x2(recv, own1) : pack_bf16x2(own0, recv);
          if (n < p.N && mm < p.M) *reinterpret_cast<uint32_t*>(p.out + (size_t)n * p.ldc + mm) = packed;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tmem_base, S::kTmemCols); }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicCAS(p.status, FLLM_OK, FLLM_ERR_MBAR_TIMEOUT);
}

// out[t][n] = bf16(sum_s ws[s][t][n] + bias[n])
__global__ void fp8_splitk_reduce_kernel(const float* __restrict__ ws, int splits, int rows, int cols, long long ldc,
                                         const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out) {
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
  uint2 o;
  o.x = pack_bf16x2(acc.x + b[0], acc.y + b[1]);
  o.y = pack_bf16x2(acc.z + b[2], acc.w + b[3]);
  *reinterpret_cast<uint2*>(out + (size_t)r * ldc + c) = o;
}

// x bf16 [T][K] -> e4m3 [T][K] and scales [T][K/128] (amax / 448 per 128 values). One warp per group.
__global__ void quant_fp8_1x128_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ xq,
                                       float* __restrict__ sx, int tokens, int K) {
  const int kb_n = K / 128;
  const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= (long long)tokens * kb_n) return;
  const int t = (int)(gw / kb_n), kb = (int)(gw - (long long)t * kb_n), lane = threadIdx.x & 31;
  const uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)t * ldx + kb * 128 + lane * 4);
  const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-10f) / 448.f, inv = 1.f / scale;
  __nv_fp8x4_e4m3 q(make_float4(a.x * inv, a.y * inv, b.x * inv, b.y * inv));
  *reinterpret_cast<uint32_t*>(xq + (size_t)t * K + kb * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(&q);
  if (lane == 0) sx[(size_t)t * kb_n + kb] = scale;
}

void quant_fp8_1x128(const void* x, long long ldx, void* xq, float* sx, int tokens, int K, cudaStream_t s) {
  if (tokens <= 0) return;
  if (K % 128) throw std::runtime_error("quant_fp8_1x128: K must be a multiple of 128");
  const long long groups = (long long)tokens * (K / 128);
  quant_fp8_1x128_kernel<<<(int)((groups + 7) / 8), 256, 0, s>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)xq, sx, tokens, K);
  cuda_check(cudaGetLastError(), "quant_fp8_1x128_kernel");
}

template <int BN>
static void launch_fp8(const CUtensorMap& ta, const CUtensorMap& tb, const Fp8GemmArgs& a, int grid, cudaStream_t s) {
  using S = Fp8Smem<BN>;
  static bool configured[kMaxDevices] = {};
  if (first_call_on_device(configured)) {
    cuda_check(cudaFuncSetAttribute(gemm_fp8_block_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal),
               "cudaFuncSetAttribute(gemm_fp8_block_kernel)");
  }
  gemm_fp8_block_kernel<BN><<<grid, kF8Threads, S::kTotal, s>>>(ta, tb, a);
  cuda_check(cudaGetLastError(), "gemm_fp8_block_kernel launch");
}

// y[T][N] = dequant(xq, sx) * dequant(wq, sw)^T (+ bias)
int linear_fp8_block(const void* xq, const float* sx, const void* wq, const float* sw, const void* bias, void* y,
                     long long ldy, int T, int N, int K, int* status, cudaStream_t stream, void* workspace,
                     size_t workspace_bytes) {
  if (T <= 0 || N <= 0) return 0;
  if (K % 128 || N % 128) throw std::runtime_error("linear_fp8_block: N and K must be multiples of 128");
  if (K / 128 > 64 * 4) throw std::runtime_error("linear_fp8_block: K above 32768 is not supported");
  Fp8GemmArgs a{};
  a.K = K; a.k_blocks = K / 128;
  a.out = reinterpret_cast<__nv_bfloat16*>(y); a.ldc = ldy;
  a.sx = sx; a.sw = sw; a.bias = reinterpret_cast<const __nv_bfloat16*>(bias); a.status = status;
  const bool swap = T <= 64;                          // decode: features fill the 128-row MMA dimension
  int bn;
  CUtensorMap ta, tb;
  if (swap) {
    bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    a.M = N; a.N = T; a.transposed = 1;
    ta = make_tmap_2d(wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, F8_BM, F8_BK, true);
    tb = make_tmap_2d(xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, T, K, K, bn, F8_BK, true);
  } else {
    bn = 128;
    a.M = T; a.N = N; a.transposed = 0;
    ta = make_tmap_2d(xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, T, K, K, F8_BM, F8_BK, true);
    tb = make_tmap_2d(wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, bn, F8_BK, true);
  }
  a.m_tiles = (a.M + F8_BM - 1) / F8_BM;
  a.n_tiles = (a.N + bn - 1) / bn;
  // Few tiles cannot pull the whole HBM bandwidth: split K until the machine is full. A split's token scales must
  // also fit their shared-memory block (64 K blocks).
  const int slots = sm_count() * (bn <= 64 ? 2 : 1);
  const int tiles = a.m_tiles * a.n_tiles;
  int splits = 1;
  if (tiles * 2 <= slots && a.k_blocks >= 8) splits = std::min(std::min(slots / tiles, a.k_blocks / 4), 16);
  splits = std::max(splits, (a.k_blocks + 63) / 64);
  while (splits > (a.k_blocks + 63) / 64 && (!workspace || (size_t)splits * T * N * 4 > workspace_bytes || (N & 3))) --splits;
  if (splits > 1 && (!workspace || (size_t)splits * T * N * 4 > workspace_bytes || (N & 3)))
    throw std::runtime_error("linear_fp8_block: K above 8192 needs a split-K workspace");
  a.kb_per_split = (a.k_blocks + splits - 1) / splits;
  a.k_splits = (a.k_blocks + a.kb_per_split - 1) / a.kb_per_split;
  a.ws = reinterpret_cast<float*>(workspace);
  const int grid = std::min(tiles * a.k_splits, slots);
  switch (bn) {
    case 16: launch_fp8<16>(ta, tb, a, grid, stream); break;
    case 32: launch_fp8<32>(ta, tb, a, grid, stream); break;
    case 64: launch_fp8<64>(ta, tb, a, grid, stream); break;
    default: launch_fp8<128>(ta, tb, a, grid, stream); break;
  }
  if (a.k_splits > 1) {
    const size_t n = (size_t)T * N;
    fp8_splitk_reduce_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, stream>>>(a.ws, a.k_splits, T, N, ldy, a.bias, a.out);
    cuda_check(cudaGetLastError(), "fp8_splitk_reduce_kernel");
    return 2;
  }
  return 1;
}

}  // namespace fllm
