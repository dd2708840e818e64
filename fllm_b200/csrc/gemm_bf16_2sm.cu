// Dense bf16 GEMM for large token counts on CTA pairs (tcgen05 cta_group::2):  y[T, N] = x[T, K] * w[N, K]^T (+ bias)
//
// Two CTAs of a cluster (two SMs) work on one 256 x 256 output tile. Each CTA stages its own 128 token rows
// of x and only its own half (128 feature rows) of the weight tile; one thread of the even CTA issues
// tcgen05.mma.cta_group::2 (256 x 256 x 16 per instruction) and the hardware feeds both tensor cores with
// both halves of the weight tile. Against the one-CTA 128 x 256 tile of gemm_bf16.cu a stage shrinks from
// 48 KB to 32 KB per SM for the same arithmetic, so seven stages instead of four cover the load latency, and
// every weight byte is read from shared memory by one SM instead of two.
//
//   TMA (both CTAs, `.cta_group::2` form: the bytes of both land on the even CTA's barrier; no cluster multicast)
//   -> 128-byte-swizzled ring -> tcgen05.mma.cta_group::2 -> accumulators in both CTAs' tensor memory
//   (128 lanes x 256 columns each, double buffered) -> tcgen05.commit on both CTAs' barriers frees the stage
//   -> four epilogue warps per CTA (tcgen05.ld -> bf16 -> global), which release the accumulator by an
//   arrive on the even CTA's barrier.
//
// Persistent: clusters walk the tile list with the token tile fastest, so the clusters in flight share weight
// tiles through L2. Every wait is bounded and reports through the status word. The reference sends these
// shapes to cuBLASLt (rust/engine/cuda/cublaslt_gemm.cu:11-14).
#include <algorithm>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

constexpr int P2_ROWS = 128;                 // rows of either operand per CTA per stage
constexpr int P2_BK = 64;                    // 64 bf16 = one 128-byte swizzle row
constexpr int P2_TILE = 256;                 // tile edge of the pair (tokens and features)
constexpr int P2_STAGES = 7;
constexpr int kP2Threads = 192;
constexpr int kP2OperandBytes = P2_ROWS * P2_BK * 2;          // 16 KB
constexpr int kP2StageBytes = 2 * kP2OperandBytes;            // x rows + weight rows
constexpr int kP2Smem = P2_STAGES * kP2StageBytes + 256 + 1024;
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;                // shared-window address of the same location in the even CTA

struct Gemm2Args {
  int M, N, K;                               // M = tokens, N = features
  int m_tiles, n_tiles, k_blocks;
  long long ldc;
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;
  int* status;
  int glu;                                   // 0 none; 1 SwiGLU, 2 GeGLU (tanh), 3 clamped SwiGLU-OAI: out is [M, N / 2]
  int glu_pd;                                // distance between a gate column and its up column: 16 (blocks of 16) or 1 (pairs)
  float glu_alpha, glu_limit;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// TMA load whose completion bytes are counted on the even CTA's barrier at the same offset.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint64_t* bar, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar) & kPeerBitMask), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive on the barrier at this offset in both CTAs once every MMA issued so far has retired (issued by the
// even CTA: one commit on its own barrier, one on the odd CTA's through its cluster-window address).
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  const uint32_t own = smem_u32(bar);
  uint32_t peer;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(own), "r"(1u));
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(own) : "memory");
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(peer) : "memory");
}

__device__ __forceinline__ void mbar_arrive_cta(uint64_t* bar, uint32_t cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(cta_rank));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_out, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__global__ void __launch_bounds__(kP2Threads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w, const Gemm2Args p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sX = smem;
  uint8_t* sW = smem + P2_STAGES * kP2OperandBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P2_STAGES * kP2StageBytes);
  uint64_t* full_bar = bars;                         // used in the even CTA: bytes of both CTAs
  uint64_t* empty_bar = bars + P2_STAGES;            // one per CTA: its own stage is free again
  uint64_t* tfull_bar = bars + 2 * P2_STAGES;        // one per CTA: accumulator buffer complete
  uint64_t* tempty_bar = bars + 2 * P2_STAGES + 2;   // used in the even CTA: both epilogues drained the buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P2_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P2_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 8); }   // 4 epilogue warps x 2 CTAs
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tma_x); tma_prefetch_desc(&tma_w); }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, 512); tmem_relinquish_pair(); }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();                                     // the peer's barriers exist before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  const int tiles = p.m_tiles * p.n_tiles;
  const int n_clusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;

  if (warp == 0) {
    if (lane == 0) {
      pdl_wait();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < tiles && ok; t += n_clusters) {
        const int n_idx = t / p.m_tiles, m_idx = t - n_idx * p.m_tiles;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * kP2StageBytes);
          tma_load_2d_pair(sX + stage * kP2OperandBytes, &tma_x, &full_bar[stage], kb * P2_BK,
                           m_idx * P2_TILE + (int)rank * P2_ROWS);
          tma_load_2d_pair(sW + stage * kP2OperandBytes, &tma_w, &full_bar[stage], kb * P2_BK,
                           n_idx * P2_TILE + (int)rank * P2_ROWS);
          if (++stage == P2_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc(P2_TILE, P2_TILE, 1, 1);       // bf16 x bf16, M = 256 over the pair, N = 256
      int stage = 0, buf = 0;
      uint32_t phase = 0, buf_phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < tiles && ok; t += n_clusters) {
        if (!mbar_wait(&tempty_bar[buf], buf_phase ^ 1, abort_flag)) break;
        tc_fence_after_sync();
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t da = make_smem_desc_sw128(smem_u32(sX + stage * kP2OperandBytes));
          const uint64_t db = make_smem_desc_sw128(smem_u32(sW + stage * kP2OperandBytes));
#pragma unroll
          for (int k = 0; k < P2_BK / 16; ++k)
            tc_mma_bf16_pair(tmem_base + buf * P2_TILE, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit_pair(&empty_bar[stage]);
          if (++stage == P2_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit_pair(&tfull_bar[buf]);
        buf ^= 1;
        if (buf == 0) buf_phase ^= 1;
      }
    }
  } else {
    const int q = warp & 3;
    int buf = 0;
    uint32_t buf_phase = 0;
    for (int t = cluster_id; t < tiles; t += n_clusters) {
      const int n_idx = t / p.m_tiles, m_idx = t - n_idx * p.m_tiles;
      if (!mbar_wait(&tfull_bar[buf], buf_phase, abort_flag)) break;
      tc_fence_after_sync();
      const int m = m_idx * P2_TILE + (int)rank * P2_ROWS + q * 32 + lane;
      const int n_base = n_idx * P2_TILE;
      const uint32_t t_row = tmem_base + buf * P2_TILE + ((uint32_t)(q * 32) << 16);
      __nv_bfloat16* dst = p.out + (size_t)m * p.ldc + n_base;
      auto gated = [&](float g, float u) -> float {
        if (p.glu == 1) return g / (1.f + __expf(-g)) * u;
        if (p.glu == 2) {
          const float c = 0.7978845608028654f * (g + 0.044715f * g * g * g);
          return 0.5f * g * (1.f + tanhf(c)) * u;
        }
        const float gg = fminf(g, p.glu_limit);
        const float uu = fminf(fmaxf(u, -p.glu_limit), p.glu_limit);
        return gg / (1.f + __expf(-p.glu_alpha * gg)) * (uu + 1.f);
      };
#pragma unroll 1
      for (int c0 = 0; c0 < P2_TILE; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c0, r);
        tmem_ld_wait();
        if (p.glu) {
          // features run along the columns: a 32-column chunk holds 16 (gate, up) pairs of this token
          const int n0 = n_base + c0;
          if (m < p.M && n0 < p.N) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              float v2[2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int gi = p.glu_pd == 16 ? i + h : 2 * (i + h), ui = p.glu_pd == 16 ? i + h + 16 : 2 * (i + h) + 1;
                float g = __uint_as_float(r[gi]), u = __uint_as_float(r[ui]);
                if (p.bias) {
                  g += __bfloat162float(p.bias[n0 + gi]);
                  u += __bfloat162float(p.bias[n0 + ui]);
                }
                v2[h] = gated(g, u);
              }
              o[i >> 1] = pack_bf16x2(v2[0], v2[1]);
            }
            uint4* d4 = reinterpret_cast<uint4*>(p.out + (size_t)m * p.ldc + n0 / 2);
            d4[0] = make_uint4(o[0], o[1], o[2], o[3]);
            d4[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        } else if (m < p.M) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            const int n = n_base + c0 + c;
            if (n < p.N) {
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[c + i]) + (p.bias ? __bfloat162float(p.bias[n + i]) : 0.f);
              uint4 o;
              o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(dst + c0 + c) = o;
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(&tempty_bar[buf], 0);
      buf ^= 1;
      if (buf == 0) buf_phase ^= 1;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();                                     // nobody frees tensor memory while the peer may still use it
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc_pair(tmem_base, 512); }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicCAS(p.status, FLLM_OK, FLLM_ERR_MBAR_TIMEOUT);
}

bool linear_bf16_pair_supported(int T, int N, int K) { return T >= 256 && N % 8 == 0 && N >= 256 && K % 8 == 0 && K >= P2_BK; }

// y[T, N] = x[T, K] * w[N, K]^T (+ bias[N]); row pitches in elements. With ex->glu the gated activation runs in the
// epilogue and y is [T, N / 2] (N a multiple of 32).
int linear_bf16_pair(const void* x, long long ldx, const void* w, long long ldw, const void* bias, void* y, long long ldy,
                     int T, int N, int K, int* status, cudaStream_t stream, const LinearExtras* ex) {
  if (!linear_bf16_pair_supported(T, N, K)) throw std::runtime_error("linear_bf16_pair: needs >= 256 tokens, N >= 256, N % 8 == 0, K % 8 == 0");
  if ((ldy & 7)) throw std::runtime_error("linear_bf16_pair: output rows must be 16-byte aligned");
  const int glu = ex ? ex->glu : 0;
  if (glu && ((N & 31) || (ex->glu_pd != 16 && ex->glu_pd != 1))) throw std::runtime_error("linear_bf16_pair: GLU needs N % 32 == 0 and a pair distance of 16 or 1");
  Gemm2Args a{};
  if (glu) { a.glu = glu; a.glu_pd = ex->glu_pd; a.glu_alpha = ex->glu_alpha; a.glu_limit = ex->glu_limit; }
  a.M = T; a.N = N; a.K = K;
  a.m_tiles = (T + P2_TILE - 1) / P2_TILE; a.n_tiles = (N + P2_TILE - 1) / P2_TILE; a.k_blocks = (K + P2_BK - 1) / P2_BK;
  a.ldc = ldy; a.out = reinterpret_cast<__nv_bfloat16*>(y); a.bias = reinterpret_cast<const __nv_bfloat16*>(bias); a.status = status;
  const CUtensorMap tx = make_tmap_2d(x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, K, ldx * 2, P2_ROWS, P2_BK, true);
  const CUtensorMap tw = make_tmap_2d(w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw * 2, P2_ROWS, P2_BK, true);
  static bool configured[kMaxDevices] = {};
  if (first_call_on_device(configured))
    cuda_check(cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kP2Smem),
               "cudaFuncSetAttribute(gemm_bf16_pair_kernel)");
  const int clusters = std::min(a.m_tiles * a.n_tiles, sm_count() / 2);
  launch_pdl_cluster(gemm_bf16_pair_kernel, dim3(2 * clusters), dim3(kP2Threads), (size_t)kP2Smem, stream, 2u, tx, tw, a);
  return 1;
}

}  // namespace fllm
