// Dense bf16 GEMM on the 5th-generation tensor cores:  D[M,N] = A[M,K] * B[N,K]^T
//
//   * both operands are K-major (row-major with K contiguous) and are staged into
//     shared memory by TMA with the 128-byte swizzle (no cluster multicast);
//   * one elected thread issues tcgen05.mma (128 x BN x 16 per instruction), the
//     fp32 accumulator lives in TMEM and is double buffered so the epilogue of
//     tile i overlaps the main loop of tile i+1;
//   * warp roles: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
//     warps 2..5 = epilogue (tcgen05.ld -> bf16 -> global);
//   * persistent grid: CTAs walk a linear list of (split, n-tile, m-tile) items.
//
// Output modes
//   row-major   out[m * ldc + n]           (prefill: A = activations, B = weight)
//   transposed  out[n * ldc + m]           (decode "swap-AB": A = weight so that
//                                           the 128-row MMA dimension is filled by
//                                           output features and the few tokens sit
//                                           in the N dimension)
//   split-K     fp32 partial sums in a workspace: for a local output a second small kernel adds
//               them; when the output leaves the GPU (reduce-scatter epilogue) the CTA that arrives
//               last for a tile adds the partial tiles in split order and runs the epilogue itself.
//
// Role in the reference: dense F16/BF16 products go to cuBLASLt for >= 9 tokens
// (rust/engine/cuda/cublaslt_gemm.cu:11-14) and to an mma.sync skinny kernel below
// that (rust/engine/cuda/linear.cu:396-507); here both cases are one tcgen05 kernel.
#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

constexpr int BM = 128;
constexpr int BK = 64;       // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;
constexpr int kMaxTp = 8;
constexpr uint32_t kPeerWaitPolls = 1u << 22;   // bounded: a few seconds with back-off, then give up

__device__ __forceinline__ int rows_owned(int tokens, int rows_per, int rank) {
  const int lo = rank * rows_per;
  return max(0, min(tokens, lo + rows_per) - lo);
}

struct GemmArgs {
  int M, N, K;
  int m_tiles, n_tiles;
  int k_blocks;            // ceil(K / BK)
  int kb_per_split;
  int k_splits;
  int transposed;          // 0: out[m*ldc+n], 1: out[n*ldc+m]
  int cluster_red;         // split-K reduced on chip: the k_splits CTAs of a tile form a thread-block cluster,
                           // park their fp32 tiles in shared memory and each adds a slice through DSMEM
  long long ldc;
  __nv_bfloat16* out;
  float* ws;               // split-K partials, [k_splits][tiles][BN][128] fp32 (tile-local, column-major)
  unsigned int* tile_counters;   // one arrival counter per tile; zero between launches
  int fixup;               // split-K: 1 = last-arriving CTA finishes the tile, 0 = dense partials + reduce kernel
  int glu;                 // gated activation folded into the epilogue: 0 none, 1 SwiGLU, 2 GeGLU (tanh), 3 clamped SwiGLU-OAI
  int glu_pd;              // lane / column distance between a gate row and its up row: 16 (blocks of 16) or 1 (pairs)
  float glu_alpha, glu_limit;
  int vec16;               // 1: output rows are 16-byte aligned (transposed stores use uint4)
  const __nv_bfloat16* bias;  // per output feature (n when row-major, m when transposed)
  int* status;
  // ---- tensor parallel (all null / zero on a single GPU) ----
  // GEMM -> reduce-scatter: token row t belongs to rank t / rows_per; its partial sums are
  // stored straight into that rank's receive buffer [src rank][rows_per][rs_ld] over NVLink,
  // then the rank's flag word for this source is bumped once per epilogue warp per tile.
  __nv_bfloat16* rs_bufs[kMaxTp];
  uint32_t* rs_flags[kMaxTp];
  int tp, my_rank, rows_per;
  int rs_bcast;                 // 1: every rank receives every row (rows_per = row capacity per source)
  long long rs_ld;
  // all-gather -> GEMM: the activation operand lives in a local buffer that peers fill row
  // block by row block; the TMA producer waits for the owning rank's flag before it loads.
  const uint32_t* ag_flags;     // [tp], bumped once per delivered row by the owning rank
  uint32_t* ag_consumed;        // [tp], rows of each source consumed by earlier launches
  int ag_tokens;                // token rows in this step (defines how many rows each rank owns)
  unsigned int* cta_done;       // last-CTA bookkeeping
  // ---- grouped (mixture of experts): swap-AB tiles over a device-built tile list ----
  // The A operand is the stack of expert matrices [experts * g_rows][K]; tile g of the list
  // multiplies expert g_tile_expert[g] with the BN permuted token rows starting at
  // g_tile_row0[g]. The number of tiles is only known on the device.
  const int* g_tile_expert;
  const int* g_tile_row0;
  const int* g_num_tiles;
  int g_rows;                   // output features per expert
};

template <int BN>
struct GemmSmem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // narrow token tiles (decode) keep two CTAs resident per SM so that a tile list
  // that is not a multiple of the SM count still drains evenly; wide tiles own the SM
  static constexpr int kCtasPerSm = BN <= 64 ? 2 : 1;
  static constexpr int kBudget = (BN <= 64 ? 98 : 200) * 1024;
  static constexpr int kStagesRaw = kBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
  static constexpr int kTmemCols = (2 * BN) < 32 ? 32 : (2 * BN);
  static constexpr int kBarBytes = 256;
  static constexpr int kStageOutBytes = 4 * 32 * 32 * 2;   // per-epilogue-warp transpose tile
  static constexpr int kTotal = kStages * kStageBytes + kBarBytes + kStageOutBytes + 1024;  // +1024 alignment slack
};

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, BN <= 64 ? 2 : 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a,
                 const __grid_constant__ CUtensorMap tma_b, const GemmArgs p) {
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * S::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * S::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
  __nv_bfloat16* stage_out = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(bars) + S::kBarBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 128);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, S::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles = p.m_tiles * p.n_tiles;
  const bool grouped = p.g_num_tiles != nullptr;
  // Let the next kernel in the stream start its own prologue now. Everything this kernel reads
  // that a predecessor may have written (activations, tile lists, counters) is touched only after
  // griddepcontrol.wait; weights are static, so their first tiles are requested before the wait.
  pdl_launch_dependents();
  if (grouped) pdl_wait();
  const int total = grouped ? *p.g_num_tiles * p.m_tiles : tiles * p.k_splits;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    int pre = 0;                 // leading k-blocks of the first item whose weight tile is already in flight
    if (lane == 0 && !grouped) {
      const int w = blockIdx.x;
      if (w < total) {
        const int split = p.cluster_red ? w % p.k_splits : w / tiles;
        const int t = p.cluster_red ? w / p.k_splits : w - split * tiles;
        const int n_idx = t / p.m_tiles;
        const int m_idx = t - n_idx * p.m_tiles;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
        pre = min(kb1 - kb0, STAGES);
        for (int i = 0; i < pre; ++i) {
          mbar_expect_tx(&full_bar[i], S::kStageBytes);
          if (p.transposed) tma_load_2d(sA + i * S::kABytes, &tma_a, &full_bar[i], (kb0 + i) * BK, m_idx * BM);
          else tma_load_2d(sB + i * S::kBBytes, &tma_b, &full_bar[i], (kb0 + i) * BK, n_idx * BN);
        }
      }
    }
    if (!grouped) pdl_wait();
    uint32_t arrived = 0;        // bit s: rank s delivered all of its rows of the gathered operand
    if (p.ag_flags && p.transposed) {
      // decode orientation: every tile needs every rank's rows, so the whole warp polls the
      // arrival counters at once (one lane per source rank) instead of one after the other
      bool mine_ok = true;
      if (lane < p.tp) {
        const int rows = rows_owned(p.ag_tokens, p.rows_per, lane);
        if (rows > 0) mine_ok = wait_flag_ge(p.ag_flags + lane, p.ag_consumed[lane] + (uint32_t)rows, kPeerWaitPolls);
      }
      if (!__all_sync(0xffffffffu, mine_ok)) {
        if (lane == 0) {
          if (p.status) atomicCAS(p.status, FLLM_OK, FLLM_ERR_PEER_TIMEOUT);
          *abort_flag = 1;
        }
      }
      arrived = 0xffffffffu;
      asm volatile("fence.proxy.async;" ::: "memory");
      __syncwarp();
    }
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = *abort_flag == 0;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const int split = p.cluster_red ? w % p.k_splits : w / tiles;
        const int t = p.cluster_red ? w / p.k_splits : w - split * tiles;
        const int n_idx = t / p.m_tiles;
        const int m_idx = t - n_idx * p.m_tiles;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
        if (p.ag_flags) {
          // token rows this tile reads: all of them when tokens sit in the N dimension
          const int t_lo = p.transposed ? n_idx * BN : m_idx * BM;
          const int t_hi = min(p.ag_tokens, t_lo + (p.transposed ? BN : BM));
          if (t_hi > t_lo) {
            for (int s = t_lo / p.rows_per; s <= (t_hi - 1) / p.rows_per && ok; ++s) {
              if (arrived & (1u << s)) continue;
              const uint32_t target = p.ag_consumed[s] + (uint32_t)rows_owned(p.ag_tokens, p.rows_per, s);
              if (!wait_flag_ge(p.ag_flags + s, target, kPeerWaitPolls)) {
                if (p.status) atomicExch(p.status, FLLM_ERR_PEER_TIMEOUT);
                *abort_flag = 1;
                ok = false;
              }
              arrived |= 1u << s;
            }
            // rows were written by peers through the generic proxy; TMA reads them through the async proxy
            asm volatile("fence.proxy.async;" ::: "memory");
          }
          if (!ok) break;
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          const bool prefetched = w == (int)blockIdx.x && kb - kb0 < pre;   // weight half already requested
          if (!prefetched) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
            mbar_expect_tx(&full_bar[stage], S::kStageBytes);
          }
          const int a_row = grouped ? p.g_tile_expert[n_idx] * p.g_rows + m_idx * BM : m_idx * BM;
          const int b_row = grouped ? p.g_tile_row0[n_idx] : n_idx * BN;
          if (!(prefetched && p.transposed))
            tma_load_2d(sA + stage * S::kABytes, &tma_a, &full_bar[stage], kb * BK, a_row);
          if (!(prefetched && !p.transposed))
            tma_load_2d(sB + stage * S::kBBytes, &tma_b, &full_bar[stage], kb * BK, b_row);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const int split = p.cluster_red ? w % p.k_splits : w / tiles;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t da = make_smem_desc_sw128(smem_u32(sA + stage * S::kABytes));
          const uint64_t db = make_smem_desc_sw128(smem_u32(sB + stage * S::kBBytes));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing 16 bf16 = 32 bytes inside the swizzle row: +2 in 16-byte units
            tc_mma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    if (!grouped) pdl_wait();  // outputs and workspaces may still be in use by the predecessor
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
      const int split = p.cluster_red ? w % p.k_splits : w / tiles;
      const int t = p.cluster_red ? w / p.k_splits : w - split * tiles;
      const int n_idx = t / p.m_tiles;
      const int m_idx = t - n_idx * p.m_tiles;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int m = m_idx * BM + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      constexpr int CH = BN < 32 ? 16 : 32;
      // where the bf16 row of a token goes: the local output, or the owning rank's receive buffer
      const bool rs = p.rs_bufs[0] != nullptr;
      // bcast: every rank receives every row (one-shot all-reduce layout [src][token][hidden]);
      // otherwise a row goes to the single rank that owns it (reduce-scatter layout)
      const int ndst = (rs && p.rs_bcast) ? p.tp : 1;
      auto row_ptr = [&](int token, int d) -> __nv_bfloat16* {
        if (!rs) return p.out + (size_t)token * p.ldc;
        if (p.rs_bcast) {
          const int dst = (p.my_rank + d) % p.tp;      // stagger destinations across ranks
          return p.rs_bufs[dst] + ((size_t)p.my_rank * p.rows_per + token) * p.rs_ld;
        }
        const int owner = token / p.rows_per;
        return p.rs_bufs[owner] + ((size_t)p.my_rank * p.rows_per + (token - owner * p.rows_per)) * p.rs_ld;
      };
      const int n_base = grouped ? p.g_tile_row0[n_idx] : n_idx * BN;
      const float bias_m = (p.transposed && p.bias && m < p.M)
                               ? __bfloat162float(p.bias[grouped ? p.g_tile_expert[n_idx] * p.g_rows + m : m])
                               : 0.f;
      __nv_bfloat16* stg = stage_out + (warp - 2) * (32 * 32);
      // gated activation of one (gate, up) pair
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
      // final values of CH columns of this thread's row -> bias, (activation,) bf16, memory
      auto emit = [&](int c0, const float (&v)[32]) {
        const int n0 = n_base + c0;
        if (!p.transposed && p.glu) {
          // features run along the columns: a 32-column chunk holds 16 (gate, up) pairs of this token
          if (m < p.M && n0 < p.N) {
            float o16[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int gi = p.glu_pd == 16 ? i : 2 * i, ui = p.glu_pd == 16 ? i + 16 : 2 * i + 1;
              float g = v[gi], u = v[ui];
              if (p.bias) {
                g += __bfloat162float(p.bias[n0 + gi]);
                u += __bfloat162float(p.bias[n0 + ui]);
              }
              o16[i] = gated(g, u);
            }
            uint4 o0, o1;
            o0.x = pack_bf16x2(o16[0], o16[1]);   o0.y = pack_bf16x2(o16[2], o16[3]);
            o0.z = pack_bf16x2(o16[4], o16[5]);   o0.w = pack_bf16x2(o16[6], o16[7]);
            o1.x = pack_bf16x2(o16[8], o16[9]);   o1.y = pack_bf16x2(o16[10], o16[11]);
            o1.z = pack_bf16x2(o16[12], o16[13]); o1.w = pack_bf16x2(o16[14], o16[15]);
            __nv_bfloat16* dst = row_ptr(m, 0) + n0 / 2;
            reinterpret_cast<uint4*>(dst)[0] = o0;
            reinterpret_cast<uint4*>(dst)[1] = o1;
          }
        } else if (!p.transposed) {
          if (m < p.M) {
#pragma unroll
            for (int c = 0; c < CH; c += 8) {
              if (n0 + c < p.N) {
                float o8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o8[i] = v[c + i];
                if (p.bias) {
                  const uint4 bb = *reinterpret_cast<const uint4*>(p.bias + n0 + c);
                  const uint32_t bw[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const float2 f = unpack_bf16x2(bw[i]);
                    o8[2 * i] += f.x;
                    o8[2 * i + 1] += f.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(o8[0], o8[1]);
                o.y = pack_bf16x2(o8[2], o8[3]);
                o.z = pack_bf16x2(o8[4], o8[5]);
                o.w = pack_bf16x2(o8[6], o8[7]);
                for (int d = 0; d < ndst; ++d) *reinterpret_cast<uint4*>(row_ptr(m, d) + n0 + c) = o;
              }
            }
          }
        } else if (p.glu) {
          // Features run along the lanes: the lane that holds a gate row and the lane that holds its up
          // row (distance glu_pd) trade one value per pair of token columns, so that each computes the
          // activation of ONE of the two columns; the warp's 16 output features of every token are then
          // staged and leave as 16-byte stores (two lanes per token).
          const bool hi = (lane & p.glu_pd) != 0;                 // this lane holds up rows
          const int fl = p.glu_pd == 16 ? (lane & 15) : (lane >> 1);  // output feature within the warp's 16
#pragma unroll
          for (int c = 0; c < CH; c += 2) {
            const float a0 = v[c] + bias_m, a1 = v[c + 1] + bias_m;
            const float recv = __shfl_xor_sync(0xffffffffu, hi ? a0 : a1, p.glu_pd);
            const float g = hi ? recv : a0, u = hi ? a1 : recv;
            stg[(c + (hi ? 1 : 0)) * 16 + fl] = __float2bfloat16(gated(g, u));
          }
          __syncwarp();
          const int f0 = 8 * (lane & 1);
          const int fo = (m_idx * BM + q * 32) / 2 + f0;          // first of 8 output features
#pragma unroll
          for (int rnd = 0; rnd < CH / 16; ++rnd) {
            const int c = (lane >> 1) + 16 * rnd;
            const int n = n0 + c;
            if (n < p.N && 2 * fo < p.M) {
              const uint4 val = *reinterpret_cast<const uint4*>(stg + c * 16 + f0);
              __nv_bfloat16* dst = row_ptr(n, 0) + fo;
              if (p.vec16) {
                *reinterpret_cast<uint4*>(dst) = val;
              } else {
                const uint32_t w4[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) reinterpret_cast<uint32_t*>(dst)[i] = w4[i];
              }
            }
          }
          __syncwarp();
        } else {
          // Transpose through a per-warp staging tile so that every store is 16 bytes: lanes hold
          // features (rows of D), memory wants 8 consecutive features of one token per store. Four
          // lanes then cover the 64 contiguous bytes a token gets from this warp, which matters
          // most when the destination is a peer GPU.
#pragma unroll
          for (int c = 0; c < CH; ++c) stg[c * 32 + lane] = __float2bfloat16(v[c] + bias_m);
          __syncwarp();
          const int f0 = 8 * (lane & 3);
          const int mm0 = m_idx * BM + q * 32 + f0;
#pragma unroll
          for (int rnd = 0; rnd < CH / 8; ++rnd) {
            const int c = (lane >> 2) + 8 * rnd;
            const int n = n0 + c;
            if (n < p.N && mm0 < p.M) {
              const uint4 val = *reinterpret_cast<const uint4*>(stg + c * 32 + f0);
              for (int d = 0; d < ndst; ++d) {
                __nv_bfloat16* dst = row_ptr(n, d) + mm0;
                if (p.vec16) {
                  *reinterpret_cast<uint4*>(dst) = val;
                } else {
                  const uint32_t w4[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
                  for (int i = 0; i < 4; ++i) reinterpret_cast<uint32_t*>(dst)[i] = w4[i];
                }
              }
            }
          }
          __syncwarp();
        }
      };
      auto load_chunk = [&](int c0, float (&v)[32]) {
        uint32_t r[32];
        if constexpr (CH == 32) {
          tmem_ld_32x32(t_row + c0, r);
        } else {
          uint32_t r16[16];
          tmem_ld_32x16(t_row + c0, r16);
#pragma unroll
          for (int i = 0; i < 16; ++i) { r[i] = r16[i]; r[i + 16] = 0; }
        }
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
      };
      bool emitted = true;       // false for split-K CTAs that were not the last to arrive
      if (p.k_splits == 1) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CH) {
          float v[32];
          load_chunk(c0, v);
          emit(c0, v);
        }
        tc_fence_before_sync();
        mbar_arrive(&tempty_bar[acc]);
      } else if (p.cluster_red) {
        // split-K inside a cluster: park the fp32 tile ([token column][feature row], lanes contiguous) in
        // the operand ring, which is idle once this CTA's only accumulator is complete; the cluster
        // adds the tiles after the barrier at the end of the kernel
        float* red = reinterpret_cast<float*>(smem);
        emitted = false;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CH) {
          float v[32];
          load_chunk(c0, v);
#pragma unroll
          for (int c = 0; c < CH; ++c) red[(c0 + c) * BM + q * 32 + lane] = v[c];
        }
        tc_fence_before_sync();
        mbar_arrive(&tempty_bar[acc]);
      } else if (!p.fixup) {
        // split-K, local output: dense fp32 partials [split][token][feature]; a second kernel adds them
        float* wsp = p.ws + (size_t)split * p.M * p.N;
        emitted = false;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CH) {
          float v[32];
          load_chunk(c0, v);
          const int n0 = n_base + c0;
          if (m < p.M) {
            if (!p.transposed) {
#pragma unroll
              for (int c = 0; c < CH; c += 4)
                if (n0 + c < p.N)
                  *reinterpret_cast<float4*>(wsp + (size_t)m * p.N + n0 + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
            } else {
#pragma unroll
              for (int c = 0; c < CH; ++c)
                if (n0 + c < p.N) wsp[(size_t)(n0 + c) * p.M + m] = v[c];
            }
          }
        }
        tc_fence_before_sync();
        mbar_arrive(&tempty_bar[acc]);
      } else {
        // split-K with a remote destination: park this split's fp32 tile ([column][row], lanes
        // contiguous), then the CTA that arrives last for the tile adds the splits in split order
        // and finishes the tile (so partial sums leave the GPU once, already reduced over K).
        const int row_l = q * 32 + lane;
        float* mine = p.ws + ((size_t)split * tiles + t) * (BM * BN);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CH) {
          float v[32];
          load_chunk(c0, v);
#pragma unroll
          for (int c = 0; c < CH; ++c) mine[(size_t)(c0 + c) * BM + row_l] = v[c];
        }
        tc_fence_before_sync();
        mbar_arrive(&tempty_bar[acc]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          const unsigned int old = atomicAdd(p.tile_counters + t, 1u);
          const int last = old == (unsigned int)(p.k_splits - 1);
          if (last) p.tile_counters[t] = 0;          // ready for the next launch
          *last_flag = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        emitted = *last_flag != 0;
        if (emitted) {
          __threadfence();
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += CH) {
            float v[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) v[c] = 0.f;
            // 2 splits x 16 columns of independent loads per round keep L2 latency off the critical path
#pragma unroll 1
            for (int h = 0; h < CH; h += 16) {
              for (int sp0 = 0; sp0 < p.k_splits; sp0 += 2) {
                float tv[2][16];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                  const int sp = min(sp0 + j, p.k_splits - 1);
                  const float* src = p.ws + ((size_t)sp * tiles + t) * (BM * BN) + (size_t)(c0 + h) * BM + row_l;
#pragma unroll
                  for (int c = 0; c < 16; ++c) tv[j][c] = __ldcg(src + (size_t)c * BM);
                }
#pragma unroll
                for (int j = 0; j < 2; ++j)
                  if (sp0 + j < p.k_splits) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) v[h + c] += tv[j][c];
                  }
              }
            }
            emit(c0, v);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // last_flag is reused by the next tile
      }
      if (rs && emitted) {
        // publish this warp's share of the tile: stores -> system fence -> one flag bump per
        // destination rank that owns token rows of the tile
        // One system-scope fence per warp, not per thread: the warp barrier orders the lanes'
        // stores before lane 0's fence, the second barrier orders the fence before the bumps.
        __syncwarp();
        if (lane == 0) __threadfence_system();
        __syncwarp();
        const int tokens = p.transposed ? p.N : p.M;
        const int t_lo = p.transposed ? n_idx * BN : m_idx * BM;
        const int t_hi = min(tokens, t_lo + (p.transposed ? BN : BM));
        if (t_hi > t_lo) {
          // the bump itself can be relaxed, one lane per destination
          const int d = p.rs_bcast ? lane : t_lo / p.rows_per + lane;
          const int d_hi = p.rs_bcast ? p.tp - 1 : (t_hi - 1) / p.rows_per;
          if (d <= d_hi)
            asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(p.rs_flags[d] + p.my_rank) : "memory");
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, S::kTmemCols);
  }
  if (p.cluster_red) {
    // Every thread of every CTA of the cluster comes here (waits that gave up leave their tile
    // unfinished but still arrive), so the hardware barrier cannot be left hanging.
    cluster_sync();
    if (warp >= 2 && !*abort_flag) {
      const int w = blockIdx.x;
      const int t = w / p.k_splits, rank = w % p.k_splits;
      const int n_idx = t / p.m_tiles, m_idx = t - n_idx * p.m_tiles;
      const int tid = threadIdx.x - 64;
      constexpr int kVec = BN * BM / 4;                       // float4 items of the tile
      const int v0 = (int)((long long)kVec * rank / p.k_splits), v1 = (int)((long long)kVec * (rank + 1) / p.k_splits);
      const uint32_t red_local = smem_u32(smem);
      for (int i = v0 + tid; i < v1; i += 128) {
        float4 acc4 = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = 0; sp < p.k_splits; ++sp) {              // split order, like the reduction kernel
          const float4 x = ld_dsmem_f4(red_local + (uint32_t)i * 16u, (uint32_t)sp);
          acc4.x += x.x; acc4.y += x.y; acc4.z += x.z; acc4.w += x.w;
        }
        const int c = i / (BM / 4), mrow = m_idx * BM + (i % (BM / 4)) * 4;
        const int n = n_idx * BN + c;
        if (n < p.N && mrow < p.M) {
          if (p.bias) {
            acc4.x += __bfloat162float(p.bias[mrow]);     acc4.y += __bfloat162float(p.bias[mrow + 1]);
            acc4.z += __bfloat162float(p.bias[mrow + 2]); acc4.w += __bfloat162float(p.bias[mrow + 3]);
          }
          uint2 o;
          o.x = pack_bf16x2(acc4.x, acc4.y);
          o.y = pack_bf16x2(acc4.z, acc4.w);
          *reinterpret_cast<uint2*>(p.out + (size_t)n * p.ldc + mrow) = o;
        }
      }
    }
    cluster_sync();                                            // peers may still be reading this CTA's tile
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicCAS(p.status, FLLM_OK, FLLM_ERR_MBAR_TIMEOUT);
  if (threadIdx.x == 0 && p.ag_flags) {
    // the last CTA to leave records that this launch consumed every rank's rows
    __threadfence();
    if (atomicAdd(p.cta_done, 1u) == gridDim.x - 1) {
      for (int s = 0; s < p.tp; ++s) p.ag_consumed[s] += (uint32_t)rows_owned(p.ag_tokens, p.rows_per, s);
      *p.cta_done = 0;
      __threadfence();
    }
  }
}

// out[i] = bf16(sum_s ws[s][i] + bias), i over a dense [rows][cols] array written with pitch ldc.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int splits, int rows, int cols,
                                     long long ldc, const __nv_bfloat16* __restrict__ bias,
                                     __nv_bfloat16* __restrict__ out) {
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
  if (bias) {
    acc.x += __bfloat162float(bias[c]);
    acc.y += __bfloat162float(bias[c + 1]);
    acc.z += __bfloat162float(bias[c + 2]);
    acc.w += __bfloat162float(bias[c + 3]);
  }
  uint2 o;
  o.x = pack_bf16x2(acc.x, acc.y);
  o.y = pack_bf16x2(acc.z, acc.w);
  *reinterpret_cast<uint2*>(out + (size_t)r * ldc + c) = o;
}

// Split-K reduction whose result leaves the GPU: out[token][feature] (bf16) is stored into the
// receive buffer of EVERY rank (one-shot all-reduce layout [src][token][hidden]) and each CTA then
// bumps every rank's arrival counter once. Many CTAs push at the same time, so the NVLink stores
// of a small decode step are spread over the whole machine instead of a few epilogue warps.
struct ReducePushArgs {
  __nv_bfloat16* rs_bufs[kMaxTp];
  uint32_t* rs_flags[kMaxTp];
  int tp, my_rank, rows_cap;
  long long rs_ld;
};

__global__ void __launch_bounds__(256)
splitk_reduce_push_kernel(const float* __restrict__ ws, int splits, int rows, int cols,
                          const __nv_bfloat16* __restrict__ bias, const ReducePushArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t n = (size_t)rows * cols;
  const size_t i4 = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 < n) {
    float4 acc = __ldcg(reinterpret_cast<const float4*>(ws + i4));
    for (int s = 1; s < splits; ++s) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(ws + (size_t)s * n + i4));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const int r = (int)(i4 / cols);
    const int c = (int)(i4 - (size_t)r * cols);
    if (bias) {
      acc.x += __bfloat162float(bias[c]);
      acc.y += __bfloat162float(bias[c + 1]);
      acc.z += __bfloat162float(bias[c + 2]);
      acc.w += __bfloat162float(bias[c + 3]);
    }
    uint2 o;
    o.x = pack_bf16x2(acc.x, acc.y);
    o.y = pack_bf16x2(acc.z, acc.w);
    for (int d = 0; d < a.tp; ++d) {
      const int dst = (a.my_rank + d) % a.tp;
      *reinterpret_cast<uint2*>(a.rs_bufs[dst] + ((size_t)a.my_rank * a.rows_cap + r) * a.rs_ld + c) = o;
    }
  }
  __syncthreads();                       // all stores of the CTA precede the fences below
  if (threadIdx.x < a.tp) {
    __threadfence_system();
    asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(a.rs_flags[threadIdx.x] + a.my_rank) : "memory");
  }
}

// FLLM_CLUSTER_SPLITK=1 reduces split-K on chip (cluster + distributed shared memory) instead of through
// partial sums in global memory + a reduction kernel. Off by default: measured on B200 it gains ~1 us on
// the 32-tile projections but clusters of 6-8 CTAs do not all fit the GPCs at once for 48 tiles
// (34.8 vs 25.6 us), and a cluster launch waits for whole-GPC room, which costs the overlap between
// consecutive kernels of a decode step (6.28 vs 5.66 ms per step).
static bool cluster_splitk_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("FLLM_CLUSTER_SPLITK");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

// Function attributes are per device: a process that drives several GPUs configures each once.
template <int BN>
static void configure_gemm() {
  using S = GemmSmem<BN>;
  static bool configured[kMaxDevices] = {};
  if (!first_call_on_device(configured)) return;
  cuda_check(cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal),
             "cudaFuncSetAttribute(gemm_bf16_kernel)");
  // ask for the largest shared-memory carve-out: the narrow decode tiles rely on two CTAs per SM
  cuda_check(cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                  cudaSharedmemCarveoutMaxShared),
             "cudaFuncSetAttribute(carveout)");
}

// Everything the GEMM does once per device (loading its modules, setting the attributes of every tile
// width), so that a host can pay for it at start-up instead of inside its first request.
void gemm_bf16_prepare_device() {
  configure_gemm<16>();
  configure_gemm<32>();
  configure_gemm<64>();
  configure_gemm<128>();
  configure_gemm<256>();
}

template <int BN>
static void launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a, int grid,
                        cudaStream_t stream) {
  using S = GemmSmem<BN>;
  configure_gemm<BN>();
  if (a.cluster_red)
    launch_pdl_cluster(gemm_bf16_kernel<BN>, dim3(grid), dim3(kGemmThreads), S::kTotal, stream, (unsigned)a.k_splits, ta,
                       tb, a);
  else
    launch_pdl(gemm_bf16_kernel<BN>, dim3(grid), dim3(kGemmThreads), S::kTotal, stream, ta, tb, a);
}

// Resident CTAs per SM of the GEMM kernel for a token-tile width (diagnostics).
int gemm_bf16_occupancy(int bn) {
  int n = 0;
#define FLLM_OCC(B) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemm_bf16_kernel<B>, kGemmThreads, GemmSmem<B>::kTotal)
  switch (bn) {
    case 16: cudaFuncSetAttribute(gemm_bf16_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<16>::kTotal); FLLM_OCC(16); break;
    case 32: cudaFuncSetAttribute(gemm_bf16_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<32>::kTotal); FLLM_OCC(32); break;
    case 64: cudaFuncSetAttribute(gemm_bf16_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<64>::kTotal); FLLM_OCC(64); break;
    case 128: cudaFuncSetAttribute(gemm_bf16_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<128>::kTotal); FLLM_OCC(128); break;
    default: cudaFuncSetAttribute(gemm_bf16_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<256>::kTotal); FLLM_OCC(256); break;
  }
#undef FLLM_OCC
  return n;
}

size_t gemm_bf16_workspace_bytes(int tokens, int features) {
  // counters + upper bound of 16 splits of fp32 tiles padded to the tile grid
  const size_t t = (size_t)((tokens + 15) / 16 * 16), f = (size_t)((features + BM - 1) / BM * BM);
  return 64 * 1024 + (size_t)16 * t * f * sizeof(float);
}

static int glu_pd_ok(int pd) { return pd == 1 || pd == 16; }

static int pick_bn_tokens(int t) {
  if (t <= 16) return 16;
  if (t <= 32) return 32;
  if (t <= 64) return 64;
  if (t <= 128) return 128;
  return 256;
}

// Tile plan of a linear layer: tokens <= 128 put the weight in the 128-row MMA dimension
// ("swap-AB") and the tokens in a narrow N tile; larger batches use the usual orientation.
static void plan_linear(int T, int N, int sms, bool* swap, int* bn) {
  *swap = T <= 128;
  if (*swap) {
    *bn = pick_bn_tokens(T);
  } else {
    *bn = N >= 256 * 64 || (N % 256 == 0 && ((T + BM - 1) / BM) * (N / 256) >= sms) ? 256 : 128;
    if (N < 128) *bn = 64;
  }
}

// Flag bumps rank `dest` receives from EACH source rank for one reduce-scatter linear of this
// shape: 4 epilogue warps x feature tiles x token tiles that overlap the rows `dest` owns.
int linear_rs_expected_signals(int T, int N, int rows_per, int dest) {
  bool swap;
  int bn;
  plan_linear(T, N, sm_count(), &swap, &bn);
  const int tok_tile = swap ? bn : BM;
  const int feat_tiles = swap ? (N + BM - 1) / BM : (N + bn - 1) / bn;
  const int lo = dest * rows_per, hi = min(T, lo + rows_per);
  if (hi <= lo) return 0;
  const int overlapping = (hi - 1) / tok_tile - lo / tok_tile + 1;
  return 4 * overlapping * feat_tiles;
}

// y[T, N] = x[T, K] * w[N, K]^T (+ bias[N]);  x row pitch ldx, y row pitch ldy (elements).
int linear_bf16(const void* x, long long ldx, const void* w, long long ldw, const void* bias,
                 void* y, long long ldy, int T, int N, int K, void* workspace,
                 size_t workspace_bytes, int* status, int force_splits, cudaStream_t stream, LinearExtras* ex) {
  return linear_bf16_tp(x, ldx, w, ldw, bias, y, ldy, T, N, K, workspace, workspace_bytes, status,
                        force_splits, nullptr, stream, ex);
}

int linear_bf16_tp(const void* x, long long ldx, const void* w, long long ldw, const void* bias,
                   void* y, long long ldy, int T, int N, int K, void* workspace,
                   size_t workspace_bytes, int* status, int force_splits, const TpLinearArgs* tpa,
                   cudaStream_t stream, LinearExtras* ex) {
  if (ex) ex->deferred_splits = 0;
  if (T <= 0 || N <= 0) return 0;
  const int glu = ex ? ex->glu : 0;
  const bool defer = ex && ex->defer_reduce;
  if (glu && ((N & 31) || (tpa && tpa->rs_bufs[0]) || (glu_pd_ok(ex->glu_pd) == 0)))
    throw std::runtime_error("linear_bf16: a gated epilogue needs N % 32 == 0, a local output and a pair distance of 1 or 16");
  if ((K & 7) || (N & 7) || (ldx & 7) || (ldw & 7) || (ldy & 1))
    throw std::runtime_error("linear_bf16: K, N and the row pitches must be multiples of 8");
  const int sms = sm_count();
  // Large local products go to the CTA-pair kernel (cta_group::2, 256 x 256 tiles) once its tiles fill the machine.
  if (!tpa && force_splits <= 0 && (ldy & 7) == 0 && linear_bf16_pair_supported(T, N, K) &&
      (long long)((T + 255) / 256) * ((N + 255) / 256) >= sms / 2)
    return linear_bf16_pair(x, ldx, w, ldw, bias, y, ldy, T, N, K, status, stream, glu ? ex : nullptr);
  GemmArgs a{};
  a.K = K;
  a.k_blocks = (K + BK - 1) / BK;
  a.out = reinterpret_cast<__nv_bfloat16*>(y);
  a.ldc = ldy;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.status = status;
  a.ws = reinterpret_cast<float*>(workspace);
  const bool rs = tpa && tpa->rs_bufs[0];
  if (tpa) {
    if (tpa->tp > kMaxTp) throw std::runtime_error("linear_bf16: tensor-parallel degree above 8");
    a.tp = tpa->tp; a.my_rank = tpa->my_rank; a.rows_per = tpa->rows_per; a.rs_ld = tpa->rs_ld;
    a.rs_bcast = tpa->rs_bcast;
    for (int i = 0; i < kMaxTp; ++i) {
      a.rs_bufs[i] = reinterpret_cast<__nv_bfloat16*>(tpa->rs_bufs[i]);
      a.rs_flags[i] = tpa->rs_flags[i];
    }
    a.ag_flags = tpa->ag_flags; a.ag_consumed = tpa->ag_consumed; a.cta_done = tpa->cta_done;
    a.ag_tokens = T;
  }

  bool swap;
  int bn;
  plan_linear(T, N, sms, &swap, &bn);
  CUtensorMap ta, tb;
  if (swap) {
    a.M = N;  // MMA rows = output features
    a.N = T;
    a.transposed = 1;
    ta = make_tmap_2d(w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw * 2, BM, BK, true);
    tb = make_tmap_2d(x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, K, ldx * 2, bn, BK, true);
  } else {
    a.M = T;
    a.N = N;
    a.transposed = 0;
    ta = make_tmap_2d(x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, K, ldx * 2, BM, BK, true);
    tb = make_tmap_2d(w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw * 2, bn, BK, true);
  }
  a.m_tiles = (a.M + BM - 1) / BM;
  a.n_tiles = (a.N + bn - 1) / bn;
  const int tiles = a.m_tiles * a.n_tiles;

  // split-K when the tile list cannot fill the machine and K is deep enough
  int splits = 1;
  if (force_splits > 0) {
    splits = force_splits;
  } else if (tiles * 4 <= sms * (bn <= 64 ? 2 : 1) * 3 && a.k_blocks >= 8) {
    // fewer tiles than 3/4 of the resident CTA slots: cut K so that every SM streams weights
    const int slots = sms * (bn <= 64 ? 2 : 1);
    splits = min(min(slots / tiles, a.k_blocks / 4), 16);
  }
  // workspace = [tile counters (kCounterBytes, zero between launches)] [fp32 partial tiles]
  constexpr size_t kCounterBytes = 64 * 1024;
  if (splits > 1 && (!workspace || workspace_bytes <= kCounterBytes || (size_t)tiles * 4 > kCounterBytes || bn > 128))
    splits = 1;
  while (splits > 1 && kCounterBytes + (size_t)splits * tiles * BM * bn * sizeof(float) > workspace_bytes) --splits;
  // A gated epilogue needs complete sums: no split-K, unless the caller takes the fp32 partials and
  // applies the activation while it adds them.
  if (glu && splits > 1 && !defer) splits = 1;
  // Broadcast destination + split-K: the GEMM keeps its fast local split path and the reduction
  // kernel does the pushing. Scatter destination + split-K: the last-arriving CTA finishes the tile.
  const bool push_reduce = rs && tpa->rs_bcast && splits > 1;
  a.fixup = (rs && !push_reduce) ? 1 : 0;
  if (a.fixup && force_splits <= 0) splits = min(splits, max(1, min(4, a.k_blocks / 8)));   // the in-kernel fixup is serial per tile: keep it short
  if (!a.fixup)
    while (splits > 1 && kCounterBytes + (size_t)splits * a.M * a.N * sizeof(float) > workspace_bytes) --splits;
  // On-chip reduction: the splits of a tile run as one thread-block cluster (at most 8 CTAs, one unit
  // per CTA) and add their tiles through distributed shared memory: no partial sums in global memory
  // and no second kernel. Decode orientation with a local output only.
  const int slots_now = sms * (bn <= 64 ? 2 : 1);
  bool cluster = cluster_splitk_enabled() && !defer && !glu && swap && !rs && splits > 1 && bn <= 128 && (N % 4) == 0 &&
                 (ldy % 4) == 0 && (reinterpret_cast<uintptr_t>(y) % 8) == 0;
  if (cluster && splits > 8) splits = 8;
  a.kb_per_split = (a.k_blocks + splits - 1) / splits;
  a.k_splits = (a.k_blocks + a.kb_per_split - 1) / a.kb_per_split;
  if (cluster && (a.k_splits < 2 || tiles * a.k_splits > slots_now)) cluster = false;
  a.cluster_red = cluster ? 1 : 0;
  a.tile_counters = reinterpret_cast<unsigned int*>(workspace);
  a.ws = a.k_splits > 1 ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + kCounterBytes) : nullptr;
  // 16-byte stores of the transposed epilogue need 16-byte aligned token rows
  a.vec16 = rs ? ((a.rs_ld & 7) == 0)
               : ((ldy & 7) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0);
  if (glu && a.k_splits == 1) {
    a.glu = glu; a.glu_pd = ex->glu_pd; a.glu_alpha = ex->glu_alpha; a.glu_limit = ex->glu_limit;
    if (!swap && ((ldy & 7) || (reinterpret_cast<uintptr_t>(y) & 15)))
      throw std::runtime_error("linear_bf16: the gated epilogue stores 16 bytes at a time; y must be 16-byte aligned");
  }

  const bool push = push_reduce && a.k_splits > 1;
  if (push) {                      // the GEMM itself writes local partials only
    for (int i = 0; i < kMaxTp; ++i) { a.rs_bufs[i] = nullptr; a.rs_flags[i] = nullptr; }
  }
  if (tpa && tpa->expected_out) {
    if (push) *tpa->expected_out = (int)(((size_t)T * N / 4 + 255) / 256);
    else if (rs) *tpa->expected_out = linear_rs_expected_signals(T, N, tpa->rs_bcast ? T : tpa->rows_per, tpa->rs_bcast ? 0 : tpa->my_rank);
  }
  const int grid = min(tiles * a.k_splits, sms * (bn <= 64 ? 2 : 1));
  switch (bn) {
    case 16: launch_gemm<16>(ta, tb, a, grid, stream); break;
    case 32: launch_gemm<32>(ta, tb, a, grid, stream); break;
    case 64: launch_gemm<64>(ta, tb, a, grid, stream); break;
    case 128: launch_gemm<128>(ta, tb, a, grid, stream); break;
    default: launch_gemm<256>(ta, tb, a, grid, stream); break;
  }
  if (push) {
    ReducePushArgs ra{};
    for (int i = 0; i < tpa->tp; ++i) {
      ra.rs_bufs[i] = reinterpret_cast<__nv_bfloat16*>(tpa->rs_bufs[i]);
      ra.rs_flags[i] = tpa->rs_flags[i];
    }
    ra.tp = tpa->tp; ra.my_rank = tpa->my_rank; ra.rows_cap = tpa->rows_per; ra.rs_ld = tpa->rs_ld;
    const int blocks = (int)(((size_t)T * N / 4 + 255) / 256);
    launch_pdl(splitk_reduce_push_kernel, dim3(blocks), dim3(256), 0, stream, (const float*)a.ws, a.k_splits, T, N,
               a.bias, ra);
    return 2;
  }
  if (a.cluster_red) return 1;
  if (a.k_splits > 1 && !a.fixup && defer) {
    ex->deferred_splits = a.k_splits;      // the consumer adds the dense [split][token][feature] partials (+ bias)
    return 1;
  }
  if (a.k_splits > 1 && !a.fixup) {
    // dense [token][feature] partials in both orientations
    const size_t n = (size_t)T * N;
    const int threads = 256;
    const int blocks = (int)((n / 4 + threads - 1) / threads);
    splitk_reduce_kernel<<<blocks, threads, 0, stream>>>(a.ws, a.k_splits, T, N, ldy, a.bias, a.out);
    cuda_check(cudaGetLastError(), "splitk_reduce_kernel launch");
    return 2;
  }
  return 1;
}

// Grouped swap-AB linear over a device-built tile list (mixture of experts):
//   y[row, :] = w_stack[expert(row)] * xp[row, :] (+ bias_stack[expert(row)])
// for the permuted, per-expert padded rows of xp. `bn` is the token-tile width the tile list was
// built for; `max_tiles` bounds the list (the real count is read on the device).
int moe_grouped_linear_bf16(const void* xp, long long ldx, const void* w_stack, long long ldw,
                            const void* bias_stack, void* y, long long ldy, int rows_cap, int n_out, int K,
                            int experts, const int* tile_expert, const int* tile_row0, const int* num_tiles,
                            int max_tiles, int bn, int* status, cudaStream_t stream) {
  if (rows_cap <= 0 || max_tiles <= 0) return 0;
  if ((K & 7) || (n_out & 7) || (ldx & 7) || (ldw & 7) || (ldy & 1))
    throw std::runtime_error("moe_grouped_linear_bf16: K, n_out and the row pitches must be multiples of 8");
  GemmArgs a{};
  a.K = K;
  a.k_blocks = (K + BK - 1) / BK;
  a.kb_per_split = a.k_blocks;
  a.k_splits = 1;
  a.out = reinterpret_cast<__nv_bfloat16*>(y);
  a.ldc = ldy;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias_stack);
  a.status = status;
  a.M = n_out;
  a.N = rows_cap;
  a.transposed = 1;
  a.m_tiles = (n_out + BM - 1) / BM;
  a.n_tiles = max_tiles;
  a.g_tile_expert = tile_expert;
  a.g_tile_row0 = tile_row0;
  a.g_num_tiles = num_tiles;
  a.g_rows = n_out;
  a.vec16 = (ldy & 7) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
  // When n_out is not a multiple of 128 the last feature tile of an expert also reads rows of the
  // next expert's matrix (or zero fill past the stack); the epilogue never stores those rows.
  CUtensorMap ta = make_tmap_2d(w_stack, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)experts * n_out, K,
                                ldw * 2, BM, BK, true);
  CUtensorMap tb = make_tmap_2d(xp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_cap, K, ldx * 2, bn, BK, true);
  const int grid = min(max_tiles * a.m_tiles, sm_count() * (bn <= 64 ? 2 : 1));
  switch (bn) {
    case 16: launch_gemm<16>(ta, tb, a, grid, stream); break;
    case 32: launch_gemm<32>(ta, tb, a, grid, stream); break;
    case 64: launch_gemm<64>(ta, tb, a, grid, stream); break;
    case 128: launch_gemm<128>(ta, tb, a, grid, stream); break;
    default: throw std::runtime_error("moe_grouped_linear_bf16: token tile must be 16, 32, 64 or 128");
  }
  return 1;
}

}  // namespace fllm
