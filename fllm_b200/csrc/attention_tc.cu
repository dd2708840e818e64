// Paged-KV FlashAttention for bf16, in two kernels that share their tile math:
//
//   fa_decode_kernel   one CTA per (kv head, sequence, kv split). The query tile is
//                      the G = hq/hkv heads that share the KV head (times up to
//                      16/G query positions: speculative verify rows), so K/V are read
//                      once for the whole group. Each of the four warps streams its own
//                      16-token pages through a private 3-stage cp.async ring: no CTA
//                      barrier in the main loop. Partial (m, l, O) are merged across
//                      warps in shared memory and across splits by fa_merge_kernel.
//   fa_prefill_kernel  one CTA per (query tile, kv head, sequence): 64 packed rows
//                      (64/G positions x G heads), 64-token K/V tiles double buffered
//                      with cp.async, causal + sliding-window masking.
//
// Both compute S = Q K^T and O += P V with mma.sync.m16n8k16 (bf16 in, fp32 out) from
// XOR-swizzled shared memory via ldmatrix, with an online softmax in the exp2 domain.
// Decode is bandwidth-bound and its query tile has 4 - 16 rows, far from the 128 rows of a
// tcgen05 MMA, so it stays on the register-level MMA path. Prefill steps with a
// group size that divides 128 and at least 128 packed query rows are handed to the tcgen05 /
// tensor-memory kernel of attention_tmem.cu; fa_prefill_kernel serves every other shape.
//
// KV cache layout: [block][kv_head][16][head_dim] bf16 (a head's page is contiguous).
// Reference counterparts: rust/engine/cuda/attention4.cu:275-495 (GQA-sharing decode with
// split-KV and merge), rust/engine/cuda/attention3.cu:57-288 (prefill tiles).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

constexpr int kPage = 16;
constexpr float kLog2e = 1.4426950408889634f;

struct FaParams {
  const __nv_bfloat16* q;
  long long ldq;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_tables;
  int max_blocks;
  const int* q_starts;   // [B+1] first token row of each sequence in the ragged batch
  const int* kv_lens;    // [B] visible KV length after this step (last query position + 1)
  __nv_bfloat16* out;
  long long ldo;
  float* ws_o;           // split partials: [T][hq][splits][D]
  float* ws_ml;          // [T][hq][splits][2]
  const float* sinks;    // [hq] or null
  int hq, hkv, group;
  int splits;
  int window;
  float scale_log2;      // softmax scale * log2(e)
  float softcap;         // 0 = off (applied to scale * s, before the exp)
  float scale;
  int decode_max_q;      // sequences with more query rows than this belong to the prefill kernel
  long long num_kv_blocks;
  int* status;
  int bidir;             // 1: no causal mask (encoders): prefill kernels only
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// F16 selects the element type of the 16-bit operands: bf16 (the cache's own type) or f16 (an e4m3 cache is
// widened to f16, which holds every e4m3 value exactly, with one conversion instruction per pair).
template <bool F16>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (F16) mma_f16(d, a, b0, b1);
  else mma_bf16(d, a, b0, b1);
}
template <bool F16>
__device__ __forceinline__ uint32_t pack_16x2(float lo, float hi) {
  if constexpr (F16) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  } else {
    return pack_bf16x2(lo, hi);
  }
}

// Row-major tile of rows x D bf16 in shared memory; 16-byte chunk c of row r lives at chunk
// index (c ^ (r & 7)) so that ldmatrix row fetches hit distinct banks.
template <int D>
__device__ __forceinline__ __nv_bfloat16* tile_ptr(__nv_bfloat16* base, int row, int chunk) {
  return base + row * D + ((chunk ^ (row & 7)) << 3);
}

// Copy `rows` contiguous rows of D bf16 from global to a swizzled tile, `nthreads` cooperating.
template <int D>
__device__ __forceinline__ void load_rows_async(__nv_bfloat16* tile, int row0, const __nv_bfloat16* src,
                                                int rows, int tid, int nthreads) {
  constexpr int CPR = D / 8;
  for (int i = tid; i < rows * CPR; i += nthreads) {
    const int r = i / CPR, c = i - r * CPR;
    cp_async16(tile_ptr<D>(tile, row0 + r, c), src + (size_t)r * D + c * 8);
  }
}

// S[16 x (8*NB)] += Q[16 x D] * K[tokens x D]^T for the NB token blocks starting at row tok0.
template <int D, int NB, bool F16 = false>
__device__ __forceinline__ void qk_tile(float (&s)[NB][4], const uint32_t (&qf)[D / 16][4],
                                        __nv_bfloat16* ktile, int tok0, int lane) {
  static_assert(NB % 2 == 0, "token blocks are processed in pairs");
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int nb = 0; nb < NB; nb += 2) {
      uint32_t b[4];
      const int j = lane >> 3;
      ldsm_x4(b, tile_ptr<D>(ktile, tok0 + (nb + (j >> 1)) * 8 + (lane & 7), 2 * kk + (j & 1)));
      mma_16816<F16>(s[nb], qf[kk], b[0], b[1]);
      mma_16816<F16>(s[nb + 1], qf[kk], b[2], b[3]);
    }
  }
}

// O[16 x D] += P[16 x (16*KT)] * V[tokens x D] for KT 16-token groups starting at row tok0.
template <int D, int KT, bool F16 = false>
__device__ __forceinline__ void pv_tile(float (&o)[D / 8][4], const uint32_t (&pf)[KT][4],
                                        __nv_bfloat16* vtile, int tok0, int lane) {
#pragma unroll
  for (int kt = 0; kt < KT; ++kt) {
#pragma unroll
    for (int db = 0; db < D / 8; db += 2) {
      uint32_t b[4];
      const int j = lane >> 3;
      ldsm_x4_t(b, tile_ptr<D>(vtile, tok0 + kt * 16 + (j & 1) * 8 + (lane & 7), db + (j >> 1)));
      mma_16816<F16>(o[db], pf[kt], b[0], b[1]);
      mma_16816<F16>(o[db + 1], pf[kt], b[2], b[3]);
    }
  }
}

// Online-softmax update for the two rows (g, g+8) a thread holds. `lim0/lim1` = number of
// visible tokens for each row, `beg0/beg1` = first visible token (sliding window).
template <int NB, int D, bool F16 = false>
__device__ __forceinline__ void softmax_update(float (&s)[NB][4], uint32_t (&pf)[NB / 2][4],
                                               float (&o)[D / 8][4], float (&m)[2], float (&l)[2],
                                               int tok_base, int lane, int lim0, int lim1, int beg0,
                                               int beg1, float scale_log2, float softcap, float scale) {
  const int t = lane & 3;
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int tok = tok_base + nb * 8 + 2 * t + (e & 1);
      const bool hi = e >= 2;
      float v = s[nb][e];
      if (softcap > 0.f) v = softcap * tanhf(v * scale / softcap) * kLog2e;
      else v *= scale_log2;
      const bool ok = hi ? (tok < lim1 && tok >= beg1) : (tok < lim0 && tok >= beg0);
      v = ok ? v : -INFINITY;
      s[nb][e] = v;
      if (hi) mx1 = fmaxf(mx1, v); else mx0 = fmaxf(mx0, v);
    }
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
  const float c0 = mn0 == -INFINITY ? 1.f : exp2f(m[0] - mn0);
  const float c1 = mn1 == -INFINITY ? 1.f : exp2f(m[1] - mn1);
  const float b0 = mn0 == -INFINITY ? 0.f : mn0, b1 = mn1 == -INFINITY ? 0.f : mn1;
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const float p0 = exp2f(s[nb][0] - b0), p1 = exp2f(s[nb][1] - b0);
    const float p2 = exp2f(s[nb][2] - b1), p3 = exp2f(s[nb][3] - b1);
    sum0 += p0 + p1;
    sum1 += p2 + p3;
    pf[nb >> 1][(nb & 1) * 2 + 0] = pack_16x2<F16>(p0, p1);
    pf[nb >> 1][(nb & 1) * 2 + 1] = pack_16x2<F16>(p2, p3);
  }
  l[0] = l[0] * c0 + sum0;
  l[1] = l[1] * c1 + sum1;
  m[0] = mn0;
  m[1] = mn1;
#pragma unroll
  for (int db = 0; db < D / 8; ++db) {
    o[db][0] *= c0; o[db][1] *= c0;
    o[db][2] *= c1; o[db][3] *= c1;
  }
}

// ------------------------------------------------------------------------------ decode
// KV8: the cache holds e4m3 bytes. Pages arrive raw (half the bytes of a bf16 page); the warp that owns a page
// widens it to f16 into a private pair of swizzled tiles right before its MMAs.
template <int D, bool KV8 = false>
struct DecodeSmem {
  static constexpr int kStages = 3;
  static constexpr int kPageElems = kPage * D;
  static constexpr int kQBytes = 16 * D * 2;
  static constexpr int kPageBytes = kPageElems * (KV8 ? 1 : 2);          // one K or V page as it arrives
  static constexpr int kWarpRing = kStages * 2 * kPageBytes;             // stages x (K, V)
  static constexpr int kWarpTiles = KV8 ? 2 * kPageElems * 2 : 0;        // widened K and V tiles
  static constexpr int kRingBytes = 4 * (kWarpRing + kWarpTiles);
  static constexpr int kMergeBytes = 4 * 16 * D * 4 + 4 * 16 * 2 * 4;
  static constexpr int kTotal = kQBytes + (kRingBytes > kMergeBytes ? kRingBytes : kMergeBytes) + 128;
};

template <int D, bool KV8 = false>
__global__ void __launch_bounds__(128) fa_decode_kernel(const FaParams p) {
  using S = DecodeSmem<D, KV8>;
  extern __shared__ __align__(128) uint8_t smem[];
  __nv_bfloat16* qtile = reinterpret_cast<__nv_bfloat16*>(smem);
  uint8_t* ring = smem + S::kQBytes;
  const int kvh = blockIdx.x, seq = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group;
  pdl_launch_dependents();
  pdl_wait();
  const int q0 = p.q_starts[seq];
  const int qn = p.q_starts[seq + 1] - q0;
  if (qn <= 0 || qn > p.decode_max_q) return;
  const int kv_len = p.kv_lens[seq];
  const int n_rows = qn * G;                       // packed rows: r = qi * G + head_in_group
  const int first_pos = kv_len - qn;               // absolute position of query 0

  // visible range over all rows of the tile
  int lo_tok = 0;
  if (p.window > 0) lo_tok = max(0, first_pos - p.window + 1);
  const int page_lo = lo_tok / kPage;
  const int page_hi = (kv_len + kPage - 1) / kPage;
  const int n_pages = page_hi - page_lo;
  const int per_split = (n_pages + p.splits - 1) / p.splits;
  const int pg0 = page_lo + split * per_split;
  const int pg1 = min(pg0 + per_split, page_hi);

  // Q tile -> shared (zero rows beyond n_rows), then fragments
  for (int i = threadIdx.x; i < 16 * (D / 8); i += 128) {
    const int r = i / (D / 8), c = i - r * (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < n_rows) {
      const int qi = r / G, hg = r - qi * G;
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + qi) * p.ldq + (size_t)(kvh * G + hg) * D + c * 8);
      if constexpr (KV8) {                                        // the MMAs run on f16 operands
        uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(w[e]);
          w[e] = pack_16x2<true>(f.x, f.y);
        }
      }
    }
    *reinterpret_cast<uint4*>(tile_ptr<D>(qtile, r, c)) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) ldsm_x4(qf[kk], tile_ptr<D>(qtile, lane & 15, 2 * kk + (lane >> 4)));

  const int g = lane >> 2;
  auto row_limits = [&](int r, int& lim, int& beg) {
    if (r < n_rows) {
      const int qi = r / G;
      lim = first_pos + qi + 1;
      beg = p.window > 0 ? max(0, lim - p.window) : 0;
    } else {
      lim = 0;
      beg = 0;
    }
  };
  int lim0, lim1, beg0, beg1;
  row_limits(g, lim0, beg0);
  row_limits(g + 8, lim1, beg1);

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  uint8_t* my_ring = ring + (size_t)warp * (S::kWarpRing + S::kWarpTiles);
  __nv_bfloat16* my_tiles = reinterpret_cast<__nv_bfloat16*>(my_ring + S::kWarpRing);     // KV8 only
  const int* table = p.block_tables + (size_t)seq * p.max_blocks;
  auto issue = [&](int it) {
    const int pg = pg0 + warp + 4 * it;
    if (pg < pg1) {
      const int blk = table[pg];
      const size_t off = ((size_t)blk * p.hkv + kvh) * S::kPageElems;
      uint8_t* st = my_ring + (size_t)(it % S::kStages) * 2 * S::kPageBytes;
      if constexpr (KV8) {                                        // raw bytes, row-major, no swizzle
        const uint8_t* kg = reinterpret_cast<const uint8_t*>(p.k_cache) + off;
        const uint8_t* vg = reinterpret_cast<const uint8_t*>(p.v_cache) + off;
        for (int i = lane; i < S::kPageBytes / 16; i += 32) {
          cp_async16(st + i * 16, kg + i * 16);
          cp_async16(st + S::kPageBytes + i * 16, vg + i * 16);
        }
      } else {
        __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(st);
        load_rows_async<D>(ks, 0, p.k_cache + off, kPage, lane, 32);
        load_rows_async<D>(ks + S::kPageElems, 0, p.v_cache + off, kPage, lane, 32);
      }
    }
    cp_async_commit();
  };
  const int my_pages = pg1 > pg0 + warp ? (pg1 - pg0 - warp + 3) / 4 : 0;
#pragma unroll
  for (int s = 0; s < S::kStages - 1; ++s) issue(s);
  for (int it = 0; it < my_pages; ++it) {
    issue(it + S::kStages - 1);
    cp_async_wait<S::kStages - 1>();
    __syncwarp();
    uint8_t* st = my_ring + (size_t)(it % S::kStages) * 2 * S::kPageBytes;
    __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(st);
    __nv_bfloat16* vs = ks + S::kPageElems;
    if constexpr (KV8) {
      // widen this page pair: 16 e4m3 bytes -> two 16-byte chunks of f16 in the swizzled tiles
      ks = my_tiles;
      vs = my_tiles + S::kPageElems;
      constexpr int CPR = D / 16;                                 // 16-byte chunks of raw bytes per row
      for (int i = lane; i < 2 * kPage * CPR; i += 32) {
        const int which = i / (kPage * CPR), c16 = i - which * (kPage * CPR);
        const int r = c16 / CPR, cc = c16 - r * CPR;
        const uint4 raw = *reinterpret_cast<const uint4*>(st + which * S::kPageBytes + r * D + cc * 16);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t h[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[e] & 0xFFFFu), __NV_E4M3);
          const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[e] >> 16), __NV_E4M3);
          h[2 * e] = (uint32_t)lo.x | ((uint32_t)lo.y << 16);
          h[2 * e + 1] = (uint32_t)hi.x | ((uint32_t)hi.y << 16);
        }
        __nv_bfloat16* tile = which ? vs : ks;
        *reinterpret_cast<uint4*>(tile_ptr<D>(tile, r, 2 * cc)) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(tile_ptr<D>(tile, r, 2 * cc + 1)) = make_uint4(h[4], h[5], h[6], h[7]);
      }
      __syncwarp();
    }
    const int tok_base = (pg0 + warp + 4 * it) * kPage;
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    qk_tile<D, 2, KV8>(s, qf, ks, 0, lane);
    uint32_t pf[1][4];
    softmax_update<2, D, KV8>(s, pf, o, m, l, tok_base, lane, lim0, lim1, beg0, beg1, p.scale_log2,
                              p.softcap, p.scale);
    pv_tile<D, 1, KV8>(o, pf, vs, 0, lane);
    __syncwarp();
  }
  cp_async_wait<0>();
  // row sums live spread over the quad
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);

  // merge the four warps through shared memory (the ring is free now)
  __syncthreads();
  float* mo = reinterpret_cast<float*>(smem + S::kQBytes);            // [4][16][D]
  float* mml = mo + 4 * 16 * D;                                       // [4][16][2]
  const int t4 = lane & 3;
#pragma unroll
  for (int db = 0; db < D / 8; ++db) {
    float* r0 = mo + ((size_t)warp * 16 + g) * D + db * 8 + 2 * t4;
    float* r1 = mo + ((size_t)warp * 16 + g + 8) * D + db * 8 + 2 * t4;
    r0[0] = o[db][0]; r0[1] = o[db][1];
    r1[0] = o[db][2]; r1[1] = o[db][3];
  }
  if (t4 == 0) {
    mml[(warp * 16 + g) * 2] = m[0];
    mml[(warp * 16 + g) * 2 + 1] = l[0];
    mml[(warp * 16 + g + 8) * 2] = m[1];
    mml[(warp * 16 + g + 8) * 2 + 1] = l[1];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_rows * (D / 2); i += 128) {
    const int r = i / (D / 2), d2 = (i - r * (D / 2)) * 2;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, mml[(w * 16 + r) * 2]);
    float ll = 0.f, a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mml[(w * 16 + r) * 2];
      const float c = mw == -INFINITY ? 0.f : exp2f(mw - mm);
      ll += mml[(w * 16 + r) * 2 + 1] * c;
      a0 += mo[((size_t)w * 16 + r) * D + d2] * c;
      a1 += mo[((size_t)w * 16 + r) * D + d2 + 1] * c;
    }
    const int qi = r / G, hg = r - qi * G;
    const int head = kvh * G + hg;
    const size_t tok = (size_t)(q0 + qi);
    if (p.splits == 1) {
      if (p.sinks) {
        const float sk = p.sinks[head] * kLog2e;
        const float mn = fmaxf(mm, sk);
        const float c = mm == -INFINITY ? 0.f : exp2f(mm - mn);
        ll = ll * c + exp2f(sk - mn);
        a0 *= c;
        a1 *= c;
      }
      const float inv = ll > 0.f ? 1.f / ll : 0.f;
      *reinterpret_cast<uint32_t*>(p.out + tok * p.ldo + (size_t)head * D + d2) = pack_bf16x2(a0 * inv, a1 * inv);
    } else {
      const size_t base = (tok * p.hq + head) * p.splits + split;
      p.ws_o[base * D + d2] = a0;
      p.ws_o[base * D + d2 + 1] = a1;
      if (d2 == 0) {
        p.ws_ml[base * 2] = mm;
        p.ws_ml[base * 2 + 1] = ll;
      }
    }
  }
}

// One warp per (token row, head): combine split partials, add the sink, normalise.
template <int D>
__global__ void __launch_bounds__(128) fa_merge_kernel(const FaParams p, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const int pair = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (pair >= T * p.hq) return;
  const int lane = threadIdx.x & 31;
  const int tok = pair / p.hq, head = pair - tok * p.hq;
  const size_t base = (size_t)pair * p.splits;
  float mm = -INFINITY;
  for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, p.ws_ml[(base + s) * 2]);
  float sk = -INFINITY;
  if (p.sinks) {
    sk = p.sinks[head] * kLog2e;
    mm = fmaxf(mm, sk);
  }
  float ll = p.sinks ? exp2f(sk - mm) : 0.f;
  constexpr int EPL = D / 32;
  float a[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) a[e] = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const float ms = p.ws_ml[(base + s) * 2];
    if (ms == -INFINITY) continue;
    const float w = exp2f(ms - mm);
    ll += p.ws_ml[(base + s) * 2 + 1] * w;
    const float* o = p.ws_o + (base + s) * D;
#pragma unroll
    for (int e = 0; e < EPL; ++e) a[e] += o[lane + 32 * e] * w;
  }
  const float inv = ll > 0.f ? 1.f / ll : 0.f;
  __nv_bfloat16* dst = p.out + (size_t)tok * p.ldo + (size_t)head * D;
#pragma unroll
  for (int e = 0; e < EPL; ++e) dst[lane + 32 * e] = __float2bfloat16(a[e] * inv);
}

// ------------------------------------------------------------------------------ prefill
template <int D, int R = 64>
struct PrefillSmem {
  static constexpr int kRows = R;            // packed query rows per CTA: 16 per warp (64 -> 4 warps, 128 -> 8 warps
                                             // sharing every K/V tile, which halves the K/V traffic per FLOP)
  static constexpr int kThreads = 2 * R;
  static constexpr int kTile = 64;           // KV tokens per tile
  static constexpr int kQBytes = kRows * D * 2;
  static constexpr int kKvBytes = 2 * 2 * kTile * D * 2;   // 2 stages x (K, V)
  static constexpr int kTotal = kQBytes + kKvBytes + 128;
};

template <int D, int R>
__global__ void __launch_bounds__(2 * R) fa_prefill_kernel(const FaParams p) {
  using S = PrefillSmem<D, R>;
  extern __shared__ __align__(128) uint8_t smem[];
  __nv_bfloat16* qtile = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* kv = reinterpret_cast<__nv_bfloat16*>(smem + S::kQBytes);
  const int qt = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group;
  const int RQ = S::kRows / G;                    // query positions per tile
  const int q0 = p.q_starts[seq];
  const int qn = p.q_starts[seq + 1] - q0;
  if (qn <= p.decode_max_q) return;               // decode kernel's share
  const int qi0 = qt * RQ;
  if (qi0 >= qn) return;
  const int nq = min(RQ, qn - qi0);
  const int n_rows = nq * G;
  const int kv_len = p.kv_lens[seq];
  const int first_pos = kv_len - qn + qi0;        // absolute position of the tile's first query
  const int hi_tok = p.bidir ? kv_len : first_pos + nq;              // exclusive
  int lo_tok = 0;
  if (p.window > 0) lo_tok = max(0, first_pos - p.window + 1);
  const int tile_lo = lo_tok / S::kTile;
  const int tile_hi = (hi_tok + S::kTile - 1) / S::kTile;

  for (int i = threadIdx.x; i < S::kRows * (D / 8); i += S::kThreads) {
    const int r = i / (D / 8), c = i - r * (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < n_rows) {
      const int qi = r / G, hg = r - qi * G;
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + qi0 + qi) * p.ldq + (size_t)(kvh * G + hg) * D + c * 8);
    }
    *reinterpret_cast<uint4*>(tile_ptr<D>(qtile, r, c)) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk)
    ldsm_x4(qf[kk], tile_ptr<D>(qtile, warp * 16 + (lane & 15), 2 * kk + (lane >> 4)));

  const int g = lane >> 2;
  auto row_limits = [&](int r, int& lim, int& beg) {
    if (r < n_rows) {
      lim = p.bidir ? kv_len : first_pos + r / G + 1;
      beg = p.window > 0 ? max(0, lim - p.window) : 0;
    } else {
      lim = 0;
      beg = 0;
    }
  };
  int lim0, lim1, beg0, beg1;
  row_limits(warp * 16 + g, lim0, beg0);
  row_limits(warp * 16 + g + 8, lim1, beg1);

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  const int* table = p.block_tables + (size_t)seq * p.max_blocks;
  const int n_pages_total = (kv_len + kPage - 1) / kPage;
  auto issue = [&](int tile) {
    if (tile < tile_hi) {
      __nv_bfloat16* ks = kv + (size_t)(tile & 1) * 2 * S::kTile * D;
      __nv_bfloat16* vs = ks + S::kTile * D;
#pragma unroll
      for (int pg = 0; pg < S::kTile / kPage; ++pg) {
        const int page = tile * (S::kTile / kPage) + pg;
        if (page < n_pages_total) {
          const int blk = table[page];
          const size_t off = ((size_t)blk * p.hkv + kvh) * kPage * D;
          load_rows_async<D>(ks, pg * kPage, p.k_cache + off, kPage, threadIdx.x, S::kThreads);
          load_rows_async<D>(vs, pg * kPage, p.v_cache + off, kPage, threadIdx.x, S::kThreads);
        } else {
          // past the sequence: V rows must be finite because they meet P = 0 in the MMA
          for (int i = threadIdx.x; i < kPage * (D / 8); i += S::kThreads)
            *reinterpret_cast<uint4*>(vs + (size_t)pg * kPage * D + i * 8) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    cp_async_commit();
  };
  issue(tile_lo);
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    issue(tile + 1);
    cp_async_wait<1>();
    __syncthreads();
    __nv_bfloat16* ks = kv + (size_t)(tile & 1) * 2 * S::kTile * D;
    __nv_bfloat16* vs = ks + S::kTile * D;
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    qk_tile<D, 8>(s, qf, ks, 0, lane);
    uint32_t pf[4][4];
    softmax_update<8, D>(s, pf, o, m, l, tile * S::kTile, lane, lim0, lim1, beg0, beg1, p.scale_log2,
                         p.softcap, p.scale);
    pv_tile<D, 4>(o, pf, vs, 0, lane);
    __syncthreads();
  }
  cp_async_wait<0>();
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  const int t4 = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = warp * 16 + g + half * 8;
    if (r >= n_rows) continue;
    const int qi = r / G, hg = r - qi * G;
    const int head = kvh * G + hg;
    float mm = m[half], ll = l[half], c = 1.f;
    if (p.sinks) {
      const float sk = p.sinks[head] * kLog2e;
      const float mn = fmaxf(mm, sk);
      c = mm == -INFINITY ? 0.f : exp2f(mm - mn);
      ll = ll * c + exp2f(sk - mn);
    }
    const float inv = ll > 0.f ? c / ll : 0.f;
    __nv_bfloat16* dst = p.out + (size_t)(q0 + qi0 + qi) * p.ldo + (size_t)head * D;
#pragma unroll
    for (int db = 0; db < D / 8; ++db)
      *reinterpret_cast<uint32_t*>(dst + db * 8 + 2 * t4) =
          pack_bf16x2(o[db][half * 2] * inv, o[db][half * 2 + 1] * inv);
  }
}

// ------------------------------------------------------------------------------ host
size_t attention_tc_workspace_bytes(int tokens, int hq, int head_dim, int max_splits) {
  return (size_t)tokens * hq * max_splits * (head_dim + 2) * sizeof(float);
}

template <int D>
static int launch_tc(FaParams p, int tokens, int num_seqs, int max_q_len, int min_q_len, int max_kv_len,
                     void* workspace, size_t workspace_bytes, cudaStream_t s, bool kv_fp8) {
  static bool configured[kMaxDevices] = {};
  if (first_call_on_device(configured)) {
    cuda_check(cudaFuncSetAttribute(fa_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    DecodeSmem<D>::kTotal), "fa_decode smem");
    cuda_check(cudaFuncSetAttribute(fa_decode_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    DecodeSmem<D, true>::kTotal), "fa_decode (e4m3 cache) smem");
    cuda_check(cudaFuncSetAttribute(fa_prefill_kernel<D, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    PrefillSmem<D, 64>::kTotal), "fa_prefill smem");
  }
  int launches = 0;
  // packed rows must fit one 16-row MMA tile; a bidirectional batch (encoder) goes to the prefill kernels whole
  const int decode_max_q = p.bidir ? 0 : 16 / p.group;
  p.decode_max_q = decode_max_q;
  if (kv_fp8 && (decode_max_q < 1 || max_q_len > decode_max_q))
    throw std::runtime_error("attention_tc: an e4m3 cache is read by the decode kernel only (query rows x group <= 16)");
  if (decode_max_q >= 1 && min_q_len <= decode_max_q) {
    // split the KV range when the grid alone cannot fill the machine
    const int ctas = num_seqs * p.hkv;
    const int pages = (max_kv_len + kPage - 1) / kPage;
    int splits = 1;
    // a grid of at least one CTA per SM streams KV well enough; splitting costs a merge launch
    if (ctas < sm_count()) splits = min(min((2 * sm_count() + ctas - 1) / ctas, (pages + 7) / 8), 32);
    splits = max(splits, 1);
    // partials of prefill sequences do not exist, so a mixed batch is never split
    if (max_q_len > decode_max_q || !workspace) splits = 1;
    while (splits > 1 && attention_tc_workspace_bytes(tokens, p.hq, D, splits) > workspace_bytes) --splits;
    p.splits = splits;
    p.ws_o = reinterpret_cast<float*>(workspace);
    p.ws_ml = p.ws_o ? p.ws_o + (size_t)tokens * p.hq * splits * D : nullptr;
    dim3 grid(p.hkv, num_seqs, splits);
    if (kv_fp8) launch_pdl(fa_decode_kernel<D, true>, grid, dim3(128), DecodeSmem<D, true>::kTotal, s, p);
    else launch_pdl(fa_decode_kernel<D>, grid, dim3(128), DecodeSmem<D>::kTotal, s, p);
    ++launches;
    if (splits > 1) {
      launch_pdl(fa_merge_kernel<D>, dim3((tokens * p.hq + 3) / 4), dim3(128), 0, s, p, tokens);
      ++launches;
    }
  }
  // Prefill tiles of at least 128 packed rows run on tcgen05 with tensor-memory accumulators; FLLM_FA_TMEM=0
  // keeps the mma.sync kernel below for every shape.
  static int use_tmem = -1;
  if (use_tmem < 0) { const char* e = getenv("FLLM_FA_TMEM"); use_tmem = e ? atoi(e) : 1; }
  if (max_q_len > decode_max_q && use_tmem && p.num_kv_blocks > 0 && max_q_len * p.group >= 128 &&
      attention_prefill_tmem_supported(D, p.group, kPage)) {
    attention_prefill_tmem(p.q, p.ldq, p.k_cache, p.v_cache, p.num_kv_blocks, p.block_tables, p.max_blocks, p.q_starts,
                           p.kv_lens, p.out, p.ldo, num_seqs, max_q_len, decode_max_q + 1, p.hq, p.hkv, D, p.scale,
                           p.window, p.sinks, p.softcap, p.status, s, 0, p.bidir);
    ++launches;
  } else if (max_q_len > decode_max_q) {
    // 64 packed rows per CTA. (128 rows, 8 warps sharing every K/V tile, measured equal - 119 vs 121 TFLOP/s at
    // 2 x 1024 tokens: the kernel is bound by the mma.sync / softmax pipeline of each warp, not by K/V traffic.)
    const int rq = 64 / p.group;
    if (rq < 1) throw std::runtime_error("attention_tc: more than 64 query heads per KV head");
    dim3 grid((max_q_len + rq - 1) / rq, p.hkv, num_seqs);
    p.splits = 1;
    fa_prefill_kernel<D, 64><<<grid, 128, PrefillSmem<D, 64>::kTotal, s>>>(p);
    ++launches;
  }
  cuda_check(cudaGetLastError(), "attention_tc launch");
  return launches;
}

int attention_tc_bf16(const void* q, long long ldq, const void* k_cache, const void* v_cache,
                      const int* block_tables, int max_blocks, const int* q_starts, const int* kv_lens,
                      void* out, long long ldo, int tokens, int num_seqs, int max_q_len, int min_q_len,
                      int max_kv_len, int hq, int hkv, int head_dim, int block_size, float scale,
                      int window, const float* sinks, float softcap, void* workspace,
                      size_t workspace_bytes, cudaStream_t s, long long num_kv_blocks, int* status, int kv_fp8, int bidir) {
  if (tokens <= 0 || num_seqs <= 0) return 0;
  if (block_size != kPage) throw std::runtime_error("attention_tc: KV block size must be 16");
  if (hq % hkv) throw std::runtime_error("attention_tc: hq must be a multiple of hkv");
  FaParams p{};
  p.q = (const __nv_bfloat16*)q; p.ldq = ldq;
  p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.block_tables = block_tables; p.max_blocks = max_blocks;
  p.q_starts = q_starts; p.kv_lens = kv_lens;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo;
  p.sinks = sinks;
  p.num_kv_blocks = num_kv_blocks; p.status = status; p.bidir = bidir;
  p.hq = hq; p.hkv = hkv; p.group = hq / hkv;
  p.window = window;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.softcap = softcap;
  if (p.group > 16) throw std::runtime_error("attention_tc: at most 16 query heads per KV head");
  switch (head_dim) {
    case 64: return launch_tc<64>(p, tokens, num_seqs, max_q_len, min_q_len, max_kv_len, workspace, workspace_bytes, s, kv_fp8 != 0);
    case 128: return launch_tc<128>(p, tokens, num_seqs, max_q_len, min_q_len, max_kv_len, workspace, workspace_bytes, s, kv_fp8 != 0);
    default: throw std::runtime_error("attention_tc: head_dim must be 64 or 128");
  }
}

}  // namespace fllm
