// Prefill attention on the fifth-generation tensor cores: S = Q K^T and O += P V both run as
// tcgen05.mma with their accumulators in tensor memory.
//
// One CTA owns 128 packed query rows (row = query position x head of one KV group, so one K/V tile
// serves every head of the group) of one sequence and walks the KV pages 128 tokens at a time:
//
//   warp 0   producer  TMA: the 8 pages of the K tile, then of the V tile, 128-byte swizzled rows
//   warp 1   issuer    S[128x128] = Q K^T   (A, B from shared memory, K-major)
//                      O[128x128] (+)= P V  (A = P from tensor memory, B = V as an MN-major operand:
//                                            the cache keeps [token][dim], which is V^T's K-major form)
//   warps 2-5 softmax  one thread per row: tcgen05.ld of the row of S, mask, running max / sum,
//                      P as bf16 written over S's first columns with tcgen05.st, and the rescale of
//                      O in tensor memory when the row maximum moved by more than 2^8
//
// Tensor memory: S/P 128 columns + O up to 128 columns = 256, shared memory 97 KB at head dim 128, so
// two CTAs share an SM and one CTA's softmax overlaps the other's MMAs. Head dim 64 and 128 are template
// instances (a tile is one or two 64-column halves). Every wait is bounded (ptx.cuh: mbar_wait) and a
// timeout is reported through the status word.
//
// Reference counterpart: rust/engine/cuda/attention3.cu:57-288 (mma.sync prefill tiles).
#include <unordered_map>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

namespace {

constexpr int kPageT = 16;
constexpr int kRowsT = 128;        // packed query rows per CTA = tensor memory lanes
constexpr int kTileT = 128;        // KV tokens per tile
constexpr int kHalfBytes = kRowsT * 128;           // one 64-column half of a 128-row tile: 16 KB
// head dim D is a template parameter (64 or 128): a 128-row tile of Q, K or V is D / 64 such halves
template <int D> constexpr int tile_bytes() { return (D / 64) * kHalfBytes; }
constexpr int kThreadsT = 192;
template <int D> constexpr int smem_one() { return 3 * tile_bytes<D>() + 256 + 1024; }   // Q, K, V, barriers, alignment slack
constexpr float kLog2eT = 1.4426950408889634f;
constexpr float kLazyRescale = 8.f;                // keep a stale row maximum while exp2 stays below 2^8

struct FaTmemParams {
  const __nv_bfloat16* q;
  long long ldq;
  const int* block_tables;
  int max_blocks;
  const int* q_starts;
  const int* kv_lens;
  __nv_bfloat16* out;
  long long ldo;
  const float* sinks;
  int* status;
  int hkv, group;
  int window;
  int min_q;             // sequences with fewer query rows are not this kernel's
  float scale_log2, softcap, scale;
  int pv_wide;           // one N=128 MMA per 16 tokens instead of two N=64 ones
  int tile_variant;      // 0: pick by shape; 1 / 2: force one / two query tiles per CTA
  int bidir;             // 1: no causal mask, every query row sees all kv_len tokens (encoders)
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Shared-memory descriptor of an operand stored as 128-byte swizzled rows with 1024 bytes between
// groups of eight rows, in either major-ness. For the MN-major use (V) every MMA covers one 64-wide
// swizzle atom along N, so both offset fields describe the same stride: eight K rows = 1024 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128_1k(uint32_t saddr, uint32_t lbo_bytes = 1024) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// One row (thread) of the softmax over one 128-token tile: reads S from tensor memory, updates the row's
// reference maximum and sum, writes P as bf16 over S's first 64 columns and, when the maximum of any row of
// the warp moved by more than 2^8, rescales the warp's rows of O. `t_s` / `t_o` already carry the lane offset.
template <int D, bool full, bool capped, bool windowed>
__device__ __forceinline__ void softmax_tile_impl(const FaTmemParams& p, uint32_t t_s, uint32_t t_o, int tok0, int lim,
                                                  int beg, bool have_o, float& m_used, float& l) {
  const float cap_in = capped ? p.scale / p.softcap : 0.f;
  const float cap_out = p.softcap * kLog2eT;
  // One warp per lane quarter runs this alone on its scheduler, so the instruction stream is written for
  // instruction-level parallelism: 64 columns per tensor-memory round trip, four independent max / sum chains.
  uint32_t sa[32], sb[32];
  float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll 1
  for (int h = 0; h < 2; ++h) {
    tmem_ld_32x32(t_s + 64 * h, sa);
    tmem_ld_32x32(t_s + 64 * h + 32, sb);
    tmem_ld_wait();
    // columns [lo, hi) of these 64 are visible to this row: one compare (two with a window) per element
    const int hi = lim - (tok0 + 64 * h), lo = beg - (tok0 + 64 * h);
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float a0 = __uint_as_float(sa[i]), a1 = __uint_as_float(sa[i + 1]);
      float b0 = __uint_as_float(sb[i]), b1 = __uint_as_float(sb[i + 1]);
      if (capped) {
        a0 = tanhf(a0 * cap_in); a1 = tanhf(a1 * cap_in); b0 = tanhf(b0 * cap_in); b1 = tanhf(b1 * cap_in);
      }
      if (!full) {
        if (i >= hi || (windowed && i < lo)) a0 = -INFINITY;
        if (i + 1 >= hi || (windowed && i + 1 < lo)) a1 = -INFINITY;
        if (i + 32 >= hi || (windowed && i + 32 < lo)) b0 = -INFINITY;
        if (i + 33 >= hi || (windowed && i + 33 < lo)) b1 = -INFINITY;
      }
      mx0 = fmaxf(mx0, a0); mx1 = fmaxf(mx1, a1); mx2 = fmaxf(mx2, b0); mx3 = fmaxf(mx3, b1);
    }
  }
  // the scale is positive, so it commutes with the maximum
  const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * (capped ? cap_out : p.scale_log2);
  // a row keeps its old reference maximum unless the new one is far above it; the decision is per
  // warp because the tensor memory accesses of the rescale are warp-wide
  const bool grow = mx > m_used + kLazyRescale || (m_used == -INFINITY && mx > -INFINITY);
  const bool warp_grow = __any_sync(0xffffffffu, grow);
  float corr = 1.f;
  if (warp_grow) {
    const float m_new = fmaxf(m_used, mx);
    corr = m_new == -INFINITY ? 1.f : ex2(m_used - m_new);     // m_used = -inf gives 0
    m_used = m_new;
    l *= corr;
  }
  const float m_ref = m_used == -INFINITY ? 0.f : m_used;
  float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll 1
  for (int h = 0; h < 2; ++h) {
    tmem_ld_32x32(t_s + 64 * h, sa);
    tmem_ld_32x32(t_s + 64 * h + 32, sb);
    tmem_ld_wait();
    const int hi = lim - (tok0 + 64 * h), lo = beg - (tok0 + 64 * h);
    uint32_t pa[16], pb[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float a0 = __uint_as_float(sa[i]), a1 = __uint_as_float(sa[i + 1]);
      float b0 = __uint_as_float(sb[i]), b1 = __uint_as_float(sb[i + 1]);
      if (capped) {
        a0 = fmaf(cap_out, tanhf(a0 * cap_in), -m_ref); a1 = fmaf(cap_out, tanhf(a1 * cap_in), -m_ref);
        b0 = fmaf(cap_out, tanhf(b0 * cap_in), -m_ref); b1 = fmaf(cap_out, tanhf(b1 * cap_in), -m_ref);
      } else {
        a0 = fmaf(a0, p.scale_log2, -m_ref); a1 = fmaf(a1, p.scale_log2, -m_ref);
        b0 = fmaf(b0, p.scale_log2, -m_ref); b1 = fmaf(b1, p.scale_log2, -m_ref);
      }
      a0 = ex2(a0); a1 = ex2(a1); b0 = ex2(b0); b1 = ex2(b1);
      if (!full) {
        if (i >= hi || (windowed && i < lo)) a0 = 0.f;
        if (i + 1 >= hi || (windowed && i + 1 < lo)) a1 = 0.f;
        if (i + 32 >= hi || (windowed && i + 32 < lo)) b0 = 0.f;
        if (i + 33 >= hi || (windowed && i + 33 < lo)) b1 = 0.f;
      }
      sum0 += a0; sum1 += a1; sum2 += b0; sum3 += b1;
      pa[i >> 1] = pack_bf16x2(a0, a1);
      pb[i >> 1] = pack_bf16x2(b0, b1);
    }
    // P columns [32h, 32h + 32) hold tokens [64h, 64h + 64): they overwrite S columns that were already read
    tmem_st_32x16(t_s + 32 * h, pa);
    tmem_st_32x16(t_s + 32 * h + 16, pb);
  }
  l += (sum0 + sum1) + (sum2 + sum3);
  if (warp_grow && have_o) {
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      tmem_ld_32x32(t_o + 32 * c, sa);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) sa[i] = __float_as_uint(__uint_as_float(sa[i]) * corr);
      uint32_t lo[16], hi[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) { lo[i] = sa[i]; hi[i] = sa[16 + i]; }
      tmem_st_32x16(t_o + 32 * c, lo);
      tmem_st_32x16(t_o + 32 * c + 16, hi);
    }
  }
  tmem_st_wait();
}

// The mask and soft-cap tests are compile-time so that the common case (a tile every row sees whole, no cap)
// carries no predicated instructions: this code runs one warp per scheduler and every issue slot counts.
template <int D>
__device__ __forceinline__ void softmax_tile(const FaTmemParams& p, uint32_t t_s, uint32_t t_o, int tok0, int lim,
                                             int beg, bool full, bool have_o, float& m_used, float& l) {
  if (p.softcap > 0.f) softmax_tile_impl<D, false, true, true>(p, t_s, t_o, tok0, lim, beg, have_o, m_used, l);
  else if (full) softmax_tile_impl<D, true, false, false>(p, t_s, t_o, tok0, lim, beg, have_o, m_used, l);
  else if (p.window > 0) softmax_tile_impl<D, false, false, true>(p, t_s, t_o, tok0, lim, beg, have_o, m_used, l);
  else softmax_tile_impl<D, false, false, false>(p, t_s, t_o, tok0, lim, beg, have_o, m_used, l);
}

// Final normalisation (with the head's sink, if any) and store of one row of O. The tensor memory loads are
// warp-wide, so rows past the tile's last query take part and only skip the store.
template <int D>
__device__ __forceinline__ void store_row(const FaTmemParams& p, uint32_t t_o, bool valid, int token, int head,
                                          float m_used, float l) {
  float ll = l, c = 1.f;
  if (p.sinks && valid) {
    const float sk2 = p.sinks[head] * kLog2eT;
    const float mn = fmaxf(m_used, sk2);
    c = m_used == -INFINITY ? 0.f : ex2(m_used - mn);
    ll = ll * c + ex2(sk2 - mn);
  }
  const float inv = ll > 0.f ? c / ll : 0.f;
  __nv_bfloat16* dst = p.out + (size_t)token * p.ldo + (size_t)head * D;
#pragma unroll 1
  for (int cc = 0; cc < D / 32; ++cc) {
    uint32_t orow[32];
    tmem_ld_32x32(t_o + 32 * cc, orow);
    tmem_ld_wait();
    if (valid) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 w;
        w.x = pack_bf16x2(__uint_as_float(orow[i]) * inv, __uint_as_float(orow[i + 1]) * inv);
        w.y = pack_bf16x2(__uint_as_float(orow[i + 2]) * inv, __uint_as_float(orow[i + 3]) * inv);
        w.z = pack_bf16x2(__uint_as_float(orow[i + 4]) * inv, __uint_as_float(orow[i + 5]) * inv);
        w.w = pack_bf16x2(__uint_as_float(orow[i + 6]) * inv, __uint_as_float(orow[i + 7]) * inv);
        *reinterpret_cast<uint4*>(dst + 32 * cc + i) = w;
      }
    }
  }
}

template <int D>
__global__ void __launch_bounds__(kThreadsT, 2)
fa_prefill_tmem_kernel(const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
                       const FaTmemParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sq = smem;
  constexpr int TB = tile_bytes<D>();
  uint8_t* sk = smem + TB;
  uint8_t* sv = smem + 2 * TB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * TB);
  uint64_t* k_full = bars + 0;
  uint64_t* v_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_empty = bars + 3;
  uint64_t* s_full = bars + 4;
  uint64_t* p_ready = bars + 5;
  uint64_t* o_done = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;      // the tiles with the longest KV range start first
  const int kvh = blockIdx.y, seq = blockIdx.z;
  const int G = p.group;
  const int RQ = kRowsT / G;
  const int q0 = p.q_starts[seq];
  const int qn = p.q_starts[seq + 1] - q0;
  if (qn < p.min_q) return;
  const int qi0 = qt * RQ;
  if (qi0 >= qn) return;
  const int nq = min(RQ, qn - qi0);
  const int n_rows = nq * G;
  const int kv_len = p.kv_lens[seq];
  const int first_pos = kv_len - qn + qi0;
  const int hi_tok = p.bidir ? kv_len : first_pos + nq;
  const int lo_tok = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int tile_lo = lo_tok / kTileT;
  const int tile_hi = (hi_tok + kTileT - 1) / kTileT;
  const int n_tiles = tile_hi - tile_lo;

  if (threadIdx.x == 0) {
    mbar_init(k_full, 1); mbar_init(v_full, 1); mbar_init(k_empty, 1); mbar_init(v_empty, 1);
    mbar_init(s_full, 1); mbar_init(p_ready, 4); mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tma_k); tma_prefetch_desc(&tma_v); }
  if (warp == 1) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  // Q rows -> shared memory in the layout TMA's 128-byte swizzle would have produced
  for (int i = threadIdx.x; i < kRowsT * (D / 8); i += kThreadsT) {
    const int r = i / (D / 8), c = i % (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < n_rows) {
      const int qi = r / G, hg = r - qi * G;
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + qi0 + qi) * p.ldq + (size_t)(kvh * G + hg) * D + c * 8);
    }
    *reinterpret_cast<uint4*>(sq + (c >> 3) * kHalfBytes + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base;            // S, later P in its first 64 columns
  const uint32_t t_o = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      const int* table = p.block_tables + (size_t)seq * p.max_blocks;
      const int last_page = (kv_len + kPageT - 1) / kPageT - 1;
      // first cache row of the tile's pages; pages past the sequence repeat its last page (finite values).
      // The next tile's table entries are requested before this tile's waits, so their latency is hidden.
      int rows[kTileT / kPageT], nxt[kTileT / kPageT];
#pragma unroll
      for (int pg = 0; pg < kTileT / kPageT; ++pg)
        nxt[pg] = table[min(tile_lo * (kTileT / kPageT) + pg, last_page)];
      for (int it = 0; it < n_tiles; ++it) {
        const int page1 = (tile_lo + it + 1) * (kTileT / kPageT);
#pragma unroll
        for (int pg = 0; pg < kTileT / kPageT; ++pg) {
          rows[pg] = (nxt[pg] * p.hkv + kvh) * kPageT;
          nxt[pg] = table[min(page1 + pg, last_page)];
        }
        if (it > 0 && !mbar_wait(k_empty, (it - 1) & 1, abort_flag)) break;
        mbar_expect_tx(k_full, TB);
#pragma unroll
        for (int pg = 0; pg < kTileT / kPageT; ++pg) {
#pragma unroll
          for (int h = 0; h < D / 64; ++h) tma_load_2d(sk + h * kHalfBytes + pg * 2048, &tma_k, k_full, 64 * h, rows[pg]);
        }
        if (it > 0 && !mbar_wait(v_empty, (it - 1) & 1, abort_flag)) break;
        mbar_expect_tx(v_full, TB);
#pragma unroll
        for (int pg = 0; pg < kTileT / kPageT; ++pg) {
#pragma unroll
          for (int h = 0; h < D / 64; ++h) tma_load_2d(sv + h * kHalfBytes + pg * 2048, &tma_v, v_full, 64 * h, rows[pg]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(128, 128, 1, 1);
      constexpr uint32_t idesc_pv = make_idesc(128, 64, 1, 1) | (1u << 16);     // B is MN-major
      constexpr uint32_t idesc_pv_wide = make_idesc(128, 128, 1, 1) | (1u << 16);
      const uint32_t q_addr = smem_u32(sq), k_addr = smem_u32(sk), v_addr = smem_u32(sv);
      for (int it = 0; it < n_tiles; ++it) {
        const uint32_t ph = it & 1;
        if (!mbar_wait(k_full, ph, abort_flag)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
          tc_mma_bf16(t_s, make_smem_desc_sw128(q_addr + off), make_smem_desc_sw128(k_addr + off), idesc_s, k > 0);
        }
        tc_commit(s_full);
        tc_commit(k_empty);
        if (!mbar_wait(p_ready, ph, abort_flag) || !mbar_wait(v_full, ph, abort_flag)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < kTileT / 16; ++k) {
          const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
          if (D == 128 && p.pv_wide) {      // the second 64-wide atom of V's rows lies one half tile further: the leading offset
            tc_mma_bf16_ts(t_o, t_s + 8 * k, smem_desc_sw128_1k(v_addr + k * 2048, kHalfBytes), idesc_pv_wide, acc);
          } else {
            tc_mma_bf16_ts(t_o, t_s + 8 * k, smem_desc_sw128_1k(v_addr + k * 2048), idesc_pv, acc);
            if (D == 128)
              tc_mma_bf16_ts(t_o + 64, t_s + 8 * k, smem_desc_sw128_1k(v_addr + kHalfBytes + k * 2048), idesc_pv, acc);
          }
        }
        tc_commit(v_empty);
        if (it == n_tiles - 1) tc_commit(o_done);
      }
    }
  } else {
    const int quarter = warp & 3;                       // the lane quarter this warp may touch
    const int r = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    int lim = 0, beg = 0;
    if (r < n_rows) {
      lim = p.bidir ? kv_len : first_pos + r / G + 1;
      beg = p.window > 0 ? max(0, lim - p.window) : 0;
    }
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
      const int tok0 = (tile_lo + it) * kTileT;
      if (!mbar_wait(s_full, it & 1, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      // whole tile visible to every row of the CTA: no per-element mask
      const bool full = p.window == 0 && tok0 + kTileT <= (p.bidir ? kv_len : first_pos + 1) && n_rows == kRowsT;
      softmax_tile<D>(p, t_s + lane_off, t_o + lane_off, tok0, lim, beg, full, it > 0, m_used, l);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (ok && mbar_wait(o_done, 0, abort_flag)) {
      tc_fence_after_sync();
      const int qi = r / G, hg = r - qi * G;
      store_row<D>(p, t_o + lane_off, r < n_rows, q0 + qi0 + qi, kvh * G + hg, m_used, l);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tmem_base, 256); }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicCAS(p.status, FLLM_OK, FLLM_ERR_MBAR_TIMEOUT);
}

// The same pipeline with two 128-row query tiles per CTA sharing every K/V tile (half the K/V traffic per
// FLOP, which is what bounds the one-tile kernel: its 64 KB per 8.4 MFLOP tile saturates L2 first). Ten warps:
// producer, issuer, and one softmax group of four warps per query tile. The issuer interleaves the two tiles
// (PV0, next S0, PV1, next S1) so that one group's softmax runs under the other tile's MMAs; K and V are
// double buffered. Tensor memory: S0 S1 O0 O1 = 512 columns, one CTA per SM.
constexpr int kThreadsT2 = 320;
template <int D> constexpr int smem_two() { return 6 * tile_bytes<D>() + 256 + 1024; }

template <int D>
__global__ void __launch_bounds__(kThreadsT2, 1)
fa_prefill_tmem2_kernel(const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
                        const FaTmemParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sq = smem;                          // two query tiles
  constexpr int TB = tile_bytes<D>();
  uint8_t* sk = smem + 2 * TB;                 // two stages
  uint8_t* sv = smem + 4 * TB;                 // two stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TB);
  uint64_t* k_full = bars + 0;                 // [2] by stage
  uint64_t* v_full = bars + 2;
  uint64_t* k_empty = bars + 4;
  uint64_t* v_empty = bars + 6;
  uint64_t* s_full = bars + 8;                 // [2] by query tile
  uint64_t* p_ready = bars + 10;
  uint64_t* o_done = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int kvh = blockIdx.y, seq = blockIdx.z;
  const int G = p.group;
  const int RQ = 2 * kRowsT / G;
  const int q0 = p.q_starts[seq];
  const int qn = p.q_starts[seq + 1] - q0;
  if (qn < p.min_q) return;
  const int qi0 = qt * RQ;
  if (qi0 >= qn) return;
  const int nq = min(RQ, qn - qi0);
  const int n_rows = nq * G;
  const int kv_len = p.kv_lens[seq];
  const int first_pos = kv_len - qn + qi0;
  const int hi_tok = p.bidir ? kv_len : first_pos + nq;
  const int lo_tok = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int tile_lo = lo_tok / kTileT;
  const int tile_hi = (hi_tok + kTileT - 1) / kTileT;
  const int n_tiles = tile_hi - tile_lo;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], 4);
    }
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tma_k); tma_prefetch_desc(&tma_v); }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  for (int i = threadIdx.x; i < 2 * kRowsT * (D / 8); i += kThreadsT2) {
    const int r = i / (D / 8), c = i % (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < n_rows) {
      const int qi = r / G, hg = r - qi * G;
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + qi0 + qi) * p.ldq + (size_t)(kvh * G + hg) * D + c * 8);
    }
    const int rr = r & (kRowsT - 1);
    *reinterpret_cast<uint4*>(sq + (r >> 7) * TB + (c >> 3) * kHalfBytes + rr * 128 + (((c & 7) ^ (rr & 7)) << 4)) = v;
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const int* table = p.block_tables + (size_t)seq * p.max_blocks;
      const int last_page = (kv_len + kPageT - 1) / kPageT - 1;
      int rows[kTileT / kPageT], nxt[kTileT / kPageT];
#pragma unroll
      for (int pg = 0; pg < kTileT / kPageT; ++pg)
        nxt[pg] = table[min(tile_lo * (kTileT / kPageT) + pg, last_page)];
      for (int it = 0; it < n_tiles; ++it) {
        const int b = it & 1;
        const uint32_t prev = ((it >> 1) - 1) & 1;       // phase of the stage's previous use
        const int page1 = (tile_lo + it + 1) * (kTileT / kPageT);
#pragma unroll
        for (int pg = 0; pg < kTileT / kPageT; ++pg) {
          rows[pg] = (nxt[pg] * p.hkv + kvh) * kPageT;
          nxt[pg] = table[min(page1 + pg, last_page)];
        }
        if (it >= 2 && !mbar_wait(&k_empty[b], prev, abort_flag)) break;
        mbar_expect_tx(&k_full[b], TB);
        uint8_t* kd = sk + b * TB;
#pragma unroll
        for (int pg = 0; pg < kTileT / kPageT; ++pg) {
#pragma unroll
          for (int h = 0; h < D / 64; ++h) tma_load_2d(kd + h * kHalfBytes + pg * 2048, &tma_k, &k_full[b], 64 * h, rows[pg]);
        }
        if (it >= 2 && !mbar_wait(&v_empty[b], prev, abort_flag)) break;
        mbar_expect_tx(&v_full[b], TB);
        uint8_t* vd = sv + b * TB;
#pragma unroll
        for (int pg = 0; pg < kTileT / kPageT; ++pg) {
#pragma unroll
          for (int h = 0; h < D / 64; ++h) tma_load_2d(vd + h * kHalfBytes + pg * 2048, &tma_v, &v_full[b], 64 * h, rows[pg]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(128, 128, 1, 1);
      constexpr uint32_t idesc_pv = make_idesc(128, 64, 1, 1) | (1u << 16);     // B is MN-major
      constexpr uint32_t idesc_pv_wide = make_idesc(128, 128, 1, 1) | (1u << 16);
      const uint32_t q_addr = smem_u32(sq), k_addr = smem_u32(sk), v_addr = smem_u32(sv);
      auto issue_s = [&](int g, int stage) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
          tc_mma_bf16(tmem_base + 128 * g, make_smem_desc_sw128(q_addr + g * TB + off),
                      make_smem_desc_sw128(k_addr + stage * TB + off), idesc_s, k > 0);
        }
      };
      auto issue_pv = [&](int g, int stage, bool first) {
        const uint32_t t_p = tmem_base + 128 * g, t_o = tmem_base + 256 + 128 * g;
        const uint32_t vb = v_addr + stage * TB;
#pragma unroll
        for (int k = 0; k < kTileT / 16; ++k) {
          const uint32_t acc = (!first || k > 0) ? 1u : 0u;
          if (D == 128 && p.pv_wide) {
            tc_mma_bf16_ts(t_o, t_p + 8 * k, smem_desc_sw128_1k(vb + k * 2048, kHalfBytes), idesc_pv_wide, acc);
          } else {
            tc_mma_bf16_ts(t_o, t_p + 8 * k, smem_desc_sw128_1k(vb + k * 2048), idesc_pv, acc);
            if (D == 128)
              tc_mma_bf16_ts(t_o + 64, t_p + 8 * k, smem_desc_sw128_1k(vb + kHalfBytes + k * 2048), idesc_pv, acc);
          }
        }
      };
      bool ok = mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0, 0);
        tc_commit(&s_full[0]);
        issue_s(1, 0);
        tc_commit(&s_full[1]);
        tc_commit(&k_empty[0]);
      }
      for (int it = 0; ok && it < n_tiles; ++it) {
        const int b = it & 1, nb = b ^ 1;
        const uint32_t ph = (it >> 1) & 1, nph = ((it + 1) >> 1) & 1;
        const bool more = it + 1 < n_tiles;
        if (!mbar_wait(&p_ready[0], it & 1, abort_flag) || !mbar_wait(&v_full[b], ph, abort_flag)) break;
        tc_fence_after_sync();
        issue_pv(0, b, it == 0);
        if (more) {
          if (!mbar_wait(&k_full[nb], nph, abort_flag)) break;
          tc_fence_after_sync();
          issue_s(0, nb);
          tc_commit(&s_full[0]);
        }
        if (!mbar_wait(&p_ready[1], it & 1, abort_flag)) break;
        tc_fence_after_sync();
        issue_pv(1, b, it == 0);
        tc_commit(&v_empty[b]);
        if (more) {
          issue_s(1, nb);
          tc_commit(&s_full[1]);
          tc_commit(&k_empty[nb]);
        } else {
          tc_commit(o_done);
        }
      }
    }
  } else {
    const int g = (warp - 2) >> 2;                      // query tile of this softmax group
    const int quarter = warp & 3;
    const int r = g * kRowsT + quarter * 32 + lane;     // packed row within the CTA
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + 128 * g + lane_off, t_o = tmem_base + 256 + 128 * g + lane_off;
    int lim = 0, beg = 0;
    if (r < n_rows) {
      lim = p.bidir ? kv_len : first_pos + r / G + 1;
      beg = p.window > 0 ? max(0, lim - p.window) : 0;
    }
    const int group_first = first_pos + (g * kRowsT) / G;
    const bool group_whole = n_rows >= (g + 1) * kRowsT;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
      const int tok0 = (tile_lo + it) * kTileT;
      if (!mbar_wait(&s_full[g], it & 1, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const bool full = p.window == 0 && tok0 + kTileT <= (p.bidir ? kv_len : group_first + 1) && group_whole;
      softmax_tile<D>(p, t_s, t_o, tok0, lim, beg, full, it > 0, m_used, l);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[g]);
    }
    if (ok && mbar_wait(o_done, 0, abort_flag)) {
      tc_fence_after_sync();
      const int qi = r / G, hg = r - qi * G;
      store_row<D>(p, t_o, r < n_rows, q0 + qi0 + qi, kvh * G + hg, m_used, l);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tmem_base, 512); }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicCAS(p.status, FLLM_OK, FLLM_ERR_MBAR_TIMEOUT);
}

struct MapKey {
  const void* k;
  const void* v;
  uint64_t rows;
  int d;
  bool operator==(const MapKey& o) const { return k == o.k && v == o.v && rows == o.rows && d == o.d; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& x) const {
    return std::hash<const void*>()(x.k) ^ (std::hash<const void*>()(x.v) * 31) ^ std::hash<uint64_t>()(x.rows * 2 + x.d / 128);
  }
};
struct MapPair { CUtensorMap k, v; };

template <int D>
void launch_tmem(const MapPair& maps, const FaTmemParams& p, int max_q_len, int num_seqs, cudaStream_t s) {
  static bool configured[kMaxDevices] = {};
  if (first_call_on_device(configured)) {
    cuda_check(cudaFuncSetAttribute(fa_prefill_tmem_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_one<D>()),
               "fa_prefill_tmem smem");
    cuda_check(cudaFuncSetAttribute(fa_prefill_tmem2_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_two<D>()),
               "fa_prefill_tmem2 smem");
  }
  // Two query tiles per CTA when that still gives every SM a CTA (tile_variant 1 / 2 forces one: tests only).
  const int forced = p.tile_variant;
  const int rq2 = 2 * kRowsT / p.group;
  const long long ctas2 = (long long)((max_q_len + rq2 - 1) / rq2) * p.hkv * num_seqs;
  const bool two = forced ? forced == 2 : (max_q_len * p.group >= 2 * kRowsT && ctas2 >= sm_count());
  if (two) {
    dim3 grid((max_q_len + rq2 - 1) / rq2, p.hkv, num_seqs);
    fa_prefill_tmem2_kernel<D><<<grid, kThreadsT2, smem_two<D>(), s>>>(maps.k, maps.v, p);
  } else {
    const int rq = kRowsT / p.group;
    dim3 grid((max_q_len + rq - 1) / rq, p.hkv, num_seqs);
    fa_prefill_tmem_kernel<D><<<grid, kThreadsT, smem_one<D>(), s>>>(maps.k, maps.v, p);
  }
  cuda_check(cudaGetLastError(), "fa_prefill_tmem launch");
}

}  // namespace

bool attention_prefill_tmem_supported(int head_dim, int group, int block_size) {
  return (head_dim == 64 || head_dim == 128) && block_size == kPageT && group >= 1 && group <= 16 && (kRowsT % group) == 0;
}

// Tensor maps depend only on the cache tensors, so they are built once per (K, V) pair.
void attention_prefill_tmem(const void* q, long long ldq, const void* k_cache, const void* v_cache, long long num_blocks,
                            const int* block_tables, int max_blocks, const int* q_starts, const int* kv_lens,
                            void* out, long long ldo, int num_seqs, int max_q_len, int min_q, int hq, int hkv,
                            int head_dim, float scale, int window, const float* sinks, float softcap, int* status,
                            cudaStream_t s, int tile_variant, int bidir) {
  static std::unordered_map<MapKey, MapPair, MapKeyHash> maps;
  const uint64_t rows = (uint64_t)num_blocks * hkv * kPageT;
  const MapKey key{k_cache, v_cache, rows, head_dim};
  auto it = maps.find(key);
  if (it == maps.end()) {
    if (maps.size() > 4096) maps.clear();
    MapPair mp;
    mp.k = make_tmap_2d(k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, head_dim, head_dim * 2, kPageT, 64, true);
    mp.v = make_tmap_2d(v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, head_dim, head_dim * 2, kPageT, 64, true);
    it = maps.emplace(key, mp).first;
  }
  FaTmemParams p{};
  p.q = (const __nv_bfloat16*)q; p.ldq = ldq;
  p.block_tables = block_tables; p.max_blocks = max_blocks;
  p.q_starts = q_starts; p.kv_lens = kv_lens;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo;
  p.sinks = sinks; p.status = status;
  p.hkv = hkv; p.group = hq / hkv;
  p.window = window; p.min_q = min_q;
  p.scale = scale; p.scale_log2 = scale * kLog2eT; p.softcap = softcap;
  p.pv_wide = 1;
  p.tile_variant = tile_variant;
  p.bidir = bidir;
  if (head_dim == 64) launch_tmem<64>(it->second, p, max_q_len, num_seqs, s);
  else launch_tmem<128>(it->second, p, max_q_len, num_seqs, s);
}

}  // namespace fllm
