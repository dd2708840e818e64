// Packed 4-bit weights x bf16 activations on tcgen05 (weights stay packed in HBM):
//
//   NVFP4   e2m1 codes, two per byte, + one e4m3 scale per 16 values + an fp32 tensor scale
//   MXFP4   e2m1 codes, two per byte, + one e8m0 (power of two) scale per 32 values
//   INT4G   unsigned 4-bit codes + one (scale, min) pair of bf16 per 32 values: value = q * scale - min.
//           This is the device form of GGUF Q4_K / Q4_0 / Q4_1 and of AWQ / GPTQ int4 groups, re-laid at
//           load time (planar codes, nibbles ordered so that two shifts-and-masks yield K-ordered pairs).
//
// Decode is bound by the bytes of weight read, so reading 4.5 bit/weight instead of 16 is the
// point. The kernel is the swap-AB GEMM of gemm_bf16.cu with one extra stage in the operand path:
// TMA brings the raw code tile (128 features x 32 bytes) into shared memory, four warps expand it
// to the 128-byte-swizzled bf16 tile the MMA wants (e2m1 -> bf16 through a byte-permute table,
// times the block scale: exact in bf16 because 3 + 4 significant bits fit its 8), publish it with
// a proxy fence + mbarrier, and the single issuing thread runs tcgen05.mma kind::f16 on it. The
// same four warps run the epilogue (tensor scale, bias, 16-byte transposed stores).
//
// Reference counterparts: rust/engine/cuda/nvfp4.cu:132-307 (mma.sync mxf4nvf4, GeForce Blackwell
// only), rust/engine/cuda/marlin_vllm (W4A16 Marlin, the sm_100 default), MXFP4 through the
// IQ4_NL look-up path (rust/engine/cuda/common.cuh:154).
#include <cuda_fp8.h>

#include <algorithm>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

constexpr int W4_BM = 128;
constexpr int W4_BK = 64;             // values per stage = one 128-byte swizzled bf16 row
constexpr int kW4Threads = 64 + 3 * 128;     // TMA warp, MMA warp, 3 groups of 4 expanding warps (8 of them run the epilogue)

struct W4Args {
  int M, N, K;                        // M = output features, N = tokens
  int m_tiles, k_blocks;
  int k_splits, kb_per_split;         // grid.y splits of the K loop; partial sums go to `ws`
  float* ws;                          // [k_splits][N][M] fp32 when k_splits > 1
  int fmt;                            // 0 NVFP4 (e4m3 / 16), 1 MXFP4 (e8m0 / 32), 2 INT4G ((scale, min) bf16 / 32)
  long long ldc;
  __nv_bfloat16* out;
  const uint8_t* scales;              // [M][K/16] bytes, [M][K/32] bytes, or [M][K/32] x {bf16 scale, bf16 min}
  float alpha;                        // tensor scale (NVFP4), 1 otherwise
  const __nv_bfloat16* bias;
  int* status;
  // grouped (mixture of experts): blockIdx.y walks a device-built tile list; tile i multiplies rows
  // [row0, row0 + BN) of the permuted activations with expert e's matrix (codes / scales / bias stacked
  // over experts, g_rows output features each)
  const int* g_tile_expert;
  const int* g_tile_row0;
  const int* g_num_tiles;
  int g_rows;
  int grid_y;                         // K splits, or the length bound of the tile list
};

constexpr int kW4Groups = 3;                                  // warp groups that take turns on the K steps

template <int BN>
struct W4Smem {
  // Codes arrive as 128-byte rows (256 values: narrower rows waste HBM bursts), so one code slot feeds
  // four 64-value MMA steps; the ring's depth sets the bytes of weight in flight per SM. Activations
  // arrive per step. The expanded bf16 operand never touches shared memory: the expanding warps store it
  // into tensor memory (32 columns per step) and the MMA reads A from there.
  static constexpr int kRawBytes = W4_BM * 128;                // 16 KB of codes = 4 steps
  static constexpr int kBBytes = BN * W4_BK * 2;
  static constexpr int kRStages = BN <= 64 ? 4 : 6;
  static constexpr int kBudget = (BN <= 64 ? 104 : 200) * 1024;
  static constexpr int kBFit = (kBudget - kRStages * kRawBytes) / kBBytes;
  static constexpr int kBStages = kBFit > 8 ? 8 : kBFit;
  // tensor memory: [0, kDCols) accumulator, then kAStages x 32 columns of expanded weights. Two CTAs
  // share the SM's 512 columns when BN <= 64.
  static constexpr int kDCols = BN < 32 ? 32 : BN;
  static constexpr int kTmemCols = BN <= 64 ? 256 : 512;
  static constexpr int kAStages = (kTmemCols - kDCols) / 32 > 8 ? 8 : (kTmemCols - kDCols) / 32;
  static constexpr int kBarBytes = 512;
  static constexpr int kLutBytes = 1024;                       // e4m3 -> bf16x2 table
  static constexpr int kTotal = kRStages * kRawBytes + kBStages * kBBytes + kBarBytes + kLutBytes + 1024;
  static_assert(kBStages >= 2, "activation ring");
  static_assert(kAStages > kW4Groups, "every group needs a slot of its own plus one in the MMA");
  static_assert((2 * kRStages + 2 * kBStages + 2 * kAStages + 2) * 8 + 8 <= kBarBytes, "barrier block");
  static_assert(8 * 32 * 32 * 2 <= kRStages * kRawBytes, "the epilogue staging reuses the code ring");
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

// 8 e2m1 codes (one 32-bit word, low nibble first) -> 8 bf16, scaled by `s2` (bf16x2 of the block scale).
// Four codes per step: two byte-permutes look the high and low bf16 bytes up in 8-entry tables held in
// registers (selector = the codes' three magnitude bits), a sign-replicating permute spreads the four sign
// bits, two more permutes interleave the bytes into bf16 pairs: about 2.75 instructions per value.
__device__ __forceinline__ void e2m1x8_to_bf16(uint32_t codes, uint32_t s2, uint32_t (&out)[4]) {
  // bf16 of {0, .5, 1, 1.5, 2, 3, 4, 6}: high bytes 00 3F 3F 3F 40 40 40 40, low bytes 00 00 80 C0 00 40 80 C0
  constexpr uint32_t HI_LO = 0x3F3F3F00u, HI_HI = 0x40404040u, LO_LO = 0xC0800000u, LO_HI = 0xC0804000u;
  const __nv_bfloat162 sc = *reinterpret_cast<const __nv_bfloat162*>(&s2);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t w = codes >> (16 * h);                          // selectors read the low 16 bits only
    const uint32_t sel = w & 0x7777u;
    uint32_t hi4 = prmt(HI_LO, HI_HI, sel);
    const uint32_t lo4 = prmt(LO_LO, LO_HI, sel);
    const uint32_t sg = prmt(w, w << 4, 0x9D8Cu);                  // byte i = 0xFF where code i is negative
    hi4 |= sg & 0x80808080u;
    uint32_t v0 = prmt(lo4, hi4, 0x5140u);                         // [lo0, hi0, lo1, hi1]
    uint32_t v1 = prmt(lo4, hi4, 0x7362u);                         // [lo2, hi2, lo3, hi3]
    __nv_bfloat162 r0 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&v0), sc);
    __nv_bfloat162 r1 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&v1), sc);
    out[2 * h] = *reinterpret_cast<uint32_t*>(&r0);
    out[2 * h + 1] = *reinterpret_cast<uint32_t*>(&r1);
  }
}

// 8 unsigned 4-bit codes -> 8 bf16 of q * s - m. Storage order: nibble j of the word holds value 2j (j < 4)
// or 2(j - 4) + 1, so ((w >> 4j) & 0x000F000F) is the K-ordered pair (2j, 2j + 1). OR-ing 0x4300 makes the
// bf16 number 128 + q exactly; one subtract and one fused multiply-add finish it.
__device__ __forceinline__ void int4x8_to_bf16(uint32_t w, uint32_t s2, uint32_t negm2, uint32_t (&out)[4]) {
  const __nv_bfloat162 sc = *reinterpret_cast<const __nv_bfloat162*>(&s2);
  const __nv_bfloat162 nm = *reinterpret_cast<const __nv_bfloat162*>(&negm2);
  const uint32_t c128 = 0x43004300u;
  const __nv_bfloat162 b128 = *reinterpret_cast<const __nv_bfloat162*>(&c128);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t t = ((w >> (4 * j)) & 0x000F000Fu) | c128;
    const __nv_bfloat162 q = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&t), b128);
    const __nv_bfloat162 r = __hfma2(q, sc, nm);
    out[j] = *reinterpret_cast<const uint32_t*>(&r);
  }
}

__device__ __forceinline__ float scale_to_float(uint8_t s, int fmt) {
  if (fmt == 0) {
    __nv_fp8_e4m3 v;
    v.__x = s;
    return static_cast<float>(v);
  }
  return __uint_as_float((uint32_t)s << 23);                       // e8m0: 2^(s - 127); s = 0 -> 0 (denormal floor)
}

template <int BN>
__global__ void __launch_bounds__(kW4Threads, BN <= 64 ? 2 : 1)
gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tma_raw, const __grid_constant__ CUtensorMap tma_b, const W4Args p) {
  using S = W4Smem<BN>;
  constexpr int RST = S::kRStages, BST = S::kBStages, AST = S::kAStages, G = kW4Groups;
  extern __shared__ uint8_t smem_raw_[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sR = smem;                                   // code slots, 16 KB each (128-byte swizzled rows)
  uint8_t* sB = sR + RST * S::kRawBytes;                // activations, BN x 128 B each
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + BST * S::kBBytes);
  uint64_t* rfull_bar = bars;                           // codes landed
  uint64_t* rempty_bar = rfull_bar + RST;               // 4 steps x 4 warps are done with the slot
  uint64_t* bfull_bar = rempty_bar + RST;               // activations landed
  uint64_t* bempty_bar = bfull_bar + BST;               // MMA retired
  uint64_t* ready_bar = bempty_bar + BST;               // expanded operand stored to tensor memory (4 warps)
  uint64_t* aempty_bar = ready_bar + AST;               // its columns consumed by the MMA
  uint64_t* tfull_bar = aempty_bar + AST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* lut = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(bars) + S::kBarBytes);
  __nv_bfloat16* stage_out = reinterpret_cast<__nv_bfloat16*>(sR);      // free once every code slot was expanded
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool grouped = p.g_tile_expert != nullptr;
  if (grouped && (int)blockIdx.y >= *p.g_num_tiles) return;       // the list is shorter than the grid (whole CTA leaves)
  const int g_expert = grouped ? p.g_tile_expert[blockIdx.y] : 0;
  const int g_row0 = grouped ? p.g_tile_row0[blockIdx.y] : 0;
  const int code_row0 = g_expert * p.g_rows + blockIdx.x * W4_BM;  // first row of this tile in the (stacked) code matrix

  if (threadIdx.x == 0) {
    for (int s = 0; s < RST; ++s) { mbar_init(&rfull_bar[s], 1); mbar_init(&rempty_bar[s], 16); }
    for (int s = 0; s < BST; ++s) { mbar_init(&bfull_bar[s], 1); mbar_init(&bempty_bar[s], 1); }
    for (int s = 0; s < AST; ++s) { mbar_init(&ready_bar[s], 4); mbar_init(&aempty_bar[s], 1); }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (threadIdx.x >= 64 && threadIdx.x < 64 + 256) {    // scale byte -> bf16x2 {s, s}
    const int i = threadIdx.x - 64;
    const float f = scale_to_float((uint8_t)i, p.fmt);
    lut[i] = pack_bf16x2(f, f);
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tma_raw); tma_prefetch_desc(&tma_b); }
  if (warp == 1) { tmem_alloc(tmem_slot, S::kTmemCols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  const int m_idx = blockIdx.x;                         // one feature tile (x one K split) per CTA
  const int kb0 = grouped ? 0 : blockIdx.y * p.kb_per_split;   // multiple of 4: code slots start on 256 values
  const int nkb = min(p.k_blocks, kb0 + p.kb_per_split) - kb0;

  if (warp == 0) {
    if (lane == 0) {
      // codes are static: request the first slots before waiting for the predecessor kernel
      const int nrb = (nkb + 3) >> 2;
      const int pre = min(nrb, RST);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&rfull_bar[i], S::kRawBytes);
        tma_load_2d(sR + i * S::kRawBytes, &tma_raw, &rfull_bar[i], (kb0 + 4 * i) * 32, code_row0);
      }
      pdl_wait();
      int rs = 0, bs = 0;
      uint32_t rphase = 0, bphase = 0;
      for (int kb = 0; kb < nkb; ++kb) {
        if ((kb & 3) == 0) {
          if ((kb >> 2) >= pre) {
            if (!mbar_wait(&rempty_bar[rs], rphase ^ 1, abort_flag)) break;
            mbar_expect_tx(&rfull_bar[rs], S::kRawBytes);
            tma_load_2d(sR + rs * S::kRawBytes, &tma_raw, &rfull_bar[rs], (kb0 + kb) * 32, code_row0);
          }
          if (++rs == RST) { rs = 0; rphase ^= 1; }
        }
        if (!mbar_wait(&bempty_bar[bs], bphase ^ 1, abort_flag)) break;
        mbar_expect_tx(&bfull_bar[bs], S::kBBytes);
        tma_load_2d(sB + bs * S::kBBytes, &tma_b, &bfull_bar[bs], (kb0 + kb) * W4_BK, g_row0);
        if (++bs == BST) { bs = 0; bphase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(W4_BM, BN, 1, 1);
      int bs = 0, as = 0;
      uint32_t bphase = 0, aphase = 0;
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb) {
        if (!mbar_wait(&bfull_bar[bs], bphase, abort_flag) || !mbar_wait(&ready_bar[as], aphase, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t ta = tmem_base + S::kDCols + as * 32;
        const uint64_t db = make_smem_desc_sw128(smem_u32(sB + bs * S::kBBytes));
#pragma unroll
        for (int k = 0; k < W4_BK / 16; ++k) tc_mma_bf16_ts(tmem_base, ta + 8 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit(&bempty_bar[bs]);
        tc_commit(&aempty_bar[as]);
        if (++bs == BST) { bs = 0; bphase ^= 1; }
        if (++as == AST) { as = 0; aphase ^= 1; }
      }
      if (ok) tc_commit(tfull_bar);
    }
  } else {
    // ------------------------------------------------ expand codes -> bf16 in tensor memory, then epilogue
    // A warp's instruction stream for one step is long and mostly serial (it runs at a few cycles per
    // instruction), so the groups take turns: group g expands steps g, g + G, ... and has G step times
    // for each. Every thread owns one row (= TMEM lane) and expands all 64 values of it.
    const int e = warp - 2;                             // 0..11
    const int q = warp & 3;                             // TMEM lane quarter this warp may touch
    const int g = e >> 2;                               // group
    const int row = q * 32 + lane;
    const int m_row = g_expert * p.g_rows + min(m_idx * W4_BM + row, p.M - 1);
    const int sbytes = p.fmt == 0 ? 4 : p.fmt == 1 ? 2 : 8;   // scale bytes per row per step
    const uint8_t* srow = p.scales + (size_t)m_row * (p.K / 64) * sbytes + (size_t)kb0 * sbytes;
    const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
    auto load_scales = [&](int kb) -> uint2 {           // this row's scales of step kb
      if (kb >= nkb) return make_uint2(0, 0);
      if (p.fmt == 0) return make_uint2(__ldg(reinterpret_cast<const uint32_t*>(srow + kb * 4)), 0);
      if (p.fmt == 1) return make_uint2((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(srow + kb * 2)), 0);
      return __ldg(reinterpret_cast<const uint2*>(srow + kb * 8));
    };
    bool ok = true;
    uint2 sc_cur = load_scales(g), sc_next = load_scales(g + G);
    for (int kb = g; kb < nkb && ok; kb += G) {
      const uint32_t sraw = sc_cur.x, sraw2 = sc_cur.y;
      sc_cur = sc_next;
      sc_next = load_scales(kb + 2 * G);                // two of this group's steps ahead
      const int rb = kb >> 2, sub = kb & 3;
      const int rs = rb % RST, as = kb % AST;
      const uint32_t rphase = (rb / RST) & 1, aphase = (kb / AST) & 1;
      uint32_t s2[4];
      if (p.fmt == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) s2[i] = lut[(sraw >> (8 * i)) & 0xFF];
      } else if (p.fmt == 1) {
        s2[0] = s2[1] = lut[sraw & 0xFF];
        s2[2] = s2[3] = lut[(sraw >> 8) & 0xFF];
      } else {                                          // {scale, min} bf16 of the two 32-value groups
        s2[0] = __byte_perm(sraw, 0, 0x1010);           // (s, s)
        s2[1] = __byte_perm(sraw, 0, 0x3232) ^ 0x80008000u;   // (-m, -m)
        s2[2] = __byte_perm(sraw2, 0, 0x1010);
        s2[3] = __byte_perm(sraw2, 0, 0x3232) ^ 0x80008000u;
      }
      if (!mbar_wait(&rfull_bar[rs], rphase, abort_flag)) { ok = false; break; }
      const uint8_t* rrow = sR + rs * S::kRawBytes + row * 128;
      const uint4 r0 = *reinterpret_cast<const uint4*>(rrow + (((2 * sub) ^ (row & 7)) << 4));
      const uint4 r1 = *reinterpret_cast<const uint4*>(rrow + (((2 * sub + 1) ^ (row & 7)) << 4));
      if (!mbar_wait(&aempty_bar[as], aphase ^ 1, abort_flag)) { ok = false; break; }
      const uint32_t t_a = t_lane + S::kDCols + as * 32;
      {
        const uint32_t words[4] = {r0.x, r0.y, r0.z, r0.w};
        uint32_t o[16];
#pragma unroll
        for (int c = 0; c < 4; ++c) {                   // 8 codes -> 4 cells of two bf16 each
          uint32_t o4[4];
          if (p.fmt == 2) int4x8_to_bf16(words[c], s2[0], s2[1], o4);
          else e2m1x8_to_bf16(words[c], s2[c >> 1], o4);
#pragma unroll
          for (int i = 0; i < 4; ++i) o[4 * c + i] = o4[i];
        }
        tmem_st_32x16(t_a, o);
      }
      {
        const uint32_t words[4] = {r1.x, r1.y, r1.z, r1.w};
        uint32_t o[16];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o4[4];
          if (p.fmt == 2) int4x8_to_bf16(words[c], s2[2], s2[3], o4);
          else e2m1x8_to_bf16(words[c], s2[2 + (c >> 1)], o4);
#pragma unroll
          for (int i = 0; i < 4; ++i) o[4 * c + i] = o4[i];
        }
        tmem_st_32x16(t_a + 16, o);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {                                  // one arrival per warp on each barrier
        mbar_arrive(&ready_bar[as]);
        mbar_arrive(&rempty_bar[rs]);                   // 4 steps x 4 warps release a code slot
      }
    }
    // a slot whose last steps do not exist (K not a multiple of 256) is never reloaded: no arrival owed
    pdl_wait();
    // Epilogue: two warps share each TMEM lane quarter and split the token columns.
    constexpr int CH = BN < 64 ? 16 : 32;
    constexpr int COLS_PER_WARP = BN >= 32 ? BN / 2 : BN;
    const int half = g;                                 // groups 0 and 1 run it
    const bool has_cols = g < 2 && (BN >= 32 || half == 0);
    if (ok && has_cols && mbar_wait(tfull_bar, 0, abort_flag)) {
      tc_fence_after_sync();
      const int m = m_idx * W4_BM + q * 32 + lane;
      const float bias_m = (p.bias && m < p.M) ? __bfloat162float(p.bias[g_expert * p.g_rows + m]) : 0.f;
      __nv_bfloat16* stg = stage_out + e * (32 * 32);
      const int c_begin = BN >= 32 ? half * COLS_PER_WARP : 0;
#pragma unroll 1
      for (int c0 = c_begin; c0 < c_begin + COLS_PER_WARP; c0 += CH) {
        uint32_t r[CH];
        if constexpr (CH == 32) tmem_ld_32x32(t_lane + c0, r);
        else tmem_ld_32x16(t_lane + c0, r);
        tmem_ld_wait();
        if (p.k_splits > 1) {                           // fp32 partial sums, lanes along features: coalesced
          float* wsp = p.ws + (size_t)blockIdx.y * p.N * p.M;
#pragma unroll
          for (int c = 0; c < CH; ++c)
            if (c0 + c < p.N && m < p.M) wsp[(size_t)(c0 + c) * p.M + m] = __uint_as_float(r[c]);
          continue;
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) stg[c * 32 + lane] = __float2bfloat16(__uint_as_float(r[c]) * p.alpha + bias_m);
        __syncwarp();
        const int f0 = 8 * (lane & 3);
        const int mm0 = m_idx * W4_BM + q * 32 + f0;
#pragma unroll
        for (int rnd = 0; rnd < CH / 8; ++rnd) {
          const int c = (lane >> 2) + 8 * rnd;
          const int n = g_row0 + c0 + c;
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
__global__ void w4_splitk_reduce_kernel(const float* __restrict__ ws, int splits, int rows, int cols, long long ldc,
                                        float alpha, const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out) {
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
  uint2 o;
  o.x = pack_bf16x2(acc.x * alpha + b[0], acc.y * alpha + b[1]);
  o.y = pack_bf16x2(acc.z * alpha + b[2], acc.w * alpha + b[3]);
  *reinterpret_cast<uint2*>(out + (size_t)r * ldc + c) = o;
}

// Expand packed weights to bf16 [M][K] (prefill path: expand once, then the dense GEMM).
__global__ void w4_dequant_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales, int fmt,
                                  float alpha, __nv_bfloat16* __restrict__ out, long long n_groups8, int K) {
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;      // one thread = 8 values
  if (g >= n_groups8) return;
  const long long e0 = g * 8;
  const long long row = e0 / K;
  const int k = (int)(e0 - row * K);
  const uint32_t w = reinterpret_cast<const uint32_t*>(codes)[g];
  if (fmt == 2) {
    const uint32_t sm = reinterpret_cast<const uint32_t*>(scales)[row * (K / 32) + k / 32];
    uint32_t o[4];
    int4x8_to_bf16(w, __byte_perm(sm, 0, 0x1010), __byte_perm(sm, 0, 0x3232) ^ 0x80008000u, o);
    *reinterpret_cast<uint4*>(out + e0) = make_uint4(o[0], o[1], o[2], o[3]);
    return;
  }
  const int bs = fmt == 0 ? 16 : 32;
  const float sf = scale_to_float(scales[row * (K / bs) + k / bs], fmt) * alpha;
  uint32_t o[4];
  e2m1x8_to_bf16(w, pack_bf16x2(1.f, 1.f), o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = unpack_bf16x2(o[i]);
    o[i] = pack_bf16x2(f.x * sf, f.y * sf);
  }
  *reinterpret_cast<uint4*>(out + e0) = make_uint4(o[0], o[1], o[2], o[3]);
}

void w4_dequant_bf16(const void* codes, const void* scales, int fmt, float alpha, void* out, long long rows, int K,
                     cudaStream_t s) {
  const long long groups = rows * K / 8;
  if (groups <= 0) return;
  w4_dequant_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, s>>>((const uint8_t*)codes, (const uint8_t*)scales, fmt,
                                                                     alpha, (__nv_bfloat16*)out, groups, K);
  cuda_check(cudaGetLastError(), "w4_dequant_kernel");
}

template <int BN>
static void launch_w4(const CUtensorMap& tr, const CUtensorMap& tb, const W4Args& a, cudaStream_t s) {
  using S = W4Smem<BN>;
  static bool configured[kMaxDevices] = {};
  if (first_call_on_device(configured)) {
    cuda_check(cudaFuncSetAttribute(gemm_w4a16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal),
               "cudaFuncSetAttribute(gemm_w4a16_kernel)");
    cuda_check(cudaFuncSetAttribute(gemm_w4a16_kernel<BN>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                    cudaSharedmemCarveoutMaxShared), "cudaFuncSetAttribute(carveout)");
  }
  launch_pdl(gemm_w4a16_kernel<BN>, dim3(a.m_tiles, a.grid_y), dim3(kW4Threads), S::kTotal, s, tr, tb, a);
}

// y[T][N] = x[T][K] * dequant(codes, scales)^T * alpha (+ bias); T <= 128.
int linear_w4a16(const void* x, long long ldx, const void* codes, const void* scales, int fmt, float alpha,
                 const void* bias, void* y, long long ldy, int T, int N, int K, void* workspace, size_t workspace_bytes,
                 int* status, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (T > 128) throw std::runtime_error("linear_w4a16: at most 128 tokens per call (expand the weight for prefill)");
  if (K % 64 || N % 8 || (ldx & 7) || (ldy & 7)) throw std::runtime_error("linear_w4a16: K % 64, N % 8 and 16-byte rows required");
  if (fmt < 0 || fmt > 2) throw std::runtime_error("linear_w4a16: fmt must be 0 (NVFP4), 1 (MXFP4) or 2 (INT4G)");
  W4Args a{};
  a.M = N; a.N = T; a.K = K; a.m_tiles = (N + W4_BM - 1) / W4_BM; a.k_blocks = K / W4_BK; a.fmt = fmt;
  a.ldc = ldy; a.out = reinterpret_cast<__nv_bfloat16*>(y); a.scales = reinterpret_cast<const uint8_t*>(scales);
  a.alpha = alpha; a.bias = reinterpret_cast<const __nv_bfloat16*>(bias); a.status = status;
  const int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : 128;
  // Few feature tiles cannot pull the whole HBM bandwidth: split K over grid.y until the machine is full.
  const int slots = sm_count() * (bn <= 64 ? 2 : 1);
  int splits = 1;
  if (a.m_tiles * 2 <= slots && a.k_blocks >= 16) splits = std::min(std::min(slots / a.m_tiles, a.k_blocks / 8), 8);
  while (splits > 1 && (!workspace || (size_t)splits * T * N * 4 > workspace_bytes)) --splits;
  a.kb_per_split = ((a.k_blocks + splits - 1) / splits + 3) & ~3;      // code slots cover four K steps
  a.k_splits = (a.k_blocks + a.kb_per_split - 1) / a.kb_per_split;
  a.ws = reinterpret_cast<float*>(workspace);
  a.grid_y = a.k_splits;
  CUtensorMap tr = make_tmap_2d(codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, K / 2, W4_BM, 128, true);
  CUtensorMap tb = make_tmap_2d(x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, K, ldx * 2, bn, W4_BK, true);
  switch (bn) {
    case 16: launch_w4<16>(tr, tb, a, stream); break;
    case 32: launch_w4<32>(tr, tb, a, stream); break;
    case 64: launch_w4<64>(tr, tb, a, stream); break;
    default: launch_w4<128>(tr, tb, a, stream); break;
  }
  if (a.k_splits > 1) {
    const size_t n = (size_t)T * N;
    launch_pdl(w4_splitk_reduce_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, stream,
               (const float*)a.ws, a.k_splits, T, N, ldy, alpha, a.bias, a.out);
    return 2;
  }
  return 1;
}

// Grouped form over a device-built tile list (mixture of experts): y[row, :] = dequant(codes[e(row)]) * xp[row, :]
// (+ bias[e(row)]) for the permuted, per-expert padded rows of xp; `bn` is the token-tile width the list was
// built for (at most 128), `max_tiles` bounds the list.
int moe_grouped_linear_w4(const void* xp, long long ldx, const void* codes_stack, const void* scales_stack, int fmt,
                          float alpha, const void* bias_stack, void* y, long long ldy, int rows_cap, int n_out, int K,
                          int experts, const int* tile_expert, const int* tile_row0, const int* num_tiles, int max_tiles,
                          int bn, int* status, cudaStream_t stream) {
  if (rows_cap <= 0 || max_tiles <= 0) return 0;
  if (K % 64 || n_out % 8 || (ldx & 7) || (ldy & 7)) throw std::runtime_error("moe_grouped_linear_w4: K % 64, n_out % 8 and 16-byte rows required");
  if (fmt < 0 || fmt > 2) throw std::runtime_error("moe_grouped_linear_w4: fmt must be 0, 1 or 2");
  if (bn != 16 && bn != 32 && bn != 64 && bn != 128) throw std::runtime_error("moe_grouped_linear_w4: token tile must be 16, 32, 64 or 128");
  W4Args a{};
  a.M = n_out; a.N = rows_cap; a.K = K; a.m_tiles = (n_out + W4_BM - 1) / W4_BM; a.k_blocks = K / W4_BK; a.fmt = fmt;
  a.ldc = ldy; a.out = reinterpret_cast<__nv_bfloat16*>(y); a.scales = reinterpret_cast<const uint8_t*>(scales_stack);
  a.alpha = alpha; a.bias = reinterpret_cast<const __nv_bfloat16*>(bias_stack); a.status = status;
  a.k_splits = 1; a.kb_per_split = a.k_blocks;
  a.g_tile_expert = tile_expert; a.g_tile_row0 = tile_row0; a.g_num_tiles = num_tiles; a.g_rows = n_out;
  // when n_out is not a multiple of 128 the last feature tile of an expert also reads rows of the next expert's
  // codes (or zero fill past the stack); the epilogue never stores those rows
  CUtensorMap tr = make_tmap_2d(codes_stack, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)experts * n_out, K / 2, K / 2,
                                W4_BM, 128, true);
  CUtensorMap tb = make_tmap_2d(xp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_cap, K, ldx * 2, bn, W4_BK, true);
  a.grid_y = max_tiles;
  switch (bn) {
    case 16: launch_w4<16>(tr, tb, a, stream); break;
    case 32: launch_w4<32>(tr, tb, a, stream); break;
    case 64: launch_w4<64>(tr, tb, a, stream); break;
    default: launch_w4<128>(tr, tb, a, stream); break;
  }
  return 1;
}

}  // namespace fllm
