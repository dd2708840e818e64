// Multi-head latent attention over the compressed cache (DeepSeek-V2 / V3 family). A token stores one row of
// 576 values: the normalised KV latent (512) followed by the rotated shared key part (64). With the key
// up-projection absorbed into the query and the value up-projection applied after the softmax, every head is a
// query of width 576 against that one row per token, and its output is a weighted sum of the 512-wide latents:
// multi-query attention whose values are a prefix of its keys. The reference's counterparts are
// rust/engine/cuda/mla_latent.cu and mla_decode.cu (absorbed query, 576-wide cache).
//
// One CTA per (query row, group of HG heads); its NW warps take every NW-th key, keep an online softmax per
// head and are merged through shared memory. A key row is fetched once per warp and used by all HG heads, so the
// cache traffic out of L2 is 1 / HG of a kernel with one head per CTA. Lane l owns key elements [18 l, 18 l + 18)
// for the dot products and latent columns [16 l, 16 l + 16) for the output.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <stdexcept>

#include "fllm_ops.h"
#include "ptx.cuh"

namespace fllm {
namespace {
using bf16 = __nv_bfloat16;
constexpr int kLatent = 512, kRope = 64, kRow = kLatent + kRope;

template <int HG, int NW>
__global__ void __launch_bounds__(NW * 32) mla_attn_kernel(const bf16* __restrict__ q_abs, long long qa_t, long long qa_h,
                                                           const bf16* __restrict__ q_pe, const bf16* __restrict__ cache,
                                                           const int* __restrict__ block_tables, int max_blocks,
                                                           const int* __restrict__ row_seq, const int* __restrict__ positions,
                                                           bf16* __restrict__ out, long long o_t, long long o_h, int H, int block_size,
                                                           float scale) {
  constexpr int EK = kRow / 32, EV = kLatent / 32;      // 18 key elements and 16 latent columns per lane
  const int h0 = blockIdx.x * HG, t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_len = positions[t] + 1;
  const int* table = block_tables + (size_t)row_seq[t] * max_blocks;

  float qv[HG][EK];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    const int h = min(h0 + g, H - 1);                    // a ragged last group repeats the last head, unstored
    // element e of the 576-wide query: the absorbed part below 512, the rotated part above (pairs never straddle)
    const bf16* qa = q_abs + (size_t)t * qa_t + (size_t)h * qa_h;
    const bf16* qr = q_pe + ((size_t)t * H + h) * kRope;
#pragma unroll
    for (int j = 0; j < EK / 2; ++j) {
      const int e = lane * EK + 2 * j;
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(e < kLatent ? qa + e : qr + (e - kLatent)));
      qv[g][2 * j] = f.x * scale, qv[g][2 * j + 1] = f.y * scale;
    }
  }
  float m[HG], l[HG], acc[HG][EV];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    m[g] = -INFINITY, l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EV; ++e) acc[g][e] = 0.f;
  }
  for (int j = warp; j < kv_len; j += NW) {
    const bf16* row = cache + ((size_t)table[j / block_size] * block_size + (j % block_size)) * kRow;
    float kvv[EK], vv[EV];
    {
      const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(row + lane * EK);
#pragma unroll
      for (int e = 0; e < EK / 2; ++e) {
        const float2 f = __bfloat1622float2(kp[e]);
        kvv[2 * e] = f.x, kvv[2 * e + 1] = f.y;
      }
      const uint4* vp = reinterpret_cast<const uint4*>(row + lane * EV);
#pragma unroll
      for (int e = 0; e < EV / 8; ++e) {
        const uint4 raw = vp[e];
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(hh[i]);
          vv[8 * e + 2 * i] = f.x, vv[8 * e + 2 * i + 1] = f.y;
        }
      }
    }
    float s[HG];
#pragma unroll
    for (int g = 0; g < HG; ++g) {
      s[g] = 0.f;
#pragma unroll
      for (int e = 0; e < EK; ++e) s[g] = fmaf(qv[g][e], kvv[e], s[g]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int g = 0; g < HG; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
    }
#pragma unroll
    for (int g = 0; g < HG; ++g) {
      const float mn = fmaxf(m[g], s[g]);
      const float corr = __expf(m[g] - mn), p = __expf(s[g] - mn);
      l[g] = l[g] * corr + p;
#pragma unroll
      for (int e = 0; e < EV; ++e) acc[g][e] = fmaf(acc[g][e], corr, p * vv[e]);
      m[g] = mn;
    }
  }
  __shared__ float sm_m[NW][HG], sm_l[NW][HG];
  __shared__ float sm_acc[NW][HG][kLatent];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    if (lane == 0) sm_m[warp][g] = m[g], sm_l[warp][g] = l[g];
#pragma unroll
    for (int e = 0; e < EV; ++e) sm_acc[warp][g][lane * EV + e] = acc[g][e];
  }
  __syncthreads();
  // warp w merges heads w, w + NW, ... of the group
  for (int g = warp; g < HG; g += NW) {
    if (h0 + g >= H) break;
    float mm = sm_m[0][g];
#pragma unroll
    for (int w = 1; w < NW; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, o[EV];
#pragma unroll
    for (int e = 0; e < EV; ++e) o[e] = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float c = sm_m[w][g] == -INFINITY ? 0.f : __expf(sm_m[w][g] - mm);
      ll = fmaf(sm_l[w][g], c, ll);
#pragma unroll
      for (int e = 0; e < EV; ++e) o[e] = fmaf(sm_acc[w][g][lane * EV + e], c, o[e]);
    }
    const float inv = ll > 0.f ? 1.f / ll : 0.f;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * o_t + (size_t)(h0 + g) * o_h + lane * EV);
#pragma unroll
    for (int e = 0; e < EV / 2; ++e) op[e] = __floats2bfloat162_rn(o[2 * e] * inv, o[2 * e + 1] * inv);
  }
}

// ------------------------------------------------------------------------------------------ tensor-core path
// One CTA per (query row, 16 heads, slice of the keys): the 16 heads are the M rows of m16n8k16 MMAs, so the latent
// row of a key is read from shared memory once for all of them. Per tile of 64 keys (double-buffered cp.async):
//   warp w of 8 computes S[16 x 8] for keys 8 w .. 8 w + 7 over the 576-wide rows (Q fragments by ldmatrix from shared
//   memory), the row maxima meet in shared memory, P = exp2(S - max) goes to shared memory as bf16, and every warp
//   accumulates O[16 x 64] for its eighth of the 512 latent columns from the whole P (values = the first 512
//   entries of the same key rows, read by transposing ldmatrix).
// With more than one key slice per row the CTAs leave (max, sum, unnormalised O) in a workspace and a second kernel
// merges them.
constexpr int kTile = 64;
constexpr float kLog2e = 1.4426950408889634f;

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
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16-byte chunk c of row r of a row-major tile with W bf16 per row sits at chunk c ^ (r & 7): the eight rows of an
// ldmatrix fetch land in distinct banks although the row pitch is a multiple of 128 bytes.
template <int W>
__device__ __forceinline__ bf16* tile_at(bf16* base, int row, int chunk) {
  return base + row * W + ((chunk ^ (row & 7)) << 3);
}

constexpr int kTcWarps = 8;

struct MlaTcSmem {
  bf16 q[16 * kRow];
  bf16 k[2][kTile * kRow];
  bf16 p[16 * kTile];
  float wmax[kTcWarps][16];
  float wsum[kTcWarps][16];
};

// part_o [rows][splits][512] fp32 and part_ml [rows][splits][2] with rows = tokens * Hpad (Hpad = head groups * 16)
__global__ void __launch_bounds__(kTcWarps * 32) mla_tc_kernel(const bf16* __restrict__ q_abs, long long qa_t, long long qa_h,
                                                               const bf16* __restrict__ q_pe, const bf16* __restrict__ cache,
                                                               const int* __restrict__ block_tables, int max_blocks,
                                                               const int* __restrict__ row_seq, const int* __restrict__ positions,
                                                               bf16* __restrict__ out, long long o_t, long long o_h, int H,
                                                               int block_size, float scale_log2, int splits,
                                                               float* __restrict__ part_o, float* __restrict__ part_ml) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  MlaTcSmem& sm = *reinterpret_cast<MlaTcSmem*>(smem_raw);
  constexpr int NT = kTcWarps * 32;
  constexpr int KPW = kTile / kTcWarps;                      // 8 keys per warp in the S phase = one n-tile
  constexpr int CPW = kLatent / kTcWarps;                    // 64 latent columns per warp in the P V phase
  const int h0 = blockIdx.x * 16, t = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3, j4 = lane >> 3;
  const int kv_len = positions[t] + 1;
  const int* table = block_tables + (size_t)row_seq[t] * max_blocks;
  const int tiles = (kv_len + kTile - 1) / kTile;
  const int per = (tiles + splits - 1) / splits;
  const int tile_lo = split * per, tile_hi = min(tiles, tile_lo + per);
  const int Hpad = gridDim.x * 16;

  // queries of the 16 heads (zero rows past the last head)
  constexpr int CPR = kRow / 8;                              // 72 chunks of 16 bytes per row
  for (int i = tid; i < 16 * CPR; i += NT) {
    const int r = i / CPR, c = i - r * CPR;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (h0 + r < H) {
      const bf16* src = c < kLatent / 8 ? q_abs + (size_t)t * qa_t + (size_t)(h0 + r) * qa_h + c * 8
                                        : q_pe + ((size_t)t * H + h0 + r) * kRope + (c - kLatent / 8) * 8;
      v = *reinterpret_cast<const uint4*>(src);
    }
    *reinterpret_cast<uint4*>(tile_at<kRow>(sm.q, r, c)) = v;
  }
  // A warp brings in its KPW rows of the tile: lane r looks up the cache row of key r once, the address travels by
  // shuffle, and the 32 lanes copy the row's 72 chunks in three steps.
  auto load_tile = [&](int tile, int buf) {
    const int key0 = tile * kTile + warp * KPW;
    const bf16* mine = nullptr;
    if (lane < KPW && key0 + lane < kv_len) {
      const int key = key0 + lane;
      mine = cache + ((size_t)table[key / block_size] * block_size + (key % block_size)) * kRow;
    }
#pragma unroll
    for (int r = 0; r < KPW; ++r) {
      const unsigned long long addr = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(mine), r);
      const bf16* src = reinterpret_cast<const bf16*>(addr);
      const int row = warp * KPW + r;
#pragma unroll
      for (int c = lane; c < CPR; c += 32) {
        bf16* dst = tile_at<kRow>(sm.k[buf], row, c);
        if (src != nullptr) cp_async16(dst, src + c * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);   // masked keys must not feed NaNs into P V
      }
    }
  };
  float o[CPW / 8][4];
#pragma unroll
  for (int i = 0; i < CPW / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  if (tile_lo < tile_hi) load_tile(tile_lo, 0);
  cp_async_commit();
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int buf = (tile - tile_lo) & 1;
    if (tile + 1 < tile_hi) load_tile(tile + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    bf16* kt = sm.k[buf];
    // ---- S = Q K^T for this warp's 8 keys, two k-steps per round (one ldmatrix.x4 brings both B fragments)
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 3
    for (int kk = 0; kk < kRow / 16; kk += 2) {
      uint32_t a0[4], a1[4], b[4];
      ldsm_x4(a0, tile_at<kRow>(sm.q, lane & 15, 2 * kk + (lane >> 4)));
      ldsm_x4(a1, tile_at<kRow>(sm.q, lane & 15, 2 * kk + 2 + (lane >> 4)));
      ldsm_x4(b, tile_at<kRow>(kt, warp * KPW + (lane & 7), 2 * kk + j4));
      mma_bf16(s, a0, b[0], b[1]);
      mma_bf16(s, a1, b[2], b[3]);
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = tile * kTile + warp * KPW + 2 * tq + (e & 1);
      const float v = key < kv_len ? s[e] * scale_log2 : -INFINITY;
      s[e] = v;
      if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if (tq == 0) sm.wmax[warp][g] = mx0, sm.wmax[warp][g + 8] = mx1;
    __syncthreads();
    float mn0 = m0, mn1 = m1;
#pragma unroll
    for (int w = 0; w < kTcWarps; ++w) mn0 = fmaxf(mn0, sm.wmax[w][g]), mn1 = fmaxf(mn1, sm.wmax[w][g + 8]);
    // a tile inside [tile_lo, tile_hi) starts below kv_len, so every row has seen a finite score by now
    const float c0 = m0 == -INFINITY ? 0.f : exp2f(m0 - mn0), c1 = m1 == -INFINITY ? 0.f : exp2f(m1 - mn1);
    m0 = mn0, m1 = mn1;
    {
      const float p0 = exp2f(s[0] - mn0), p1 = exp2f(s[1] - mn0), p2 = exp2f(s[2] - mn1), p3 = exp2f(s[3] - mn1);
      l0 = l0 * c0 + p0 + p1, l1 = l1 * c1 + p2 + p3;
      const int col = warp * KPW + 2 * tq;
      *reinterpret_cast<__nv_bfloat162*>(tile_at<kTile>(sm.p, g, col >> 3) + (col & 7)) = __floats2bfloat162_rn(p0, p1);
      *reinterpret_cast<__nv_bfloat162*>(tile_at<kTile>(sm.p, g + 8, col >> 3) + (col & 7)) = __floats2bfloat162_rn(p2, p3);
    }
#pragma unroll
    for (int i = 0; i < CPW / 8; ++i) o[i][0] *= c0, o[i][1] *= c0, o[i][2] *= c1, o[i][3] *= c1;
    __syncthreads();
    // ---- O += P V for this warp's 64 latent columns
#pragma unroll
    for (int kq = 0; kq < kTile / 16; ++kq) {
      uint32_t pa[4];
      ldsm_x4(pa, tile_at<kTile>(sm.p, lane & 15, 2 * kq + (lane >> 4)));
#pragma unroll
      for (int db = 0; db < CPW / 8; db += 2) {
        uint32_t b[4];
        ldsm_x4_t(b, tile_at<kRow>(kt, kq * 16 + (j4 & 1) * 8 + (lane & 7), warp * (CPW / 8) + db + (j4 >> 1)));
        mma_bf16(o[db], pa, b[0], b[1]);
        mma_bf16(o[db + 1], pa, b[2], b[3]);
      }
    }
    __syncthreads();                                          // P, the maxima and this key buffer are free again
  }
  cp_async_wait<0>();
  // ---- row sums over the quad and the warps
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (tq == 0) sm.wsum[warp][g] = l0, sm.wsum[warp][g + 8] = l1;
  __syncthreads();
  float L0 = 0.f, L1 = 0.f;
#pragma unroll
  for (int w = 0; w < kTcWarps; ++w) L0 += sm.wsum[w][g], L1 += sm.wsum[w][g + 8];
  if (splits == 1) {
    const float i0 = L0 > 0.f ? 1.f / L0 : 0.f, i1 = L1 > 0.f ? 1.f / L1 : 0.f;
#pragma unroll
    for (int db = 0; db < CPW / 8; ++db) {
      const int col = warp * CPW + db * 8 + 2 * tq;
      if (h0 + g < H)
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * o_t + (size_t)(h0 + g) * o_h + col) = __floats2bfloat162_rn(o[db][0] * i0, o[db][1] * i0);
      if (h0 + g + 8 < H)
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * o_t + (size_t)(h0 + g + 8) * o_h + col) = __floats2bfloat162_rn(o[db][2] * i1, o[db][3] * i1);
    }
    return;
  }
  const size_t r0 = ((size_t)t * Hpad + h0 + g) * splits + split, r1 = ((size_t)t * Hpad + h0 + g + 8) * splits + split;
  if (warp == 0 && tq == 0) {
    part_ml[2 * r0] = m0, part_ml[2 * r0 + 1] = L0;
    part_ml[2 * r1] = m1, part_ml[2 * r1 + 1] = L1;
  }
#pragma unroll
  for (int db = 0; db < CPW / 8; ++db) {
    const int col = warp * CPW + db * 8 + 2 * tq;
    *reinterpret_cast<float2*>(part_o + r0 * kLatent + col) = make_float2(o[db][0], o[db][1]);
    *reinterpret_cast<float2*>(part_o + r1 * kLatent + col) = make_float2(o[db][2], o[db][3]);
  }
}

// out(t, h) = sum_s exp2(m_s - m) O_s / sum_s exp2(m_s - m) l_s; grid (H, tokens), 128 threads x 4 columns
__global__ void __launch_bounds__(128) mla_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                                                        int Hpad, bf16* __restrict__ out, long long o_t, long long o_h) {
  const int h = blockIdx.x, t = blockIdx.y;
  const size_t r = ((size_t)t * Hpad + h) * splits;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[2 * (r + s)]);
  float L = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[2 * (r + s)];
    if (ms == -INFINITY) continue;                           // a slice with no keys
    const float c = exp2f(ms - mm);
    L = fmaf(part_ml[2 * (r + s) + 1], c, L);
    const float4 v = *reinterpret_cast<const float4*>(part_o + (r + s) * kLatent + threadIdx.x * 4);
    acc.x = fmaf(v.x, c, acc.x), acc.y = fmaf(v.y, c, acc.y), acc.z = fmaf(v.z, c, acc.z), acc.w = fmaf(v.w, c, acc.w);
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * o_t + (size_t)h * o_h + threadIdx.x * 4);
  op[0] = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
  op[1] = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
}

// Per token: RMSNorm of the 512 latent values and rotation of the 64 shared key values into the token's cache row
// (skipped for padding rows, slot < 0), and rotation of every head's 64 query values into q_pe [T][H][64]. Pairs are
// neighbours (x[2i], x[2i+1]); cos / sin carry the YaRN attention factor.
__global__ void __launch_bounds__(128) mla_prepare_kernel(const bf16* __restrict__ ckv, long long ldc, const bf16* __restrict__ q, long long ldq,
                                                          int q_head_stride, int q_rope_offset, const int* __restrict__ positions,
                                                          const int* __restrict__ slots, const float* __restrict__ inv_freq, float attn_factor,
                                                          const bf16* __restrict__ norm_w, float eps, bf16* __restrict__ cache,
                                                          bf16* __restrict__ q_pe, int H) {
  const int t = blockIdx.x, tid = threadIdx.x;
  const float pos = (float)positions[t];
  const int slot = slots[t];
  const bf16* row = ckv + (size_t)t * ldc;
  // latent: four values per thread
  float v[4], ss = 0.f;
  {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(row + tid * 4);
    const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
    ss = a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
  }
  __shared__ float part[4];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) part[tid >> 5] = ss;
  __syncthreads();
  const float inv = rsqrtf((part[0] + part[1] + part[2] + part[3]) / kLatent + eps);
  if (slot >= 0) {
    bf16* dst = cache + (size_t)slot * kRow;
    __nv_bfloat162* d = reinterpret_cast<__nv_bfloat162*>(dst + tid * 4);
    const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(norm_w + tid * 4);
    const float2 w0 = __bfloat1622float2(w[0]), w1 = __bfloat1622float2(w[1]);
    d[0] = __floats2bfloat162_rn(v[0] * inv * w0.x, v[1] * inv * w0.y);
    d[1] = __floats2bfloat162_rn(v[2] * inv * w1.x, v[3] * inv * w1.y);
    if (tid < kRope / 2) {
      float sn, cs;
      sincosf(pos * inv_freq[tid], &sn, &cs);
      sn *= attn_factor, cs *= attn_factor;
      const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + kLatent + 2 * tid));
      *reinterpret_cast<__nv_bfloat162*>(dst + kLatent + 2 * tid) = __floats2bfloat162_rn(x.x * cs - x.y * sn, x.x * sn + x.y * cs);
    }
  }
  for (int i = tid; i < H * (kRope / 2); i += 128) {
    const int h = i / (kRope / 2), f = i % (kRope / 2);
    float sn, cs;
    sincosf(pos * inv_freq[f], &sn, &cs);
    sn *= attn_factor, cs *= attn_factor;
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q + (size_t)t * ldq + (size_t)h * q_head_stride + q_rope_offset + 2 * f));
    *reinterpret_cast<__nv_bfloat162*>(q_pe + ((size_t)t * H + h) * kRope + 2 * f) = __floats2bfloat162_rn(x.x * cs - x.y * sn, x.x * sn + x.y * cs);
  }
}
}  // namespace

// q_abs: absorbed query part, element (t, h, e) at q_abs[t * qa_t + h * qa_h + e] (e < 512); q_pe [tokens][H][64] rotated
// query part; cache [blocks][block_size][576]; out element (t, h, e) at out[t * o_t + h * o_h + e].
size_t attention_mla_workspace_bytes(int tokens, int H, int splits) {
  const size_t rows = (size_t)tokens * ((H + 15) / 16 * 16) * splits;
  return rows * (kLatent + 2) * sizeof(float);
}

// How many key slices a step gets: enough CTAs for the machine, at least four tiles of keys per slice.
int attention_mla_splits(int tokens, int H, int max_kv_len) {
  const int ctas = tokens * ((H + 15) / 16);
  const int tiles = (max_kv_len + kTile - 1) / kTile;
  int splits = 1;
  while (splits < 16 && ctas * splits < 148 && tiles / (splits * 2) >= 4) splits *= 2;
  return splits;
}

// Tensor-core path. workspace: attention_mla_workspace_bytes(tokens, H, splits) bytes when splits > 1.
void attention_mla_tc_bf16(const void* q_abs, long long qa_t, long long qa_h, const void* q_pe, const void* cache, const int* block_tables,
                           int max_blocks, const int* row_seq, const int* positions, void* out, long long o_t, long long o_h, int tokens,
                           int H, int block_size, float scale, int splits, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  if (tokens <= 0) return;
  if ((qa_t & 7) || (qa_h & 7) || (o_t & 1) || (o_h & 1) || (reinterpret_cast<uintptr_t>(cache) & 15) ||
      (reinterpret_cast<uintptr_t>(q_abs) & 15) || (reinterpret_cast<uintptr_t>(q_pe) & 15) || (reinterpret_cast<uintptr_t>(out) & 3))
    throw std::runtime_error("attention_mla_tc_bf16: 16-byte aligned query rows and cache, even output strides are required");
  if (splits < 1) splits = 1;
  if (splits > 1 && workspace_bytes < attention_mla_workspace_bytes(tokens, H, splits))
    throw std::runtime_error("attention_mla_tc_bf16: workspace too small for the requested key slices");
  static bool configured = false;                            // per process; every device of a process runs the same binary
  if (!configured) {
    cudaFuncSetAttribute(mla_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(MlaTcSmem));
    configured = true;
  }
  const int groups = (H + 15) / 16;
  float* po = static_cast<float*>(workspace);
  float* pml = splits > 1 ? po + (size_t)tokens * groups * 16 * splits * kLatent : nullptr;
  mla_tc_kernel<<<dim3(groups, tokens, splits), kTcWarps * 32, sizeof(MlaTcSmem), s>>>(
      static_cast<const bf16*>(q_abs), qa_t, qa_h, static_cast<const bf16*>(q_pe), static_cast<const bf16*>(cache), block_tables, max_blocks,
      row_seq, positions, static_cast<bf16*>(out), o_t, o_h, H, block_size, scale * kLog2e, splits, po, pml);
  if (splits > 1)
    mla_merge_kernel<<<dim3(H, tokens), 128, 0, s>>>(po, pml, splits, groups * 16, static_cast<bf16*>(out), o_t, o_h);
}

void attention_mla_bf16(const void* q_abs, long long qa_t, long long qa_h, const void* q_pe, const void* cache, const int* block_tables,
                        int max_blocks, const int* row_seq, const int* positions, void* out, long long o_t, long long o_h, int tokens,
                        int H, int block_size, float scale, cudaStream_t s) {
  if (tokens <= 0) return;
  if ((qa_t & 1) || (qa_h & 1) || (o_t & 1) || (o_h & 1) || (reinterpret_cast<uintptr_t>(cache) & 15) ||
      (reinterpret_cast<uintptr_t>(q_abs) & 3) || (reinterpret_cast<uintptr_t>(q_pe) & 3) || (reinterpret_cast<uintptr_t>(out) & 3))
    throw std::runtime_error("attention_mla_bf16: even strides, 4-byte aligned queries / output and a 16-byte aligned cache are required");
  // Few rows (decode): two heads per CTA and eight warps over the keys, so that a step fills the machine and a warp
  // walks an eighth of the context; many rows (prefill): four heads per CTA, which quarters the cache traffic out of L2.
  const bf16* qa = static_cast<const bf16*>(q_abs);
  const bf16* qr = static_cast<const bf16*>(q_pe);
  const bf16* cp = static_cast<const bf16*>(cache);
  bf16* op = static_cast<bf16*>(out);
  if ((long long)((H + 3) / 4) * tokens < 2 * 148) {
    mla_attn_kernel<2, 8><<<dim3((H + 1) / 2, tokens), 256, 0, s>>>(qa, qa_t, qa_h, qr, cp, block_tables, max_blocks, row_seq, positions, op,
                                                                   o_t, o_h, H, block_size, scale);
  } else {
    mla_attn_kernel<4, 4><<<dim3((H + 3) / 4, tokens), 128, 0, s>>>(qa, qa_t, qa_h, qr, cp, block_tables, max_blocks, row_seq, positions, op,
                                                                   o_t, o_h, H, block_size, scale);
  }
}

// ckv [tokens][>= 576] (latent | shared key part, leading dimension ldc); q [tokens][H][head] with the 64 rotary values of a
// head at q_rope_offset; cache rows are addressed by slot (block * block_size + offset; negative = no write).
void mla_prepare_bf16(const void* ckv, long long ldc, const void* q, long long ldq, int q_head_stride, int q_rope_offset,
                      const int* positions, const int* slots, const float* inv_freq, float attn_factor, const void* norm_w, float eps,
                      void* cache, void* q_pe, int tokens, int H, cudaStream_t s) {
  if (tokens <= 0) return;
  if ((ldc & 1) || (ldq & 1) || (q_head_stride & 1) || (q_rope_offset & 1) || (reinterpret_cast<uintptr_t>(ckv) & 3) ||
      (reinterpret_cast<uintptr_t>(q) & 3) || (reinterpret_cast<uintptr_t>(cache) & 3) || (reinterpret_cast<uintptr_t>(norm_w) & 3))
    throw std::runtime_error("mla_prepare_bf16: even strides and 4-byte aligned tensors are required");
  mla_prepare_kernel<<<tokens, 128, 0, s>>>(static_cast<const bf16*>(ckv), ldc, static_cast<const bf16*>(q), ldq, q_head_stride, q_rope_offset,
                                            positions, slots, inv_freq, attn_factor, static_cast<const bf16*>(norm_w), eps,
                                            static_cast<bf16*>(cache), static_cast<bf16*>(q_pe), H);
}

}  // namespace fllm
