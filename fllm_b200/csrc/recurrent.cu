// Recurrent token mixers on ragged batches: depthwise causal convolution, the Mamba-1 and Mamba-2 selective scans,
// and the matrix-state family (RWKV-6, RWKV-7, gated delta rule, Kimi delta attention) plus the gated RMSNorm that
// follows a scan. The reference keeps one file per family (rust/engine/cuda/mamba1.cu, mamba2.cu, rwkv.cu,
// deltanet.cu, kda.cu, shortconv.cu) and a chunk-parallel scan (scan.cu); here every family walks its tokens with the
// state held in registers, one CTA per (sequence, head, slice of state rows): a step touches each state element
// once, so the work per token is the state size and the per-token inputs are prefetched one token ahead. With 148 SMs
// the grid is sequences x heads x row tiles, which covers the machine from one 2048-token prefill chunk upwards.
//
// Batch layout (shared by every kernel): q_starts[B + 1] = first token row of each sequence, seq_state[B] = row of the
// state pool that belongs to the sequence, positions[T]: a sequence whose first token of the step sits at position 0
// starts from a zero state. States live in fp32 (convolution windows in bf16: they are copies of bf16 inputs).
#include <algorithm>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "fllm_ops.h"

namespace fllm {
namespace {
using bf16 = __nv_bfloat16;

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// n consecutive bf16 values (n a multiple of 8, 16-byte aligned) widened into fp32 registers
template <int N>
__device__ __forceinline__ void load_bf16(const bf16* __restrict__ p, float (&out)[N]) {
  static_assert(N % 8 == 0, "slices are whole 16-byte words");
#pragma unroll
  for (int i = 0; i < N / 8; ++i) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p + 8 * i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      out[8 * i + 2 * j] = f.x;
      out[8 * i + 2 * j + 1] = f.y;
    }
  }
}
template <int N>
__device__ __forceinline__ void load_f32(const float* __restrict__ p, float (&out)[N]) {
#pragma unroll
  for (int i = 0; i < N / 4; ++i) {
    const float4 v = *reinterpret_cast<const float4*>(p + 4 * i);
    out[4 * i] = v.x, out[4 * i + 1] = v.y, out[4 * i + 2] = v.z, out[4 * i + 3] = v.w;
  }
}
template <int N>
__device__ __forceinline__ void store_f32(float* __restrict__ p, const float (&v)[N]) {
#pragma unroll
  for (int i = 0; i < N / 4; ++i)
    *reinterpret_cast<float4*>(p + 4 * i) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}
// sum over the LANES consecutive lanes that share one state row (LANES a power of two up to 32)
template <int LANES>
__device__ __forceinline__ float row_sum(float v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------------------ causal conv1d
// One CTA per (128 channels, sequence, run of `seg_tokens` tokens): the tokens of the run are spread over threadIdx.y,
// every thread owns two neighbouring channels. Only the CTA of a sequence's first run reads the sequence's window for
// its channels (later runs see their whole history in x, which nothing writes), so after a barrier that CTA moves the
// window forward in place. The last run of the grid goes on to the sequence's end.
template <int W>
__global__ void __launch_bounds__(256) conv1d_kernel(const bf16* __restrict__ x, long long ldx, const float* __restrict__ w,
                                                     const float* __restrict__ bias, bf16* __restrict__ state,
                                                     const int* __restrict__ q_starts, const int* __restrict__ seq_state,
                                                     const int* __restrict__ positions, bf16* __restrict__ y, long long ldy,
                                                     int C, int act, int seg_tokens) {
  const int s = blockIdx.y;
  const int c = (blockIdx.x * 64 + threadIdx.x) * 2;
  const int t0 = q_starts[s], n = q_starts[s + 1] - t0;
  const int p_lo = blockIdx.z * seg_tokens, p_hi = blockIdx.z + 1 == gridDim.z ? n : min(n, p_lo + seg_tokens);
  if (n <= 0 || (p_lo >= n && blockIdx.z != 0)) return;
  const bool active = c < C;
  const bool fresh = positions[t0] == 0;
  bf16* st = state + (long long)seq_state[s] * (W - 1) * C;
  float wv[2][W], hist[2][W - 1], bv[2] = {0.f, 0.f};
  if (active) {
#pragma unroll
    for (int j = 0; j < W; ++j) wv[0][j] = w[(long long)c * W + j], wv[1][j] = w[(long long)(c + 1) * W + j];
    if (bias != nullptr) bv[0] = bias[c], bv[1] = bias[c + 1];
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
      float2 h = make_float2(0.f, 0.f);
      if (!fresh && blockIdx.z == 0) h = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(st + (long long)j * C + c));
      hist[0][j] = h.x, hist[1][j] = h.y;
    }
    // each row of threads walks a contiguous piece of the run with the last W - 1 inputs in registers: one load per token
    const int per = (p_hi - p_lo + (int)blockDim.y - 1) / (int)blockDim.y;
    const int a0 = p_lo + (int)threadIdx.y * per, a1 = min(p_hi, a0 + per);
    float win[2][W - 1];
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
      const int i = a0 - (W - 1) + j;
      float2 v = make_float2(0.f, 0.f);
      if (a0 < a1) {
        if (i >= 0) v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + (long long)(t0 + i) * ldx + c));
        else v = make_float2(hist[0][(W - 1) + i], hist[1][(W - 1) + i]);
      }
      win[0][j] = v.x, win[1][j] = v.y;
    }
#pragma unroll 4
    for (int p = a0; p < a1; ++p) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + (long long)(t0 + p) * ldx + c));
      float o0 = fmaf(wv[0][W - 1], v.x, bv[0]), o1 = fmaf(wv[1][W - 1], v.y, bv[1]);
#pragma unroll
      for (int j = 0; j < W - 1; ++j) o0 = fmaf(wv[0][j], win[0][j], o0), o1 = fmaf(wv[1][j], win[1][j], o1);
#pragma unroll
      for (int j = 0; j + 1 < W - 1; ++j) win[0][j] = win[0][j + 1], win[1][j] = win[1][j + 1];
      win[0][W - 2] = v.x, win[1][W - 2] = v.y;
      if (act) o0 = silu_f(o0), o1 = silu_f(o1);
      *reinterpret_cast<__nv_bfloat162*>(y + (long long)(t0 + p) * ldy + c) = __floats2bfloat162_rn(o0, o1);
    }
  }
  if (blockIdx.z != 0) return;
  __syncthreads();
  if (active && threadIdx.y == 0) {
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
      const int i = n - (W - 1) + j;
      __nv_bfloat162 v;
      if (i >= 0) v = *reinterpret_cast<const __nv_bfloat162*>(x + (long long)(t0 + i) * ldx + c);
      else v = __floats2bfloat162_rn(hist[0][(W - 1) + i], hist[1][(W - 1) + i]);
      *reinterpret_cast<__nv_bfloat162*>(st + (long long)j * C + c) = v;
    }
  }
}

// ------------------------------------------------------------------------------------------ Mamba-2 (SSD)
// h[p][n] = exp(dt A) h[p][n] + dt x[p] B[n];  y[p] = sum_n h[p][n] C[n] + D x[p]      (one A, dt, D per head)
//
// Long prompts of few sequences leave most SMs idle if a sequence is walked by one CTA per (head, row tile). The
// recurrence is diagonal, so a sequence can be cut into segments of `seg_len` tokens that run side by side:
//   kLocal    every segment but the last runs from a zero state and leaves its end state and the sum of its time steps;
//   combine   start state of segment s + 1 = end state of s + exp(A sum dt_s) * start state of s (a short serial pass);
//   kFinal    every segment runs again from its true start state and writes y; the segment with the sequence's last token
//             stores the state. Sequences of one segment (decode rows of a mixed step) run only here, as the plain walk.
// Twice the arithmetic, `segs` times the parallelism. kWhole is the plain walk (decode, short chunks, large batches).
enum { kWhole = 0, kLocal = 1, kFinal = 2 };
struct Mamba2Args {
  const bf16 *x, *dt, *Bm, *Cm;
  long long ldx, lddt, ldb, ldc, ldy;
  const float *A, *D, *dt_bias;
  float* state;                 // [slots][H][P][N]
  const int *q_starts, *seq_state, *positions;
  bf16* y;
  int H, P, G;
  float dt_min, dt_max;
  int skip_from;                // sequences with at least this many tokens in the step are left to another path (0 = none)
  int seg_len, segs;            // segmented modes only
  float* seg_state;             // [B][segs - 1][H][P][N]: end states (kLocal), then start states of segments 1.. (combine)
  float* seg_start0;            // [B][H][P][N]: a continued sequence's state before the step, copied by combine, so that
                                // kFinal's first segment does not read the pool row that its last segment overwrites
  float* seg_dt;                // [B][segs - 1][H]: sum of the time steps of a segment
};

template <int N, int NPT, int MODE>
__global__ void __launch_bounds__(128) mamba2_scan_kernel(const Mamba2Args a) {
  constexpr int TPN = N / NPT, ROWS = 128 / TPN;
  const int ptiles = (a.P + ROWS - 1) / ROWS;
  const int h = blockIdx.x / ptiles, p = (blockIdx.x % ptiles) * ROWS + threadIdx.x / TPN;
  const int ln = threadIdx.x % TPN, s = blockIdx.y, seg = MODE == kWhole ? 0 : blockIdx.z;
  const int t0 = a.q_starts[s], n = a.q_starts[s + 1] - t0;
  if (n <= 0 || (a.skip_from > 0 && n >= a.skip_from)) return;
  const bool valid = p < a.P;
  const int pc = valid ? p : a.P - 1;                        // lanes of a ragged last tile repeat the last row, unstored
  float* st = a.state + (((long long)a.seq_state[s] * a.H + h) * a.P + pc) * N + ln * NPT;
  float* sg = nullptr;                                       // this thread's slice of seg_state[s][.]
  if (MODE != kWhole) sg = a.seg_state + ((((long long)s * (a.segs - 1)) * a.H + h) * a.P + pc) * N + ln * NPT;
  const long long seg_stride = (long long)a.H * a.P * N;
  // tokens [lo, hi) of the sequence's step
  // (the last segment of kFinal runs to the end of the step even if `segs` was sized for a shorter one)
  // the segment that holds the sequence's last token stores the state; segments after it (short sequences, decode rows of a
  // mixed step) have nothing to do, and a sequence of one segment runs as the plain walk inside kFinal
  const int seg_last = MODE == kWhole ? 0 : min(a.segs - 1, (n - 1) / a.seg_len);
  if ((MODE == kLocal && seg >= seg_last) || (MODE == kFinal && seg > seg_last)) return;
  const int lo = MODE == kWhole ? 0 : seg * a.seg_len;
  const int hi = (MODE == kWhole || (MODE == kFinal && seg == seg_last)) ? n : (seg + 1) * a.seg_len;
  float hs[NPT];
  const bool from_pool = MODE == kWhole || (MODE == kFinal && seg == 0);
  if (MODE == kLocal || (from_pool && a.positions[t0] == 0)) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) hs[i] = 0.f;
  } else if (from_pool) {
    load_f32<NPT>(MODE == kFinal && seg_last > 0 ? a.seg_start0 + (((long long)s * a.H + h) * a.P + pc) * N + ln * NPT : st, hs);
  } else {
    load_f32<NPT>(sg + (seg - 1) * seg_stride, hs);
  }
  const int g = h / (a.H / a.G);
  const float A = a.A[h], D = a.D != nullptr ? a.D[h] : 0.f, dtb = a.dt_bias != nullptr ? a.dt_bias[h] : 0.f;
  float dt_sum = 0.f;
  if (lo < hi) {
    const long long tb = t0 + lo;
    const bf16* xp = a.x + tb * a.ldx + h * a.P + pc;
    const bf16* dtp = a.dt + tb * a.lddt + h;
    const bf16* bp = a.Bm + tb * a.ldb + g * N + ln * NPT;
    const bf16* cp = a.Cm + tb * a.ldc + g * N + ln * NPT;
    bf16* yp = a.y + tb * a.ldy + h * a.P + pc;
    float Bn[NPT], Cn[NPT], xn = __bfloat162float(*xp), dtn = __bfloat162float(*dtp);
    load_bf16<NPT>(bp, Bn);
    if (MODE != kLocal) load_bf16<NPT>(cp, Cn);
    for (int t = lo; t < hi; ++t) {
      float Bc[NPT], Cc[NPT];
      const float xv = xn;
      float dt = softplus_f(dtn + dtb);
      dt = fminf(fmaxf(dt, a.dt_min), a.dt_max);
#pragma unroll
      for (int i = 0; i < NPT; ++i) Bc[i] = Bn[i], Cc[i] = Cn[i];
      if (t + 1 < hi) {                                       // next token's inputs travel while this one is applied
        xp += a.ldx, dtp += a.lddt, bp += a.ldb, cp += a.ldc;
        xn = __bfloat162float(*xp), dtn = __bfloat162float(*dtp);
        load_bf16<NPT>(bp, Bn);
        if (MODE != kLocal) load_bf16<NPT>(cp, Cn);
      }
      const float dA = __expf(dt * A), dx = dt * xv;
      dt_sum += dt;
      if (MODE == kLocal) {
#pragma unroll
        for (int i = 0; i < NPT; ++i) hs[i] = fmaf(hs[i], dA, dx * Bc[i]);
      } else {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};                  // four chains instead of one of NPT dependent adds
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
          hs[i] = fmaf(hs[i], dA, dx * Bc[i]);
          acc[i & 3] = fmaf(hs[i], Cc[i], acc[i & 3]);
        }
        const float tot = row_sum<TPN>((acc[0] + acc[1]) + (acc[2] + acc[3]));
        if (ln == 0 && valid) *yp = __float2bfloat16(fmaf(D, xv, tot));
        yp += a.ldy;
      }
    }
  }
  if (MODE == kLocal) {
    if (valid) store_f32<NPT>(sg + seg * seg_stride, hs);
    if (blockIdx.x % ptiles == 0 && threadIdx.x == 0) a.seg_dt[((long long)s * (a.segs - 1) + seg) * a.H + h] = dt_sum;
  } else if (valid && (MODE == kWhole || seg == seg_last)) {
    store_f32<NPT>(st, hs);
  }
}

// start[seg + 1] = end_local[seg] + exp(A sum dt[seg]) * start[seg], in place over seg_state; one thread per four state values
__global__ void mamba2_combine_kernel(const Mamba2Args a, int N) {
  const long long per_seq = (long long)a.H * a.P * N;
  const long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const int s = blockIdx.y;
  if (i4 >= per_seq) return;
  const int t0 = a.q_starts[s];
  const int n = a.q_starts[s + 1] - t0;
  if (n <= 0 || (a.skip_from > 0 && n >= a.skip_from)) return;
  const int seg_last = min(a.segs - 1, (n - 1) / a.seg_len);
  if (seg_last == 0) return;
  const int h = (int)(i4 / ((long long)a.P * N));
  float4 carry = make_float4(0.f, 0.f, 0.f, 0.f);
  if (a.positions[t0] != 0) {
    carry = *reinterpret_cast<const float4*>(a.state + (long long)a.seq_state[s] * per_seq + i4);
    *reinterpret_cast<float4*>(a.seg_start0 + (long long)s * per_seq + i4) = carry;
  }
  float* sg = a.seg_state + (long long)s * (a.segs - 1) * per_seq + i4;
  const float A = a.A[h];
  for (int seg = 0; seg < seg_last; ++seg) {
    const float d = __expf(A * a.seg_dt[((long long)s * (a.segs - 1) + seg) * a.H + h]);
    float4 e = *reinterpret_cast<const float4*>(sg + seg * per_seq);
    carry = make_float4(fmaf(carry.x, d, e.x), fmaf(carry.y, d, e.y), fmaf(carry.z, d, e.z), fmaf(carry.w, d, e.w));
    *reinterpret_cast<float4*>(sg + seg * per_seq) = carry;
  }
}

// ------------------------------------------------------------------------------------------ Mamba-1
// h[d][n] = exp(dt[d] A[d][n]) h[d][n] + dt[d] B[n] x[d];  y[d] = (sum_n h[d][n] C[n] + D[d] x[d]) * silu(z[d])
struct Mamba1Args {
  const bf16 *x, *dt, *Bm, *Cm, *z;
  long long ldx, lddt, ldb, ldc, ldz, ldy;
  const float *A, *D, *dt_bias;   // A [Dm][N]
  float* state;                   // [slots][Dm][N]
  const int *q_starts, *seq_state, *positions;
  bf16* y;
  int Dm;
  int seg_len, segs;              // sequence-parallel form (see the Mamba-2 kernel): segments, then combine, then the outputs
  float* seg_state;               // [B][segs - 1][Dm][N]
  float* seg_start0;              // [B][Dm][N]: a continued sequence's state before the step (written by combine)
  float* seg_dt;                  // [B][segs - 1][Dm]: sum of a channel's time steps over a segment
};

template <int N, int MODE>
__global__ void __launch_bounds__(128) mamba1_scan_kernel(const Mamba1Args a) {
  const int d = blockIdx.x * 128 + threadIdx.x, s = blockIdx.y, seg = MODE == kWhole ? 0 : blockIdx.z;
  const int t0 = a.q_starts[s], n = a.q_starts[s + 1] - t0;
  if (n <= 0 || d >= a.Dm) return;
  float* st = a.state + ((long long)a.seq_state[s] * a.Dm + d) * N;
  const long long seg_stride = (long long)a.Dm * N;
  float* sg = MODE == kWhole ? nullptr : a.seg_state + ((long long)s * (a.segs - 1) * a.Dm + d) * N;
  const int seg_last = MODE == kWhole ? 0 : min(a.segs - 1, (n - 1) / a.seg_len);
  if ((MODE == kLocal && seg >= seg_last) || (MODE == kFinal && seg > seg_last)) return;
  const int lo = MODE == kWhole ? 0 : seg * a.seg_len;
  const int hi = (MODE == kWhole || (MODE == kFinal && seg == seg_last)) ? n : (seg + 1) * a.seg_len;
  float hs[N], A[N];
  load_f32<N>(a.A + (long long)d * N, A);
  const bool from_pool = MODE == kWhole || (MODE == kFinal && seg == 0);
  if (MODE == kLocal || (from_pool && a.positions[t0] == 0)) {
#pragma unroll
    for (int i = 0; i < N; ++i) hs[i] = 0.f;
  } else if (from_pool) {
    load_f32<N>(MODE == kFinal && seg_last > 0 ? a.seg_start0 + ((long long)s * a.Dm + d) * N : st, hs);
  } else {
    load_f32<N>(sg + (seg - 1) * seg_stride, hs);
  }
  const float D = a.D != nullptr ? a.D[d] : 0.f, dtb = a.dt_bias != nullptr ? a.dt_bias[d] : 0.f;
  float dt_sum = 0.f;
  for (int t = t0 + lo; t < t0 + hi; ++t) {
    float Bc[N], Cc[N];
    load_bf16<N>(a.Bm + (long long)t * a.ldb, Bc);           // the same words for the whole warp: one broadcast fetch
    if (MODE != kLocal) load_bf16<N>(a.Cm + (long long)t * a.ldc, Cc);
    const float xv = __bfloat162float(a.x[(long long)t * a.ldx + d]);
    const float dt = softplus_f(__bfloat162float(a.dt[(long long)t * a.lddt + d]) + dtb);
    const float dx = dt * xv;
    dt_sum += dt;
    if (MODE == kLocal) {
#pragma unroll
      for (int i = 0; i < N; ++i) hs[i] = fmaf(hs[i], __expf(dt * A[i]), dx * Bc[i]);
      continue;
    }
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
      hs[i] = fmaf(hs[i], __expf(dt * A[i]), dx * Bc[i]);
      acc = fmaf(hs[i], Cc[i], acc);
    }
    acc = fmaf(D, xv, acc);
    if (a.z != nullptr) acc *= silu_f(__bfloat162float(a.z[(long long)t * a.ldz + d]));
    a.y[(long long)t * a.ldy + d] = __float2bfloat16(acc);
  }
  if (MODE == kLocal) {
    store_f32<N>(sg + seg * seg_stride, hs);
    a.seg_dt[((long long)s * (a.segs - 1) + seg) * a.Dm + d] = dt_sum;
  } else if (MODE == kWhole || seg == seg_last) {
    store_f32<N>(st, hs);
  }
}

// start[seg + 1] = end_local[seg] + exp(A sum dt[seg]) * start[seg] per channel and state entry, in place over seg_state
template <int N>
__global__ void mamba1_combine_kernel(const Mamba1Args a) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
  const int t0 = a.q_starts[s];
  const int n = a.q_starts[s + 1] - t0;
  if (d >= a.Dm || n <= 0) return;
  const int seg_last = min(a.segs - 1, (n - 1) / a.seg_len);
  if (seg_last == 0) return;
  float carry[N], A[N];
  load_f32<N>(a.A + (long long)d * N, A);
  if (a.positions[t0] != 0) {
    load_f32<N>(a.state + ((long long)a.seq_state[s] * a.Dm + d) * N, carry);
    store_f32<N>(a.seg_start0 + ((long long)s * a.Dm + d) * N, carry);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) carry[i] = 0.f;
  }
  float* sg = a.seg_state + ((long long)s * (a.segs - 1) * a.Dm + d) * N;
  for (int seg = 0; seg < seg_last; ++seg) {
    const float sdt = a.seg_dt[((long long)s * (a.segs - 1) + seg) * a.Dm + d];
    float e[N];
    load_f32<N>(sg + (long long)seg * a.Dm * N, e);
#pragma unroll
    for (int i = 0; i < N; ++i) carry[i] = fmaf(carry[i], __expf(A[i] * sdt), e[i]);
    store_f32<N>(sg + (long long)seg * a.Dm * N, carry);
  }
}

// ------------------------------------------------------------------------------------------ matrix-state family
// State S[v][k] per head, one thread row per v with DK / NPT lanes along k. d = exp(w) is the decay.
//   kRwkv6      y = sum_k r (u k v + S);               S = S d + k v
//   kRwkv7      sa = sum_k S a;  S = S d + sa b + v k;   y = sum_k S r
//   kGatedDelta S = S d (one d per head);  m = sum_k S k;  S += k (v - m) beta;  y = sum_k S q
//   kKda        as kGatedDelta with one d per key channel
enum { kRwkv6 = 0, kRwkv7 = 1, kGatedDelta = 2, kKda = 3 };
struct MatrixStateArgs {
  const bf16 *r, *k, *v, *a, *b;     // r doubles as q; a, b only RWKV-7
  const float* w;                    // log decay: [T][H*DK] (per channel) or [T][H] (kGatedDelta)
  const float* u;                    // RWKV-6 bonus [H*DK]
  const bf16* beta;                  // [T][H] delta-rule step size (already through its sigmoid)
  long long ldr, ldk, ldv, lda, ldb, ldw, ldbeta, ldy;
  float* state;                      // [slots][H][DV][DK]
  const int *q_starts, *seq_state, *positions;
  bf16* y;
  int H, DV, kv_ratio;               // value heads per key head (q, k, w of head h come from head h / kv_ratio)
  int l2norm;                        // delta kinds: normalise q and k over DK inside the kernel
  float q_scale;
  // kGatedDelta with raw gates (w == nullptr): beta holds the logit of the step size, gate_raw [T][H] the logit a of the
  // decay; step size = sigmoid(beta), log decay = gate_A[h] * softplus(a + gate_dt_bias[h])
  const bf16* gate_raw;
  long long ldgate;
  const float *gate_A, *gate_dt_bias;
};

template <int KIND, int DK>
__global__ void __launch_bounds__(128) matrix_state_kernel(const MatrixStateArgs a) {
  constexpr int NPT = 16, TPK = DK / NPT, ROWS = 128 / TPK;
  const int vtiles = (a.DV + ROWS - 1) / ROWS;
  const int h = blockIdx.x / vtiles, v = (blockIdx.x % vtiles) * ROWS + threadIdx.x / TPK;
  const int lk = threadIdx.x % TPK, s = blockIdx.y;
  const int t0 = a.q_starts[s], n = a.q_starts[s + 1] - t0;
  if (n <= 0) return;
  const bool valid = v < a.DV;
  const int vc = valid ? v : a.DV - 1;
  const int hk = h / a.kv_ratio;
  float* st = a.state + (((long long)a.seq_state[s] * a.H + h) * a.DV + vc) * DK + lk * NPT;
  float S[NPT];
  if (a.positions[t0] == 0) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) S[i] = 0.f;
  } else {
    load_f32<NPT>(st, S);
  }
  float u[NPT];
  if (KIND == kRwkv6) load_f32<NPT>(a.u + (long long)hk * DK + lk * NPT, u);
  const long long ko = (long long)hk * DK + lk * NPT;
  for (int t = t0; t < t0 + n; ++t) {
    float r[NPT], k[NPT], d[NPT];
    load_bf16<NPT>(a.r + t * a.ldr + ko, r);
    load_bf16<NPT>(a.k + t * a.ldk + ko, k);
    const float vv = __bfloat162float(a.v[t * a.ldv + (long long)h * a.DV + vc]);
    if (KIND == kGatedDelta) {
      const float dh = a.w != nullptr
                           ? __expf(a.w[t * a.ldw + h])
                           : __expf(a.gate_A[h] * softplus_f(__bfloat162float(a.gate_raw[t * a.ldgate + h]) + a.gate_dt_bias[h]));
#pragma unroll
      for (int i = 0; i < NPT; ++i) d[i] = dh;
    } else {
      load_f32<NPT>(a.w + t * a.ldw + ko, d);
#pragma unroll
      for (int i = 0; i < NPT; ++i) d[i] = __expf(d[i]);
    }
    float out = 0.f;
    if (KIND == kRwkv6) {
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        const float kv = k[i] * vv;
        out = fmaf(r[i], fmaf(u[i], kv, S[i]), out);
        S[i] = fmaf(S[i], d[i], kv);
      }
      out = row_sum<TPK>(out);
    } else if (KIND == kRwkv7) {
      float av[NPT], bv[NPT], sa = 0.f;
      load_bf16<NPT>(a.a + t * a.lda + ko, av);
      load_bf16<NPT>(a.b + t * a.ldb + ko, bv);
#pragma unroll
      for (int i = 0; i < NPT; ++i) sa = fmaf(S[i], av[i], sa);
      sa = row_sum<TPK>(sa);
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        S[i] = fmaf(S[i], d[i], fmaf(sa, bv[i], vv * k[i]));
        out = fmaf(S[i], r[i], out);
      }
      out = row_sum<TPK>(out);
    } else {
      float qs = a.q_scale;
      if (a.l2norm) {
        float qq = 0.f, kk = 0.f;
#pragma unroll
        for (int i = 0; i < NPT; ++i) qq = fmaf(r[i], r[i], qq), kk = fmaf(k[i], k[i], kk);
        qq = row_sum<TPK>(qq), kk = row_sum<TPK>(kk);
        qs *= rsqrtf(qq + 1e-6f);
        const float ks = rsqrtf(kk + 1e-6f);
#pragma unroll
        for (int i = 0; i < NPT; ++i) k[i] *= ks;
      }
      float m = 0.f;
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        S[i] *= d[i];
        m = fmaf(S[i], k[i], m);
      }
      m = row_sum<TPK>(m);
      float step = __bfloat162float(a.beta[t * a.ldbeta + h]);
      if (KIND == kGatedDelta && a.w == nullptr) step = 1.f / (1.f + __expf(-step));
      const float delta = (vv - m) * step;
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        S[i] = fmaf(k[i], delta, S[i]);
        out = fmaf(S[i], r[i], out);
      }
      out = row_sum<TPK>(out) * qs;
    }
    if (lk == 0 && valid) a.y[t * a.ldy + (long long)h * a.DV + vc] = __float2bfloat16(out);
  }
  if (valid) store_f32<NPT>(st, S);
}

// ------------------------------------------------------------------------------------------ gated RMSNorm
// Per (token, group of `gs` channels): mode 0  y = rmsnorm(x * silu(z)) * w   (Mamba-2: gate first)
//                                      mode 1  y = rmsnorm(x) * w * silu(z)   (gated delta net: norm first)
// w has `wlen` entries (D for Mamba-2, the head width when every head shares one weight). One warp per group.
// y may be x (every element is read and then written by the same thread).
__global__ void __launch_bounds__(128) gated_rmsnorm_kernel(const bf16* x, long long ldx, const bf16* __restrict__ z, long long ldz,
                                                            const bf16* __restrict__ w, int wlen, bf16* y, long long ldy, int T, int D,
                                                            int gs, float eps, int mode) {
  const int groups = D / gs;
  const long long item = (long long)blockIdx.x * 4 + threadIdx.x / 32;
  if (item >= (long long)T * groups) return;
  const int t = (int)(item / groups), g = (int)(item % groups), lane = threadIdx.x % 32;
  const bf16* xr = x + t * ldx + (long long)g * gs;
  const bf16* zr = z != nullptr ? z + t * ldz + (long long)g * gs : nullptr;
  float ss = 0.f;
  for (int i = lane; i < gs; i += 32) {
    float v = __bfloat162float(xr[i]);
    if (mode == 0 && zr != nullptr) v *= silu_f(__bfloat162float(zr[i]));
    ss = fmaf(v, v, ss);
  }
  ss = row_sum<32>(ss);
  const float inv = rsqrtf(ss / gs + eps);
  bf16* yr = y + t * ldy + (long long)g * gs;
  for (int i = lane; i < gs; i += 32) {
    float v = __bfloat162float(xr[i]);
    const float gate = zr != nullptr ? silu_f(__bfloat162float(zr[i])) : 1.f;
    if (mode == 0) v *= gate;
    v = v * inv * __bfloat162float(w[(g * gs + i) % wlen]);
    if (mode == 1) v *= gate;
    yr[i] = __float2bfloat16(v);
  }
}

// The same for wide groups (Mamba-2 normalises the whole inner width at once): one CTA of 256 threads per (token, group),
// two channels per thread and step, the (gated) row kept in registers between the two passes when it fits (up to 8192 channels).
__global__ void __launch_bounds__(256) gated_rmsnorm_wide_kernel(const bf16* x, long long ldx, const bf16* __restrict__ z, long long ldz,
                                                                 const bf16* __restrict__ w, int wlen, bf16* y, long long ldy, int D, int gs,
                                                                 float eps, int mode) {
  constexpr int KEEP = 16;                                 // pairs kept per thread: 256 * 16 * 2 = 8192 channels
  const int groups = D / gs;
  const int t = blockIdx.x / groups, g = blockIdx.x % groups;
  const __nv_bfloat162* xr = reinterpret_cast<const __nv_bfloat162*>(x + t * ldx + (long long)g * gs);
  const __nv_bfloat162* zr = z != nullptr ? reinterpret_cast<const __nv_bfloat162*>(z + t * ldz + (long long)g * gs) : nullptr;
  const int pairs = gs / 2;
  float2 keep[KEEP];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int p = threadIdx.x + i * 256;
    keep[i] = make_float2(0.f, 0.f);
    if (p < pairs) {
      keep[i] = __bfloat1622float2(xr[p]);
      if (mode == 0 && zr != nullptr) {
        const float2 zz = __bfloat1622float2(zr[p]);
        keep[i].x *= silu_f(zz.x), keep[i].y *= silu_f(zz.y);
      }
      ss = fmaf(keep[i].x, keep[i].x, fmaf(keep[i].y, keep[i].y, ss));
    }
  }
  for (int p = threadIdx.x + KEEP * 256; p < pairs; p += 256) {     // beyond the kept part: read again in the second pass
    float2 v = __bfloat1622float2(xr[p]);
    if (mode == 0 && zr != nullptr) {
      const float2 zz = __bfloat1622float2(zr[p]);
      v.x *= silu_f(zz.x), v.y *= silu_f(zz.y);
    }
    ss = fmaf(v.x, v.x, fmaf(v.y, v.y, ss));
  }
  __shared__ float part[8];
  ss = row_sum<32>(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += part[i];
  const float inv = rsqrtf(tot / gs + eps);
  __nv_bfloat162* yr = reinterpret_cast<__nv_bfloat162*>(y + t * ldy + (long long)g * gs);
  auto weight = [&](int p) {
    const int c = (g * gs + 2 * p) % wlen;
    return make_float2(__bfloat162float(w[c]), __bfloat162float(w[(c + 1) % wlen]));
  };
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int p = threadIdx.x + i * 256;
    if (p < pairs) {
      const float2 ww = weight(p);
      float2 v = make_float2(keep[i].x * inv * ww.x, keep[i].y * inv * ww.y);
      if (mode == 1 && zr != nullptr) {
        const float2 zz = __bfloat1622float2(zr[p]);
        v.x *= silu_f(zz.x), v.y *= silu_f(zz.y);
      }
      yr[p] = __floats2bfloat162_rn(v.x, v.y);
    }
  }
  for (int p = threadIdx.x + KEEP * 256; p < pairs; p += 256) {
    float2 v = __bfloat1622float2(xr[p]);
    float2 gt = make_float2(1.f, 1.f);
    if (zr != nullptr) {
      const float2 zz = __bfloat1622float2(zr[p]);
      gt = make_float2(silu_f(zz.x), silu_f(zz.y));
    }
    if (mode == 0) v.x *= gt.x, v.y *= gt.y;
    const float2 ww = weight(p);
    v = make_float2(v.x * inv * ww.x, v.y * inv * ww.y);
    if (mode == 1) v.x *= gt.x, v.y *= gt.y;
    yr[p] = __floats2bfloat162_rn(v.x, v.y);
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
}  // namespace

// ---------------------------------------------------------------------------------------------- launchers
// Every launcher returns 0 on success or a negative code naming the argument it rejected, before any launch.
int causal_conv1d(const void* x, long long ldx, const float* w, const float* bias, void* state, const int* q_starts,
                  const int* seq_state, const int* positions, void* y, long long ldy, int B, int C, int W, int act,
                  int max_q_len, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (C % 2 || (ldx % 2) || (ldy % 2) || x == y) return -1;
  if (W < 2 || W > 4) return -2;
  constexpr int seg_tokens = 64;                       // 16 tokens per thread
  const int runs = std::min(std::max((max_q_len + seg_tokens - 1) / seg_tokens, 1), 65535);
  const dim3 grid((C / 2 + 63) / 64, B, runs), block(64, 4);
  auto xs = static_cast<const bf16*>(x);
  auto ys = static_cast<bf16*>(y);
  auto ss = static_cast<bf16*>(state);
  if (W == 2) conv1d_kernel<2><<<grid, block, 0, stream>>>(xs, ldx, w, bias, ss, q_starts, seq_state, positions, ys, ldy, C, act, seg_tokens);
  if (W == 3) conv1d_kernel<3><<<grid, block, 0, stream>>>(xs, ldx, w, bias, ss, q_starts, seq_state, positions, ys, ldy, C, act, seg_tokens);
  if (W == 4) conv1d_kernel<4><<<grid, block, 0, stream>>>(xs, ldx, w, bias, ss, q_starts, seq_state, positions, ys, ldy, C, act, seg_tokens);
  return 0;
}

// seg_len > 0 with segs > 1: the sequence-parallel form (seg_state: B * (segs - 1) * H * P * N floats, seg_dt: B * (segs - 1) * H
// floats); segs must cover the longest sequence of the step (segs * seg_len >= its tokens).
int mamba2_scan(const void* x, long long ldx, const void* dt, long long lddt, const void* Bm, long long ldb, const void* Cm,
                long long ldc, const float* A, const float* D, const float* dt_bias, float* state, const int* q_starts,
                const int* seq_state, const int* positions, void* y, long long ldy, int B, int H, int P, int G, int N,
                float dt_min, float dt_max, int seg_len, int segs, float* seg_state, float* seg_dt, int skip_from,
                cudaStream_t stream) {
  if (B <= 0) return 0;
  if (!aligned16(Bm) || !aligned16(Cm) || (ldb % 8) || (ldc % 8) || G <= 0 || H % G) return -1;
  const bool segmented = seg_len > 0 && segs > 1;
  if (segmented && (seg_state == nullptr || seg_dt == nullptr || !aligned16(seg_state))) return -3;
  Mamba2Args a{static_cast<const bf16*>(x), static_cast<const bf16*>(dt), static_cast<const bf16*>(Bm), static_cast<const bf16*>(Cm),
               ldx, lddt, ldb, ldc, ldy, A, D, dt_bias, state, q_starts, seq_state, positions, static_cast<bf16*>(y), H, P, G,
               dt_min, dt_max, skip_from, seg_len, segs, seg_state,
               segmented ? seg_state + (long long)B * (segs - 1) * H * P * N : nullptr, seg_dt};
#define FLLM_M2(N_, NPT_)                                                                                          \
  {                                                                                                                \
    constexpr int rows = 128 / (N_ / NPT_);                                                                        \
    const unsigned gx = H * ((P + rows - 1) / rows);                                                               \
    if (!segmented) {                                                                                              \
      mamba2_scan_kernel<N_, NPT_, kWhole><<<dim3(gx, B), 128, 0, stream>>>(a);                                    \
    } else {                                                                                                       \
      mamba2_scan_kernel<N_, NPT_, kLocal><<<dim3(gx, B, segs - 1), 128, 0, stream>>>(a);                          \
      const long long per_seq = (long long)H * P * N_;                                                             \
      mamba2_combine_kernel<<<dim3((unsigned)((per_seq / 4 + 255) / 256), B), 256, 0, stream>>>(a, N_);            \
      mamba2_scan_kernel<N_, NPT_, kFinal><<<dim3(gx, B, segs), 128, 0, stream>>>(a);                              \
    }                                                                                                              \
    return 0;                                                                                                      \
  }
  switch (N) {
    case 16: FLLM_M2(16, 16)
    case 32: FLLM_M2(32, 16)
    case 64: FLLM_M2(64, 16)
    case 128: FLLM_M2(128, 16)
    case 256: FLLM_M2(256, 16)
  }
#undef FLLM_M2
  return -2;
}

int mamba1_scan(const void* x, long long ldx, const void* dt, long long lddt, const void* Bm, long long ldb, const void* Cm,
                long long ldc, const void* z, long long ldz, const float* A, const float* D, const float* dt_bias, float* state,
                const int* q_starts, const int* seq_state, const int* positions, void* y, long long ldy, int B, int Dm, int N,
                int seg_len, int segs, float* seg_state, float* seg_dt, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (!aligned16(Bm) || !aligned16(Cm) || (ldb % 8) || (ldc % 8)) return -1;
  const bool segmented = seg_len > 0 && segs > 1;
  if (segmented && (seg_state == nullptr || seg_dt == nullptr || !aligned16(seg_state))) return -3;
  Mamba1Args a{static_cast<const bf16*>(x), static_cast<const bf16*>(dt), static_cast<const bf16*>(Bm), static_cast<const bf16*>(Cm),
               static_cast<const bf16*>(z), ldx, lddt, ldb, ldc, ldz, ldy, A, D, dt_bias, state, q_starts, seq_state, positions,
               static_cast<bf16*>(y), Dm, seg_len, segs, seg_state,
               segmented ? seg_state + (long long)B * (segs - 1) * Dm * N : nullptr, seg_dt};
  const unsigned gx = (Dm + 127) / 128;
#define FLLM_M1(N_)                                                                           \
  {                                                                                           \
    if (!segmented) {                                                                         \
      mamba1_scan_kernel<N_, kWhole><<<dim3(gx, B), 128, 0, stream>>>(a);                     \
    } else {                                                                                  \
      mamba1_scan_kernel<N_, kLocal><<<dim3(gx, B, segs - 1), 128, 0, stream>>>(a);           \
      mamba1_combine_kernel<N_><<<dim3(gx, B), 128, 0, stream>>>(a);                          \
      mamba1_scan_kernel<N_, kFinal><<<dim3(gx, B, segs), 128, 0, stream>>>(a);               \
    }                                                                                         \
    return 0;                                                                                 \
  }
  if (N == 16) FLLM_M1(16)
  if (N == 8) FLLM_M1(8)
#undef FLLM_M1
  return -2;
}

int matrix_state_scan(int kind, const void* r, long long ldr, const void* k, long long ldk, const void* v, long long ldv,
                      const void* a_, long long lda, const void* b_, long long ldb, const float* w, long long ldw, const float* u,
                      const void* beta, long long ldbeta, float* state, const int* q_starts, const int* seq_state,
                      const int* positions, void* y, long long ldy, int B, int H, int DK, int DV, int kv_ratio, int l2norm,
                      float q_scale, const void* gate_raw, long long ldgate, const float* gate_A, const float* gate_dt_bias,
                      cudaStream_t stream) {
  if (B <= 0) return 0;
  if (!aligned16(r) || !aligned16(k) || (ldr % 8) || (ldk % 8) || kv_ratio <= 0 || H % kv_ratio) return -1;
  if (w == nullptr && (kind != kGatedDelta || gate_raw == nullptr || gate_A == nullptr || gate_dt_bias == nullptr)) return -4;
  if (kind != kGatedDelta && (!aligned16(w) || (ldw % 4))) return -1;
  if (kind == kRwkv7 && (!aligned16(a_) || !aligned16(b_) || (lda % 8) || (ldb % 8))) return -1;
  if (kind == kRwkv6 && !aligned16(u)) return -1;
  MatrixStateArgs m{static_cast<const bf16*>(r), static_cast<const bf16*>(k), static_cast<const bf16*>(v), static_cast<const bf16*>(a_),
                    static_cast<const bf16*>(b_), w, u, static_cast<const bf16*>(beta), ldr, ldk, ldv, lda, ldb, ldw, ldbeta, ldy, state,
                    q_starts, seq_state, positions, static_cast<bf16*>(y), H, DV, kv_ratio, l2norm, q_scale,
                    static_cast<const bf16*>(gate_raw), ldgate, gate_A, gate_dt_bias};
#define FLLM_MS(KIND_, DK_)                                                                        \
  {                                                                                                \
    constexpr int rows = 128 / (DK_ / 16);                                                         \
    matrix_state_kernel<KIND_, DK_><<<dim3(H * ((DV + rows - 1) / rows), B), 128, 0, stream>>>(m); \
    return 0;                                                                                      \
  }
#define FLLM_MS_DK(KIND_)           \
  switch (DK) {                     \
    case 32: FLLM_MS(KIND_, 32)     \
    case 64: FLLM_MS(KIND_, 64)     \
    case 128: FLLM_MS(KIND_, 128)   \
    case 256: FLLM_MS(KIND_, 256)   \
    default: return -2;             \
  }
  switch (kind) {
    case kRwkv6: FLLM_MS_DK(kRwkv6)
    case kRwkv7: FLLM_MS_DK(kRwkv7)
    case kGatedDelta: FLLM_MS_DK(kGatedDelta)
    case kKda: FLLM_MS_DK(kKda)
  }
#undef FLLM_MS_DK
#undef FLLM_MS
  return -3;
}

void gated_rmsnorm(const void* x, long long ldx, const void* z, long long ldz, const void* w, int wlen, void* y, long long ldy, int T,
                   int D, int group_size, float eps, int norm_before_gate, cudaStream_t stream) {
  if (T <= 0) return;
  const long long items = (long long)T * (D / group_size);
  const bool pairs_ok = group_size % 2 == 0 && ldx % 2 == 0 && ldy % 2 == 0 && (z == nullptr || ldz % 2 == 0) &&
                        (reinterpret_cast<uintptr_t>(x) & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 3) == 0 &&
                        (reinterpret_cast<uintptr_t>(z) & 3) == 0;
  if (group_size >= 1024 && pairs_ok) {
    gated_rmsnorm_wide_kernel<<<(unsigned)items, 256, 0, stream>>>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(z), ldz,
                                                                   static_cast<const bf16*>(w), wlen, static_cast<bf16*>(y), ldy, D,
                                                                   group_size, eps, norm_before_gate);
    return;
  }
  gated_rmsnorm_kernel<<<(unsigned)((items + 3) / 4), 128, 0, stream>>>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(z), ldz,
                                                                       static_cast<const bf16*>(w), wlen, static_cast<bf16*>(y), ldy, T, D,
                                                                       group_size, eps, norm_before_gate);
}

}  // namespace fllm
