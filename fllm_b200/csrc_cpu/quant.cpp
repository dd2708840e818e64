// Host codecs of the packed weight formats: scalar, branch-light loops that the
// compiler vectorises, OpenMP over rows. The K-quant search is the weighted
// least-squares scale/min fit used by the GGML reference quantizer, restated here.
#include "quant.h"

#include <math.h>
#include <string.h>

#include <algorithm>

// ---------------------------------------------------------------------------- scalar formats
float fllm_fp16_to_fp32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

uint16_t fllm_fp32_to_fp16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000;
  const int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
  uint32_t man = x & 0x7fffff;
  if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00 | (man ? 0x200 : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000;
    const int shift = 14 - exp;
    uint32_t h = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) ++h;
    return (uint16_t)(sign | h);
  }
  uint32_t h = ((uint32_t)exp << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fff;
  if (rem > 0x1000 || (rem == 0x1000 && (h & 1))) ++h;
  return (uint16_t)(sign | h);
}

float fllm_bf16_to_fp32(uint16_t h) {
  const uint32_t b = (uint32_t)h << 16;
  float f;
  memcpy(&f, &b, 4);
  return f;
}

uint16_t fllm_fp32_to_bf16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  if ((x & 0x7fffffff) > 0x7f800000) return (uint16_t)((x >> 16) | 0x40);
  x += 0x7fff + ((x >> 16) & 1);
  return (uint16_t)(x >> 16);
}

float fllm_e4m3_to_fp32(uint8_t v) {
  const int s = v >> 7, e = (v >> 3) & 0xf, m = v & 7;
  float r;
  if (e == 0) r = ldexpf((float)m, -9);
  else if (e == 15 && m == 7) r = NAN;
  else r = ldexpf(1.f + m / 8.f, e - 7);
  return s ? -r : r;
}

uint8_t fllm_fp32_to_e4m3(float f) {
  if (isnan(f)) return 0x7f;
  const uint8_t s = signbit(f) ? 0x80 : 0;
  float a = fabsf(f);
  if (a >= 448.f) return s | 0x7e;
  if (a < ldexpf(1.f, -10)) return s;      // below half of the smallest subnormal
  int e;
  frexpf(a, &e);                           // a = m * 2^e, m in [0.5, 1)
  int E = e - 1 + 7;
  if (E <= 0) {
    const int q = (int)nearbyintf(ldexpf(a, 9));
    return s | (uint8_t)(q >= 8 ? 0x08 : q);
  }
  int q = (int)nearbyintf(ldexpf(a, 3 - (e - 1))) - 8;
  if (q == 8) { q = 0; ++E; }
  if (E > 15 || (E == 15 && q == 7)) return s | 0x7e;
  return s | (uint8_t)(E << 3) | (uint8_t)q;
}

static const float kE2M1[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};

float fllm_e2m1_to_fp32(uint8_t v) {
  const float r = kE2M1[v & 7];
  return (v & 8) ? -r : r;
}

uint8_t fllm_fp32_to_e2m1(float f) {
  const uint8_t s = signbit(f) ? 8 : 0;
  const float a = fabsf(f);
  // round to nearest, ties to even mantissa
  uint8_t q;
  if (a <= 0.25f) q = 0;
  else if (a < 0.75f) q = 1;
  else if (a <= 1.25f) q = 2;
  else if (a < 1.75f) q = 3;
  else if (a <= 2.5f) q = 4;
  else if (a < 3.5f) q = 5;
  else if (a <= 5.f) q = 6;
  else q = 7;
  return s | q;
}

// ---------------------------------------------------------------------------- tables
int fllm_block_size(int type) {
  switch (type) {
    case FLLM_F32: case FLLM_F16: case FLLM_BF16: case FLLM_FP8_E4M3: return 1;
    case FLLM_Q4_0: case FLLM_Q4_1: case FLLM_Q5_0: case FLLM_Q5_1: case FLLM_Q8_0: case FLLM_IQ4_NL: case FLLM_MXFP4: return 32;
    case FLLM_NVFP4: return 16;
    case FLLM_Q2_K: case FLLM_Q3_K: case FLLM_Q4_K: case FLLM_Q5_K: case FLLM_Q6_K: case FLLM_Q8_K: case FLLM_IQ4_XS: return 256;
    default: return 0;
  }
}

int fllm_block_bytes(int type) {
  switch (type) {
    case FLLM_F32: return 4;
    case FLLM_F16: case FLLM_BF16: return 2;
    case FLLM_FP8_E4M3: return 1;
    case FLLM_Q4_0: return 18;
    case FLLM_Q4_1: return 20;
    case FLLM_Q5_0: return 22;
    case FLLM_Q5_1: return 24;
    case FLLM_Q2_K: return 84;
    case FLLM_Q3_K: return 110;
    case FLLM_IQ4_NL: return 18;
    case FLLM_IQ4_XS: return 136;
    case FLLM_Q8_0: return 34;
    case FLLM_MXFP4: return 17;
    case FLLM_NVFP4: return 9;
    case FLLM_Q4_K: return 144;
    case FLLM_Q5_K: return 176;
    case FLLM_Q6_K: return 210;
    case FLLM_Q8_K: return (int)sizeof(BlockQ8K);
    default: return 0;
  }
}

int64_t fllm_row_bytes(int type, int64_t ncols) {
  const int bs = fllm_block_size(type);
  if (!bs || ncols % bs) return -1;
  return ncols / bs * fllm_block_bytes(type);
}

// ---------------------------------------------------------------------------- K-quant helpers
static inline int nearest_int(float f) { return (int)nearbyintf(f); }

// Weighted fit of x ~ scale * L + min with L in [0, nmax]; returns scale, *the_min = -min.
static float fit_scale_min(int n, int nmax, const float* x, const float* w, uint8_t* L, float* the_min,
                           uint8_t* Laux, float rmin, float rdelta, int nstep) {
  float mn = x[0], mx = x[0], sum_w = w[0], sum_x = w[0] * x[0];
  for (int i = 1; i < n; ++i) {
    mn = std::min(mn, x[i]);
    mx = std::max(mx, x[i]);
    sum_w += w[i];
    sum_x += w[i] * x[i];
  }
  if (mn > 0) mn = 0;
  if (mx == mn) {
    for (int i = 0; i < n; ++i) L[i] = 0;
    *the_min = -mn;
    return 0.f;
  }
  float iscale = nmax / (mx - mn), scale = 1 / iscale, best = 0;
  for (int i = 0; i < n; ++i) {
    const int l = std::max(0, std::min(nmax, nearest_int(iscale * (x[i] - mn))));
    L[i] = (uint8_t)l;
    const float d = scale * l + mn - x[i];
    best += w[i] * d * d;
  }
  for (int is = 0; is <= nstep; ++is) {
    iscale = (rmin + rdelta * is + nmax) / (mx - mn);
    float sl = 0, sl2 = 0, sxl = 0;
    for (int i = 0; i < n; ++i) {
      const int l = std::max(0, std::min(nmax, nearest_int(iscale * (x[i] - mn))));
      Laux[i] = (uint8_t)l;
      sl += w[i] * l;
      sl2 += w[i] * l * l;
      sxl += w[i] * l * x[i];
    }
    const float D = sum_w * sl2 - sl * sl;
    if (D > 0) {
      float ts = (sum_w * sxl - sum_x * sl) / D, tm = (sl2 * sum_x - sl * sxl) / D;
      if (tm > 0) { tm = 0; ts = sxl / sl2; }
      float mad = 0;
      for (int i = 0; i < n; ++i) {
        const float d = ts * Laux[i] + tm - x[i];
        mad += w[i] * d * d;
      }
      if (mad < best) {
        memcpy(L, Laux, n);
        best = mad;
        scale = ts;
        mn = tm;
      }
    }
  }
  *the_min = -mn;
  return scale;
}

static inline void get_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) {
    *d = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

static void pack_scales_k4(const uint8_t* ls, const uint8_t* lm, uint8_t* out) {
  memset(out, 0, 12);
  for (int j = 0; j < 8; ++j) {
    if (j < 4) {
      out[j] = ls[j];
      out[j + 4] = lm[j];
    } else {
      out[j + 4] = (ls[j] & 0xF) | ((lm[j] & 0xF) << 4);
      out[j - 4] |= (ls[j] >> 4) << 6;
      out[j] |= (lm[j] >> 4) << 6;
    }
  }
}

static void quantize_block_q4k(const float* x, BlockQ4K* y) {
  uint8_t L[QK_K], Laux[32], ls[8], lm[8];
  float w[32], mins[8], scales[8];
  float max_scale = 0, max_min = 0;
  for (int j = 0; j < 8; ++j) {
    float s2 = 0;
    for (int l = 0; l < 32; ++l) s2 += x[32 * j + l] * x[32 * j + l];
    const float av = sqrtf(s2 / 32);
    for (int l = 0; l < 32; ++l) w[l] = av + fabsf(x[32 * j + l]);
    scales[j] = fit_scale_min(32, 15, x + 32 * j, w, L + 32 * j, &mins[j], Laux, -1.f, 0.1f, 20);
    max_scale = std::max(max_scale, scales[j]);
    max_min = std::max(max_min, mins[j]);
  }
  const float inv_s = max_scale > 0 ? 63.f / max_scale : 0.f, inv_m = max_min > 0 ? 63.f / max_min : 0.f;
  for (int j = 0; j < 8; ++j) {
    ls[j] = (uint8_t)std::min(63, nearest_int(inv_s * scales[j]));
    lm[j] = (uint8_t)std::min(63, nearest_int(inv_m * mins[j]));
  }
  pack_scales_k4(ls, lm, y->scales);
  y->d = fllm_fp32_to_fp16(max_scale / 63.f);
  y->dmin = fllm_fp32_to_fp16(max_min / 63.f);
  const float d = fllm_fp16_to_fp32(y->d), dmin = fllm_fp16_to_fp32(y->dmin);
  for (int j = 0; j < 8; ++j) {
    uint8_t sc, m;
    get_scale_min_k4(j, y->scales, &sc, &m);
    const float dd = d * sc;
    if (dd == 0) continue;
    const float dm = dmin * m;
    for (int i = 0; i < 32; ++i)
      L[32 * j + i] = (uint8_t)std::max(0, std::min(15, nearest_int((x[32 * j + i] + dm) / dd)));
  }
  for (int j = 0; j < 4; ++j)
    for (int l = 0; l < 32; ++l) y->qs[32 * j + l] = L[64 * j + l] | (L[64 * j + 32 + l] << 4);
}

static void dequantize_block_q4k(const BlockQ4K* b, float* y) {
  const float d = fllm_fp16_to_fp32(b->d), dmin = fllm_fp16_to_fp32(b->dmin);
  for (int j = 0; j < 4; ++j) {
    uint8_t s0, m0, s1, m1;
    get_scale_min_k4(2 * j, b->scales, &s0, &m0);
    get_scale_min_k4(2 * j + 1, b->scales, &s1, &m1);
    for (int l = 0; l < 32; ++l) {
      y[64 * j + l] = d * s0 * (b->qs[32 * j + l] & 0xF) - dmin * m0;
      y[64 * j + 32 + l] = d * s1 * (b->qs[32 * j + l] >> 4) - dmin * m1;
    }
  }
}

static void quantize_block_q5k(const float* x, BlockQ5K* y) {
  uint8_t L[QK_K], Laux[32], ls[8], lm[8];
  float w[32], mins[8], scales[8];
  float max_scale = 0, max_min = 0;
  for (int j = 0; j < 8; ++j) {
    float s2 = 0;
    for (int l = 0; l < 32; ++l) s2 += x[32 * j + l] * x[32 * j + l];
    const float av = sqrtf(s2 / 32);
    for (int l = 0; l < 32; ++l) w[l] = av + fabsf(x[32 * j + l]);
    scales[j] = fit_scale_min(32, 31, x + 32 * j, w, L + 32 * j, &mins[j], Laux, -0.5f, 0.1f, 15);
    max_scale = std::max(max_scale, scales[j]);
    max_min = std::max(max_min, mins[j]);
  }
  const float inv_s = max_scale > 0 ? 63.f / max_scale : 0.f, inv_m = max_min > 0 ? 63.f / max_min : 0.f;
  for (int j = 0; j < 8; ++j) {
    ls[j] = (uint8_t)std::min(63, nearest_int(inv_s * scales[j]));
    lm[j] = (uint8_t)std::min(63, nearest_int(inv_m * mins[j]));
  }
  pack_scales_k4(ls, lm, y->scales);
  y->d = fllm_fp32_to_fp16(max_scale / 63.f);
  y->dmin = fllm_fp32_to_fp16(max_min / 63.f);
  const float d = fllm_fp16_to_fp32(y->d), dmin = fllm_fp16_to_fp32(y->dmin);
  for (int j = 0; j < 8; ++j) {
    uint8_t sc, m;
    get_scale_min_k4(j, y->scales, &sc, &m);
    const float dd = d * sc;
    if (dd == 0) continue;
    const float dm = dmin * m;
    for (int i = 0; i < 32; ++i)
      L[32 * j + i] = (uint8_t)std::max(0, std::min(31, nearest_int((x[32 * j + i] + dm) / dd)));
  }
  memset(y->qh, 0, 32);
  uint8_t m1 = 1, m2 = 2;
  for (int n = 0; n < 4; ++n) {
    for (int j = 0; j < 32; ++j) {
      int l1 = L[64 * n + j], l2 = L[64 * n + 32 + j];
      if (l1 > 15) { l1 -= 16; y->qh[j] |= m1; }
      if (l2 > 15) { l2 -= 16; y->qh[j] |= m2; }
      y->qs[32 * n + j] = (uint8_t)(l1 | (l2 << 4));
    }
    m1 <<= 2;
    m2 <<= 2;
  }
}

static void dequantize_block_q5k(const BlockQ5K* b, float* y) {
  const float d = fllm_fp16_to_fp32(b->d), dmin = fllm_fp16_to_fp32(b->dmin);
  uint8_t u1 = 1, u2 = 2;
  for (int j = 0; j < 4; ++j) {
    uint8_t s0, m0, s1, m1;
    get_scale_min_k4(2 * j, b->scales, &s0, &m0);
    get_scale_min_k4(2 * j + 1, b->scales, &s1, &m1);
    for (int l = 0; l < 32; ++l) {
      y[64 * j + l] = d * s0 * ((b->qs[32 * j + l] & 0xF) + ((b->qh[l] & u1) ? 16 : 0)) - dmin * m0;
      y[64 * j + 32 + l] = d * s1 * ((b->qs[32 * j + l] >> 4) + ((b->qh[l] & u2) ? 16 : 0)) - dmin * m1;
    }
    u1 <<= 2;
    u2 <<= 2;
  }
}

// symmetric fit x ~ scale * q, q in [-nmax, nmax-1]; returns scale
static float fit_scale_sym(int n, int nmax, const float* x, int8_t* L) {
  float amax = 0, maxv = 0;
  for (int i = 0; i < n; ++i)
    if (fabsf(x[i]) > amax) { amax = fabsf(x[i]); maxv = x[i]; }
  if (amax < 1e-30f) {
    for (int i = 0; i < n; ++i) L[i] = 0;
    return 0.f;
  }
  float best_scale = 0, best_err = INFINITY;
  for (int is = -9; is <= 9; ++is) {
    const float iscale = -(nmax + 0.1f * is) / maxv;
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
      const int l = std::max(-nmax, std::min(nmax - 1, nearest_int(iscale * x[i])));
      const float wgt = x[i] * x[i];
      sumlx += wgt * x[i] * l;
      suml2 += wgt * l * l;
    }
    if (suml2 <= 0) continue;
    const float sc = sumlx / suml2;
    float err = 0;
    for (int i = 0; i < n; ++i) {
      const int l = std::max(-nmax, std::min(nmax - 1, nearest_int(iscale * x[i])));
      const float d = sc * l - x[i];
      err += x[i] * x[i] * d * d;
    }
    if (err < best_err) { best_err = err; best_scale = sc; }
  }
  const float inv = best_scale != 0 ? 1.f / best_scale : 0.f;
  for (int i = 0; i < n; ++i) L[i] = (int8_t)std::max(-nmax, std::min(nmax - 1, nearest_int(inv * x[i])));
  return best_scale;
}

static void quantize_block_q6k(const float* x, BlockQ6K* y) {
  int8_t L[QK_K];
  float scales[16];
  float max_scale = 0, max_abs = 0;
  for (int ib = 0; ib < 16; ++ib) {
    scales[ib] = fit_scale_sym(16, 32, x + 16 * ib, L + 16 * ib);
    if (fabsf(scales[ib]) > max_abs) { max_abs = fabsf(scales[ib]); max_scale = scales[ib]; }
  }
  if (max_abs < 1e-30f) {
    memset(y, 0, sizeof(*y));
    return;
  }
  const float iscale = -128.f / max_scale;
  y->d = fllm_fp32_to_fp16(1 / iscale);
  for (int ib = 0; ib < 16; ++ib) y->scales[ib] = (int8_t)std::min(127, nearest_int(iscale * scales[ib]));
  const float dd = fllm_fp16_to_fp32(y->d);
  uint8_t Lu[QK_K];
  for (int j = 0; j < 16; ++j) {
    const float d = dd * y->scales[j];
    for (int i = 0; i < 16; ++i) {
      int l = d != 0 ? nearest_int(x[16 * j + i] / d) : 0;
      l = std::max(-32, std::min(31, l));
      Lu[16 * j + i] = (uint8_t)(l + 32);
    }
  }
  for (int n = 0; n < 2; ++n) {
    const uint8_t* Ln = Lu + 128 * n;
    for (int l = 0; l < 32; ++l) {
      const uint8_t q1 = Ln[l] & 0xF, q2 = Ln[l + 32] & 0xF, q3 = Ln[l + 64] & 0xF, q4 = Ln[l + 96] & 0xF;
      y->ql[64 * n + l] = q1 | (q3 << 4);
      y->ql[64 * n + l + 32] = q2 | (q4 << 4);
      y->qh[32 * n + l] = (Ln[l] >> 4) | ((Ln[l + 32] >> 4) << 2) | ((Ln[l + 64] >> 4) << 4) | ((Ln[l + 96] >> 4) << 6);
    }
  }
}

static void dequantize_block_q6k(const BlockQ6K* b, float* y) {
  const float d = fllm_fp16_to_fp32(b->d);
  for (int n = 0; n < 2; ++n) {
    const uint8_t* ql = b->ql + 64 * n;
    const uint8_t* qh = b->qh + 32 * n;
    const int8_t* sc = b->scales + 8 * n;
    float* yo = y + 128 * n;
    for (int l = 0; l < 32; ++l) {
      const int is = l / 16;
      const int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
      const int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
      const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      yo[l] = d * sc[is] * q1;
      yo[l + 32] = d * sc[is + 2] * q2;
      yo[l + 64] = d * sc[is + 4] * q3;
      yo[l + 96] = d * sc[is + 6] * q4;
    }
  }
}

void quantize_row_q8_K(const float* x, BlockQ8K* y, int64_t n) {
  for (int64_t b = 0; b < n / QK_K; ++b) {
    const float* xb = x + b * QK_K;
    float amax = 0;
    for (int i = 0; i < QK_K; ++i) amax = std::max(amax, fabsf(xb[i]));
    if (amax == 0) {
      memset(&y[b], 0, sizeof(BlockQ8K));
      continue;
    }
    const float inv = 127.f / amax;
    for (int i = 0; i < QK_K; ++i) y[b].qs[i] = (int8_t)std::max(-127, std::min(127, nearest_int(inv * xb[i])));
    for (int j = 0; j < 16; ++j) {
      int s = 0;
      for (int i = 0; i < 16; ++i) s += y[b].qs[16 * j + i];
      y[b].bsums[j] = (int16_t)s;
    }
    y[b].d = amax / 127.f;
  }
}

// integer dot of a Q4_K weight row with a Q8_K activation row
float dot_q4_K_q8_K(const BlockQ4K* w, const BlockQ8K* a, int64_t nblocks) {
  float acc = 0;
  for (int64_t b = 0; b < nblocks; ++b) {
    const float d = fllm_fp16_to_fp32(w[b].d) * a[b].d, dmin = fllm_fp16_to_fp32(w[b].dmin) * a[b].d;
    int32_t sum_q = 0, sum_m = 0;
    for (int j = 0; j < 4; ++j) {
      uint8_t s0, m0, s1, m1;
      get_scale_min_k4(2 * j, w[b].scales, &s0, &m0);
      get_scale_min_k4(2 * j + 1, w[b].scales, &s1, &m1);
      const uint8_t* q = w[b].qs + 32 * j;
      const int8_t* x0 = a[b].qs + 64 * j;
      const int8_t* x1 = x0 + 32;
      int32_t p0 = 0, p1 = 0;
      for (int l = 0; l < 32; ++l) {
        p0 += (int32_t)(q[l] & 0xF) * x0[l];
        p1 += (int32_t)(q[l] >> 4) * x1[l];
      }
      sum_q += s0 * p0 + s1 * p1;
      sum_m += m0 * (a[b].bsums[4 * j] + a[b].bsums[4 * j + 1]) + m1 * (a[b].bsums[4 * j + 2] + a[b].bsums[4 * j + 3]);
    }
    acc += d * sum_q - dmin * sum_m;
  }
  return acc;
}

float dot_q6_K_q8_K(const BlockQ6K* w, const BlockQ8K* a, int64_t nblocks) {
  float acc = 0;
  for (int64_t b = 0; b < nblocks; ++b) {
    const float d = fllm_fp16_to_fp32(w[b].d) * a[b].d;
    int32_t sum = 0;
    for (int n = 0; n < 2; ++n) {
      const uint8_t* ql = w[b].ql + 64 * n;
      const uint8_t* qh = w[b].qh + 32 * n;
      const int8_t* sc = w[b].scales + 8 * n;
      const int8_t* x = a[b].qs + 128 * n;
      int32_t p[8] = {0};
      for (int l = 0; l < 32; ++l) {
        const int is = l / 16;
        p[is] += ((int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32) * x[l];
        p[is + 2] += ((int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32) * x[l + 32];
        p[is + 4] += ((int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32) * x[l + 64];
        p[is + 6] += ((int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32) * x[l + 96];
      }
      for (int k = 0; k < 8; ++k) sum += sc[k] * p[k];
    }
    acc += d * sum;
  }
  return acc;
}


// ---------------------------------------------------------------------------- further GGML block types
// The non-linear 4-bit code book of IQ4_NL / IQ4_XS (part of the file format).
static const int8_t kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

static inline int nearest_code_iq4(float v) {          // index of the closest code-book entry
  int best = 0;
  float bd = fabsf(v - kIq4nl[0]);
  for (int i = 1; i < 16; ++i) {
    const float d = fabsf(v - kIq4nl[i]);
    if (d < bd) { bd = d; best = i; }
  }
  return best;
}

// min / max affine fit of n values onto codes 0..nmax: x ~ d * q + m
static inline void affine_fit(const float* x, int n, int nmax, float* d, float* m) {
  float lo = x[0], hi = x[0];
  for (int i = 1; i < n; ++i) { lo = std::min(lo, x[i]); hi = std::max(hi, x[i]); }
  *m = lo;
  *d = (hi - lo) / (float)nmax;
}

static void dequantize_block_q2k(const BlockQ2K* b, float* y) {
  const float d = fllm_fp16_to_fp32(b->d), dmin = fllm_fp16_to_fp32(b->dmin);
  const uint8_t* q = b->qs;
  int is = 0;
  for (int n = 0; n < QK_K; n += 128) {
    for (int shift = 0; shift < 8; shift += 2) {
      for (int half = 0; half < 2; ++half) {
        const uint8_t sc = b->scales[is++];
        const float dl = d * (sc & 0xF), ml = dmin * (sc >> 4);
        for (int l = 0; l < 16; ++l) *y++ = dl * ((q[l + 16 * half] >> shift) & 3) - ml;
      }
    }
    q += 32;
  }
}

// 16 sub-blocks of 16 values: 2-bit codes with a 4-bit scale and a 4-bit minimum per sub-block
static void quantize_block_q2k(const float* x, BlockQ2K* b) {
  float sd[16], sm[16], maxd = 0.f, maxm = 0.f;
  for (int j = 0; j < 16; ++j) {
    float d, m;
    affine_fit(x + 16 * j, 16, 3, &d, &m);
    if (m > 0.f) { d = (m + 3.f * d) / 3.f; m = 0.f; }      // the format only stores minima <= 0 (as -min >= 0)
    sd[j] = d; sm[j] = -m;
    maxd = std::max(maxd, d); maxm = std::max(maxm, -m);
  }
  const float dd = maxd / 15.f, dm = maxm / 15.f;
  b->d = fllm_fp32_to_fp16(dd);
  b->dmin = fllm_fp32_to_fp16(dm);
  const float ddr = fllm_fp16_to_fp32(b->d), dmr = fllm_fp16_to_fp32(b->dmin);
  uint8_t L[QK_K];
  for (int j = 0; j < 16; ++j) {
    const int ls = ddr > 0 ? std::min(15, nearest_int(sd[j] / ddr)) : 0;
    const int lm = dmr > 0 ? std::min(15, nearest_int(sm[j] / dmr)) : 0;
    b->scales[j] = (uint8_t)(ls | (lm << 4));
    const float dl = ddr * ls, ml = dmr * lm;
    for (int i = 0; i < 16; ++i) {
      const int q = dl > 0 ? nearest_int((x[16 * j + i] + ml) / dl) : 0;
      L[16 * j + i] = (uint8_t)std::max(0, std::min(3, q));
    }
  }
  for (int n = 0; n < QK_K; n += 128)
    for (int l = 0; l < 32; ++l)
      b->qs[n / 4 + l] = L[n + l] | (L[n + l + 32] << 2) | (L[n + l + 64] << 4) | (L[n + l + 96] << 6);
}

// Q3_K: 3-bit codes (2 low bits in qs, the third bit in hmask, value = code - 4), sixteen 6-bit scales (offset 32)
static void unpack_scales_q3k(const uint8_t* s12, int8_t* sc16) {
  for (int j = 0; j < 16; ++j) {
    const int lo = j < 8 ? (s12[j] & 0xF) : (s12[j - 8] >> 4);
    const int hi = (s12[8 + (j & 3)] >> (2 * (j >> 2))) & 3;
    sc16[j] = (int8_t)((lo | (hi << 4)) - 32);
  }
}

static void dequantize_block_q3k(const BlockQ3K* b, float* y) {
  const float d_all = fllm_fp16_to_fp32(b->d);
  int8_t sc[16];
  unpack_scales_q3k(b->scales, sc);
  const uint8_t* q = b->qs;
  const uint8_t* hm = b->hmask;
  uint8_t m = 1;
  int is = 0;
  for (int n = 0; n < QK_K; n += 128) {
    for (int shift = 0; shift < 8; shift += 2) {
      for (int half = 0; half < 2; ++half) {
        const float dl = d_all * sc[is++];
        for (int l = 0; l < 16; ++l) {
          const int idx = l + 16 * half;
          *y++ = dl * ((int)((q[idx] >> shift) & 3) - ((hm[idx] & m) ? 0 : 4));
        }
      }
      m <<= 1;
    }
    q += 32;
  }
}

static void quantize_block_q3k(const float* x, BlockQ3K* b) {
  float sd[16], amax_s = 0.f;
  for (int j = 0; j < 16; ++j) {
    float amax = 0.f, mx = 0.f;
    for (int i = 0; i < 16; ++i)
      if (fabsf(x[16 * j + i]) > amax) { amax = fabsf(x[16 * j + i]); mx = x[16 * j + i]; }
    sd[j] = mx / -4.f;                                     // the extreme value maps to code -4
    amax_s = std::max(amax_s, fabsf(sd[j]));
  }
  const float dd = amax_s / 31.f;
  b->d = fllm_fp32_to_fp16(dd);
  const float ddr = fllm_fp16_to_fp32(b->d);
  int ls[16];
  memset(b->scales, 0, 12);
  memset(b->hmask, 0, 32);
  uint8_t L[QK_K];
  for (int j = 0; j < 16; ++j) {
    ls[j] = ddr > 0 ? std::max(-32, std::min(31, nearest_int(sd[j] / ddr))) : 0;
    const int u = ls[j] + 32;
    if (j < 8) b->scales[j] |= (u & 0xF); else b->scales[j - 8] |= ((u & 0xF) << 4);
    b->scales[8 + (j & 3)] |= ((u >> 4) << (2 * (j >> 2)));
    const float dl = ddr * ls[j];
    for (int i = 0; i < 16; ++i) {
      const int q = dl != 0.f ? nearest_int(x[16 * j + i] / dl) : 0;
      L[16 * j + i] = (uint8_t)(std::max(-4, std::min(3, q)) + 4);      // 0..7
    }
  }
  uint8_t m = 1;
  int pos = 0;
  for (int n = 0; n < QK_K; n += 128) {
    for (int k = 0; k < 4; ++k) {
      for (int l = 0; l < 32; ++l) {
        const int v = L[n + 32 * k + l];
        if (v > 3) b->hmask[l] |= m;
      }
      m <<= 1;
    }
    for (int l = 0; l < 32; ++l)
      b->qs[pos + l] = (L[n + l] & 3) | ((L[n + l + 32] & 3) << 2) | ((L[n + l + 64] & 3) << 4) | ((L[n + l + 96] & 3) << 6);
    pos += 32;
  }
}

static void dequantize_block_iq4xs(const BlockIQ4XS* b, float* y) {
  const float d = fllm_fp16_to_fp32(b->d);
  const uint8_t* qs = b->qs;
  for (int ib = 0; ib < QK_K / 32; ++ib) {
    const int ls = ((b->scales_l[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((b->scales_h >> (2 * ib)) & 3) << 4);
    const float dl = d * (ls - 32);
    for (int j = 0; j < 16; ++j) {
      y[j] = dl * kIq4nl[qs[j] & 0xF];
      y[j + 16] = dl * kIq4nl[qs[j] >> 4];
    }
    y += 32;
    qs += 16;
  }
}

static void quantize_block_iq4xs(const float* x, BlockIQ4XS* b) {
  float sd[8], amax_s = 0.f;
  for (int ib = 0; ib < 8; ++ib) {
    float amax = 0.f, mx = 0.f;
    for (int i = 0; i < 32; ++i)
      if (fabsf(x[32 * ib + i]) > amax) { amax = fabsf(x[32 * ib + i]); mx = x[32 * ib + i]; }
    sd[ib] = mx / -127.f;
    amax_s = std::max(amax_s, fabsf(sd[ib]));
  }
  const float dd = amax_s / 31.f;
  b->d = fllm_fp32_to_fp16(dd);
  const float ddr = fllm_fp16_to_fp32(b->d);
  b->scales_h = 0;
  memset(b->scales_l, 0, 4);
  for (int ib = 0; ib < 8; ++ib) {
    const int ls = ddr > 0 ? std::max(-32, std::min(31, nearest_int(sd[ib] / ddr))) : 0;
    const int u = ls + 32;
    b->scales_l[ib / 2] |= (uint8_t)((u & 0xF) << (4 * (ib % 2)));
    b->scales_h |= (uint16_t)((u >> 4) << (2 * ib));
    const float dl = ddr * ls, id = dl != 0.f ? 1.f / dl : 0.f;
    for (int j = 0; j < 16; ++j)
      b->qs[16 * ib + j] = (uint8_t)(nearest_code_iq4(x[32 * ib + j] * id) | (nearest_code_iq4(x[32 * ib + 16 + j] * id) << 4));
  }
}

// ---------------------------------------------------------------------------- row codecs
static void quantize_row(int type, const float* x, uint8_t* out, int64_t n) {
  switch (type) {
    case FLLM_F32: memcpy(out, x, n * 4); break;
    case FLLM_F16: for (int64_t i = 0; i < n; ++i) ((uint16_t*)out)[i] = fllm_fp32_to_fp16(x[i]); break;
    case FLLM_BF16: for (int64_t i = 0; i < n; ++i) ((uint16_t*)out)[i] = fllm_fp32_to_bf16(x[i]); break;
    case FLLM_FP8_E4M3: for (int64_t i = 0; i < n; ++i) out[i] = fllm_fp32_to_e4m3(x[i]); break;
    case FLLM_Q8_0: {
      auto* y = (BlockQ8_0*)out;
      for (int64_t b = 0; b < n / 32; ++b) {
        float amax = 0;
        for (int i = 0; i < 32; ++i) amax = std::max(amax, fabsf(x[32 * b + i]));
        const float d = amax / 127.f, id = d ? 1.f / d : 0.f;
        y[b].d = fllm_fp32_to_fp16(d);
        for (int i = 0; i < 32; ++i) y[b].qs[i] = (int8_t)nearest_int(x[32 * b + i] * id);
      }
    } break;
    case FLLM_Q4_0: {
      auto* y = (BlockQ4_0*)out;
      for (int64_t b = 0; b < n / 32; ++b) {
        float amax = 0, mx = 0;
        for (int i = 0; i < 32; ++i)
          if (fabsf(x[32 * b + i]) > amax) { amax = fabsf(x[32 * b + i]); mx = x[32 * b + i]; }
        const float d = mx / -8.f, id = d ? 1.f / d : 0.f;
        y[b].d = fllm_fp32_to_fp16(d);
        for (int i = 0; i < 16; ++i) {
          const int a = std::min(15, (int)(x[32 * b + i] * id + 8.5f));
          const int c = std::min(15, (int)(x[32 * b + 16 + i] * id + 8.5f));
          y[b].qs[i] = (uint8_t)(a | (c << 4));
        }
      }
    } break;
    case FLLM_MXFP4: {
      auto* y = (BlockMXFP4*)out;
      for (int64_t b = 0; b < n / 32; ++b) {
        float amax = 0;
        for (int i = 0; i < 32; ++i) amax = std::max(amax, fabsf(x[32 * b + i]));
        // shared power-of-two scale: largest magnitude maps into e2m1's range (max 6 = 1.5 * 2^2)
        int e = amax > 0 ? (int)floorf(log2f(amax)) - 2 : -127;
        e = std::max(-127, std::min(127, e));
        y[b].e = (uint8_t)(e + 127);
        const float inv = ldexpf(1.f, -e);
        for (int i = 0; i < 16; ++i) {
          const uint8_t lo = fllm_fp32_to_e2m1(x[32 * b + i] * inv), hi = fllm_fp32_to_e2m1(x[32 * b + 16 + i] * inv);
          y[b].qs[i] = lo | (hi << 4);
        }
      }
    } break;
    case FLLM_NVFP4: {
      auto* y = (BlockNVFP4*)out;
      for (int64_t b = 0; b < n / 16; ++b) {
        float amax = 0;
        for (int i = 0; i < 16; ++i) amax = std::max(amax, fabsf(x[16 * b + i]));
        const uint8_t s8 = fllm_fp32_to_e4m3(amax / 6.f);
        const float s = fllm_e4m3_to_fp32(s8), inv = s > 0 ? 1.f / s : 0.f;
        y[b].scale = s8;
        for (int i = 0; i < 8; ++i) {
          const uint8_t lo = fllm_fp32_to_e2m1(x[16 * b + 2 * i] * inv), hi = fllm_fp32_to_e2m1(x[16 * b + 2 * i + 1] * inv);
          y[b].qs[i] = lo | (hi << 4);
        }
      }
    } break;
    case FLLM_Q4_1: {
      auto* y = (BlockQ4_1*)out;
      for (int64_t b = 0; b < n / 32; ++b) {
        float d, m;
        affine_fit(x + 32 * b, 32, 15, &d, &m);
        y[b].d = fllm_fp32_to_fp16(d);
        y[b].m = fllm_fp32_to_fp16(m);
        const float id = d ? 1.f / d : 0.f;
        for (int i = 0; i < 16; ++i) {
          const int a = std::max(0, std::min(15, nearest_int((x[32 * b + i] - m) * id)));
          const int c = std::max(0, std::min(15, nearest_int((x[32 * b + 16 + i] - m) * id)));
          y[b].qs[i] = (uint8_t)(a | (c << 4));
        }
      }
    } break;
    case FLLM_Q5_0: {
      auto* y = (BlockQ5_0*)out;
      for (int64_t b = 0; b < n / 32; ++b) {
        float amax = 0, mx = 0;
        for (int i = 0; i < 32; ++i)
          if (fabsf(x[32 * b + i]) > amax) { amax = fabsf(x[32 * b + i]); mx = x[32 * b + i]; }
        const float d = mx / -16.f, id = d ? 1.f / d : 0.f;
        y[b].d = fllm_fp32_to_fp16(d);
        uint32_t qh = 0;
        for (int i = 0; i < 16; ++i) {
          const int a = std::min(31, (int)(x[32 * b + i] * id + 16.5f));
          const int c = std::min(31, (int)(x[32 * b + 16 + i] * id + 16.5f));
          y[b].qs[i] = (uint8_t)((a & 0xF) | ((c & 0xF) << 4));
          qh |= (uint32_t)((a & 0x10) >> 4) << i;
          qh |= (uint32_t)((c & 0x10) >> 4) << (i + 16);
        }
        memcpy(y[b].qh, &qh, 4);
      }
    } break;
    case FLLM_Q5_1: {
      auto* y = (BlockQ5_1*)out;
      for (int64_t b = 0; b < n / 32; ++b) {
        float d, m;
        affine_fit(x + 32 * b, 32, 31, &d, &m);
        y[b].d = fllm_fp32_to_fp16(d);
        y[b].m = fllm_fp32_to_fp16(m);
        const float id = d ? 1.f / d : 0.f;
        uint32_t qh = 0;
        for (int i = 0; i < 16; ++i) {
          const int a = std::max(0, std::min(31, nearest_int((x[32 * b + i] - m) * id)));
          const int c = std::max(0, std::min(31, nearest_int((x[32 * b + 16 + i] - m) * id)));
          y[b].qs[i] = (uint8_t)((a & 0xF) | ((c & 0xF) << 4));
          qh |= (uint32_t)((a & 0x10) >> 4) << i;
          qh |= (uint32_t)((c & 0x10) >> 4) << (i + 16);
        }
        memcpy(y[b].qh, &qh, 4);
      }
    } break;
    case FLLM_IQ4_NL: {
      auto* y = (BlockIQ4NL*)out;
      for (int64_t b = 0; b < n / 32; ++b) {
        float amax = 0, mx = 0;
        for (int i = 0; i < 32; ++i)
          if (fabsf(x[32 * b + i]) > amax) { amax = fabsf(x[32 * b + i]); mx = x[32 * b + i]; }
        const float d = mx / -127.f, id = d ? 1.f / d : 0.f;
        y[b].d = fllm_fp32_to_fp16(d);
        for (int i = 0; i < 16; ++i)
          y[b].qs[i] = (uint8_t)(nearest_code_iq4(x[32 * b + i] * id) | (nearest_code_iq4(x[32 * b + 16 + i] * id) << 4));
      }
    } break;
    case FLLM_Q2_K: for (int64_t b = 0; b < n / QK_K; ++b) quantize_block_q2k(x + b * QK_K, (BlockQ2K*)out + b); break;
    case FLLM_Q3_K: for (int64_t b = 0; b < n / QK_K; ++b) quantize_block_q3k(x + b * QK_K, (BlockQ3K*)out + b); break;
    case FLLM_IQ4_XS: for (int64_t b = 0; b < n / QK_K; ++b) quantize_block_iq4xs(x + b * QK_K, (BlockIQ4XS*)out + b); break;
    case FLLM_Q4_K: for (int64_t b = 0; b < n / QK_K; ++b) quantize_block_q4k(x + b * QK_K, (BlockQ4K*)out + b); break;
    case FLLM_Q5_K: for (int64_t b = 0; b < n / QK_K; ++b) quantize_block_q5k(x + b * QK_K, (BlockQ5K*)out + b); break;
    case FLLM_Q6_K: for (int64_t b = 0; b < n / QK_K; ++b) quantize_block_q6k(x + b * QK_K, (BlockQ6K*)out + b); break;
    case FLLM_Q8_K: quantize_row_q8_K(x, (BlockQ8K*)out, n); break;
  }
}

static void dequantize_row(int type, const uint8_t* in, float* y, int64_t n) {
  switch (type) {
    case FLLM_F32: memcpy(y, in, n * 4); break;
    case FLLM_F16: for (int64_t i = 0; i < n; ++i) y[i] = fllm_fp16_to_fp32(((const uint16_t*)in)[i]); break;
    case FLLM_BF16: for (int64_t i = 0; i < n; ++i) y[i] = fllm_bf16_to_fp32(((const uint16_t*)in)[i]); break;
    case FLLM_FP8_E4M3: for (int64_t i = 0; i < n; ++i) y[i] = fllm_e4m3_to_fp32(in[i]); break;
    case FLLM_Q8_0: {
      auto* b = (const BlockQ8_0*)in;
      for (int64_t k = 0; k < n / 32; ++k) {
        const float d = fllm_fp16_to_fp32(b[k].d);
        for (int i = 0; i < 32; ++i) y[32 * k + i] = d * b[k].qs[i];
      }
    } break;
    case FLLM_Q4_0: {
      auto* b = (const BlockQ4_0*)in;
      for (int64_t k = 0; k < n / 32; ++k) {
        const float d = fllm_fp16_to_fp32(b[k].d);
        for (int i = 0; i < 16; ++i) {
          y[32 * k + i] = d * ((int)(b[k].qs[i] & 0xF) - 8);
          y[32 * k + 16 + i] = d * ((int)(b[k].qs[i] >> 4) - 8);
        }
      }
    } break;
    case FLLM_MXFP4: {
      auto* b = (const BlockMXFP4*)in;
      for (int64_t k = 0; k < n / 32; ++k) {
        const float d = ldexpf(1.f, (int)b[k].e - 127);
        for (int i = 0; i < 16; ++i) {
          y[32 * k + i] = d * fllm_e2m1_to_fp32(b[k].qs[i] & 0xF);
          y[32 * k + 16 + i] = d * fllm_e2m1_to_fp32(b[k].qs[i] >> 4);
        }
      }
    } break;
    case FLLM_NVFP4: {
      auto* b = (const BlockNVFP4*)in;
      for (int64_t k = 0; k < n / 16; ++k) {
        const float d = fllm_e4m3_to_fp32(b[k].scale);
        for (int i = 0; i < 8; ++i) {
          y[16 * k + 2 * i] = d * fllm_e2m1_to_fp32(b[k].qs[i] & 0xF);
          y[16 * k + 2 * i + 1] = d * fllm_e2m1_to_fp32(b[k].qs[i] >> 4);
        }
      }
    } break;
    case FLLM_Q4_1: {
      auto* b = (const BlockQ4_1*)in;
      for (int64_t k = 0; k < n / 32; ++k) {
        const float d = fllm_fp16_to_fp32(b[k].d), m = fllm_fp16_to_fp32(b[k].m);
        for (int i = 0; i < 16; ++i) {
          y[32 * k + i] = d * (b[k].qs[i] & 0xF) + m;
          y[32 * k + 16 + i] = d * (b[k].qs[i] >> 4) + m;
        }
      }
    } break;
    case FLLM_Q5_0: case FLLM_Q5_1: {
      for (int64_t k = 0; k < n / 32; ++k) {
        float d, m = 0.f;
        const uint8_t *qs, *qhp;
        if (type == FLLM_Q5_0) {
          auto* b = (const BlockQ5_0*)in + k;
          d = fllm_fp16_to_fp32(b->d); qs = b->qs; qhp = b->qh;
        } else {
          auto* b = (const BlockQ5_1*)in + k;
          d = fllm_fp16_to_fp32(b->d); m = fllm_fp16_to_fp32(b->m); qs = b->qs; qhp = b->qh;
        }
        uint32_t qh;
        memcpy(&qh, qhp, 4);
        for (int i = 0; i < 16; ++i) {
          const int a = (qs[i] & 0xF) | (((qh >> i) & 1) << 4);
          const int c = (qs[i] >> 4) | (((qh >> (i + 16)) & 1) << 4);
          y[32 * k + i] = type == FLLM_Q5_0 ? d * (a - 16) : d * a + m;
          y[32 * k + 16 + i] = type == FLLM_Q5_0 ? d * (c - 16) : d * c + m;
        }
      }
    } break;
    case FLLM_IQ4_NL: {
      auto* b = (const BlockIQ4NL*)in;
      for (int64_t k = 0; k < n / 32; ++k) {
        const float d = fllm_fp16_to_fp32(b[k].d);
        for (int i = 0; i < 16; ++i) {
          y[32 * k + i] = d * kIq4nl[b[k].qs[i] & 0xF];
          y[32 * k + 16 + i] = d * kIq4nl[b[k].qs[i] >> 4];
        }
      }
    } break;
    case FLLM_Q2_K: for (int64_t b = 0; b < n / QK_K; ++b) dequantize_block_q2k((const BlockQ2K*)in + b, y + b * QK_K); break;
    case FLLM_Q3_K: for (int64_t b = 0; b < n / QK_K; ++b) dequantize_block_q3k((const BlockQ3K*)in + b, y + b * QK_K); break;
    case FLLM_IQ4_XS: for (int64_t b = 0; b < n / QK_K; ++b) dequantize_block_iq4xs((const BlockIQ4XS*)in + b, y + b * QK_K); break;
    case FLLM_Q4_K: for (int64_t b = 0; b < n / QK_K; ++b) dequantize_block_q4k((const BlockQ4K*)in + b, y + b * QK_K); break;
    case FLLM_Q5_K: for (int64_t b = 0; b < n / QK_K; ++b) dequantize_block_q5k((const BlockQ5K*)in + b, y + b * QK_K); break;
    case FLLM_Q6_K: for (int64_t b = 0; b < n / QK_K; ++b) dequantize_block_q6k((const BlockQ6K*)in + b, y + b * QK_K); break;
    case FLLM_Q8_K: {
      auto* b = (const BlockQ8K*)in;
      for (int64_t k = 0; k < n / QK_K; ++k)
        for (int i = 0; i < QK_K; ++i) y[QK_K * k + i] = b[k].d * b[k].qs[i];
    } break;
  }
}

int fllm_quantize(int type, const float* src, void* dst, int64_t nrows, int64_t ncols) {
  const int64_t rb = fllm_row_bytes(type, ncols);
  if (rb < 0) return -1;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t r = 0; r < nrows; ++r) quantize_row(type, src + r * ncols, (uint8_t*)dst + r * rb, ncols);
  return 0;
}

int fllm_dequantize(int type, const void* src, float* dst, int64_t nrows, int64_t ncols) {
  const int64_t rb = fllm_row_bytes(type, ncols);
  if (rb < 0) return -1;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t r = 0; r < nrows; ++r) dequantize_row(type, (const uint8_t*)src + r * rb, dst + r * ncols, ncols);
  return 0;
}
