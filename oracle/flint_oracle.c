/* TEST INFRASTRUCTURE -- not product code. See flint_oracle.h for what this restates and how it
 * is pinned. Compile with -ffp-contract=off so that no product-sum is fused behind our back. */
#include "flint_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---- scalar codecs -------------------------------------------------------------------- */

float fo_e4m3_decode(uint8_t code) {
  /* flint/cuda/gemm_fp8_cutlass_test.cc:95-102 */
  int sign = code >> 7;
  int exponent = (code >> 3) & 0xf;
  int mantissa = code & 0x7;
  float mag;
  if (exponent == 0xf && mantissa == 0x7) return NAN; /* flint/dtype.h:80-86: no inf, one NaN */
  if (exponent == 0) {
    mag = ldexpf((float)mantissa, -9);
  } else {
    mag = ldexpf(1.0f + (float)mantissa / 8.0f, exponent - 7);
  }
  return sign ? -mag : mag;
}

uint8_t fo_e4m3_encode(float x) {
  /* tools/model_writer.py:170-172: clamp to +-448, then round to nearest even. */
  uint8_t sign;
  float a;
  int e;
  float m;
  int q;
  if (isnan(x)) return 0x7f;
  sign = signbit(x) ? 0x80 : 0x00;
  a = fabsf(x);
  if (a > 448.0f) a = 448.0f;
  if (a < 0.015625f) { /* below the smallest normal 2^-6: subnormal grid of 2^-9 */
    q = (int)nearbyintf(a * 512.0f); /* exact scaling; RNE in the default rounding mode */
    return (uint8_t)(sign | q);      /* q == 8 is 0x08, the smallest normal */
  }
  m = frexpf(a, &e); /* a = m * 2^e, m in [0.5, 1) */
  m *= 2.0f;
  e -= 1;
  q = (int)nearbyintf((m - 1.0f) * 8.0f);
  if (q == 8) {
    q = 0;
    e += 1;
  }
  return (uint8_t)(sign | ((e + 7) << 3) | q);
}

static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

float fo_e2m1_decode(uint8_t nibble) {
  float mag = kE2M1[nibble & 7];
  return (nibble & 8) ? -mag : mag;
}

uint8_t fo_e2m1_encode(float x) {
  uint8_t sign;
  float a;
  int code;
  if (isnan(x)) return 0x7; /* the format has no NaN; saturate */
  sign = signbit(x) ? 0x8 : 0x0;
  a = fabsf(x);
  /* Nearest of the eight magnitudes; a tie goes to the even code. */
  if (a <= 0.25f) code = 0;
  else if (a < 0.75f) code = 1;
  else if (a <= 1.25f) code = 2;
  else if (a < 1.75f) code = 3;
  else if (a <= 2.5f) code = 4;
  else if (a < 3.5f) code = 5;
  else if (a <= 5.0f) code = 6;
  else code = 7;
  return (uint8_t)(sign | code);
}

uint16_t fo_bf16_from_f32(float x) {
  /* waifu/src/qwen_image/pipeline.rs:69-76 */
  uint32_t bits;
  memcpy(&bits, &x, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x0040u);
  bits += 0x7fffu + ((bits >> 16) & 1u);
  return (uint16_t)(bits >> 16);
}

float fo_bf16_to_f32(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
  float x;
  memcpy(&x, &bits, 4);
  return x;
}

uint16_t fo_f16_from_f32(float x) {
  uint32_t bits, sign, mant;
  int32_t exp;
  memcpy(&bits, &x, 4);
  sign = (bits >> 16) & 0x8000u;
  exp = (int32_t)((bits >> 23) & 0xff);
  mant = bits & 0x7fffffu;
  if (exp == 0xff) return (uint16_t)(sign | 0x7c00u | (mant ? 0x200u : 0)); /* inf / NaN */
  exp = exp - 127 + 15;
  if (exp >= 0x1f) return (uint16_t)(sign | 0x7c00u); /* overflow -> inf */
  if (exp <= 0) {
    /* subnormal half (or zero): shift the 24-bit significand, RNE */
    uint32_t sig, shift, halfway, rem, q;
    if (exp < -10) return (uint16_t)sign;
    sig = mant | 0x800000u;
    shift = (uint32_t)(14 - exp); /* 14..24 */
    q = sig >> shift;
    rem = sig & ((1u << shift) - 1u);
    halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q += 1;
    return (uint16_t)(sign | q);
  }
  {
    uint32_t q = ((uint32_t)exp << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q += 1; /* carries into the exponent */
    return (uint16_t)(sign | q);
  }
}

float fo_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  int exp = (h >> 10) & 0x1f;
  uint32_t mant = h & 0x3ffu;
  float mag;
  uint32_t bits;
  if (exp == 0x1f) {
    bits = sign | 0x7f800000u | (mant << 13);
    memcpy(&mag, &bits, 4);
    return mag;
  }
  if (exp == 0) mag = ldexpf((float)mant, -24);
  else mag = ldexpf(1.0f + (float)mant / 1024.0f, exp - 15);
  return sign ? -mag : mag;
}

static inline float widen16(uint16_t v, int is_bf16) {
  return is_bf16 ? fo_bf16_to_f32(v) : fo_f16_to_f32(v);
}

/* ---- quantizers ------------------------------------------------------------------------ */

void fo_quantize_fp8_tensor(const float *w, int64_t numel, uint8_t *codes, float *scale) {
  float amax = 0.0f;
  float s, divisor;
  int64_t i;
  for (i = 0; i < numel; ++i) {
    float a = fabsf(w[i]);
    if (a > amax) amax = a;
  }
  s = amax / 448.0f;
  divisor = s > 0.0f ? s : 1.0f; /* model_writer.py:168 */
  for (i = 0; i < numel; ++i) codes[i] = fo_e4m3_encode(w[i] / divisor);
  *scale = s;
}

void fo_quantize_fp8_rows(const float *w, int rows, int k, uint8_t *codes, float *scales) {
  int r;
#pragma omp parallel for schedule(static)
  for (r = 0; r < rows; ++r) {
    fo_quantize_fp8_tensor(w + (int64_t)r * k, k, codes + (int64_t)r * k, scales + r);
  }
}

void fo_quantize_fp8_act(const uint16_t *x, int is_bf16, int rows, int k, uint8_t *codes,
                         float *scales) {
  int r;
#pragma omp parallel for schedule(static)
  for (r = 0; r < rows; ++r) {
    const uint16_t *row = x + (int64_t)r * k;
    uint8_t *out = codes + (int64_t)r * k;
    float amax = 0.0f, s, divisor, inv;
    int j;
    for (j = 0; j < k; ++j) {
      float a = fabsf(widen16(row[j], is_bf16));
      if (a > amax) amax = a;
    }
    s = amax / 448.0f;
    divisor = s > 0.0f ? s : 1.0f;
    inv = 1.0f / divisor; /* one IEEE reciprocal per row, then one multiply per element */
    for (j = 0; j < k; ++j) out[j] = fo_e4m3_encode(widen16(row[j], is_bf16) * inv);
    scales[r] = s;
  }
}

void fo_quantize_fp8_act_amax(const uint16_t *x, int is_bf16, int rows, int k, const float *amax,
                              uint8_t *codes, float *scales) {
  /* fo_quantize_fp8_act with the rows' maxima given (taken over a wider row than x). */
  int r;
#pragma omp parallel for schedule(static)
  for (r = 0; r < rows; ++r) {
    const uint16_t *row = x + (int64_t)r * k;
    uint8_t *out = codes + (int64_t)r * k;
    float s = amax[r] / 448.0f, divisor, inv;
    int j;
    divisor = s > 0.0f ? s : 1.0f;
    inv = 1.0f / divisor;
    for (j = 0; j < k; ++j) out[j] = fo_e4m3_encode(widen16(row[j], is_bf16) * inv);
    scales[r] = s;
  }
}

static void nvfp4_block(const float *v, float global, uint8_t *codes8, uint8_t *scale_code) {
  /* 16 values -> 8 bytes of e2m1 pairs + one unsigned e4m3 block scale. */
  float amax = 0.0f, sdec, denom, inv;
  uint8_t sc;
  int j;
  for (j = 0; j < 16; ++j) {
    float a = fabsf(v[j]);
    if (a > amax) amax = a;
  }
  sc = (global > 0.0f) ? fo_e4m3_encode(amax / (6.0f * global)) : 0;
  sdec = fo_e4m3_decode(sc);
  denom = sdec * global;
  if (!(denom > 0.0f)) {
    memset(codes8, 0, 8);
    *scale_code = 0;
    return;
  }
  inv = 1.0f / denom; /* one IEEE reciprocal per block, then one multiply per element */
  for (j = 0; j < 8; ++j) {
    uint8_t lo = fo_e2m1_encode(v[2 * j] * inv);
    uint8_t hi = fo_e2m1_encode(v[2 * j + 1] * inv);
    codes8[j] = (uint8_t)(lo | (hi << 4));
  }
  *scale_code = sc;
}

void fo_quantize_nvfp4_weight(const float *w, int rows, int k, uint8_t *codes,
                              uint8_t *block_scales, float *global_scale) {
  float amax = 0.0f, g;
  int64_t i, numel = (int64_t)rows * k;
  int r;
  for (i = 0; i < numel; ++i) {
    float a = fabsf(w[i]);
    if (a > amax) amax = a;
  }
  g = amax / (448.0f * 6.0f);
  *global_scale = g;
#pragma omp parallel for schedule(static)
  for (r = 0; r < rows; ++r) {
    int b;
    for (b = 0; b < k / 16; ++b) {
      nvfp4_block(w + (int64_t)r * k + 16 * b, g, codes + ((int64_t)r * k) / 2 + 8 * b,
                  block_scales + (int64_t)r * (k / 16) + b);
    }
  }
}

void fo_quantize_nvfp4_act(const uint16_t *x, int is_bf16, int rows, int k, uint8_t *codes,
                           uint8_t *block_scales) {
  int r;
#pragma omp parallel for schedule(static)
  for (r = 0; r < rows; ++r) {
    int b, j;
    float v[16];
    for (b = 0; b < k / 16; ++b) {
      for (j = 0; j < 16; ++j) v[j] = widen16(x[(int64_t)r * k + 16 * b + j], is_bf16);
      nvfp4_block(v, 1.0f, codes + ((int64_t)r * k) / 2 + 8 * b,
                  block_scales + (int64_t)r * (k / 16) + b);
    }
  }
}

/* ---- decoders -------------------------------------------------------------------------- */

void fo_decode_e4m3(const uint8_t *codes, int64_t numel, float *out) {
  float table[256];
  int64_t i;
  int c;
  for (c = 0; c < 256; ++c) table[c] = fo_e4m3_decode((uint8_t)c);
#pragma omp parallel for schedule(static)
  for (i = 0; i < numel; ++i) out[i] = table[codes[i]];
}

void fo_decode_nvfp4(const uint8_t *codes, const uint8_t *block_scales, int rows, int k,
                     float *out) {
  int r;
#pragma omp parallel for schedule(static)
  for (r = 0; r < rows; ++r) {
    int j;
    for (j = 0; j < k; ++j) {
      uint8_t byte = codes[((int64_t)r * k + j) / 2];
      uint8_t nib = (j & 1) ? (byte >> 4) : (byte & 0xf);
      float s = fo_e4m3_decode(block_scales[(int64_t)r * (k / 16) + j / 16]);
      out[(int64_t)r * k + j] = fo_e2m1_decode(nib) * s;
    }
  }
}

void fo_widen_16(const uint16_t *x, int is_bf16, int64_t numel, float *out) {
  int64_t i;
#pragma omp parallel for schedule(static)
  for (i = 0; i < numel; ++i) out[i] = widen16(x[i], is_bf16);
}

void fo_narrow_16(const float *x, int is_bf16, int64_t numel, uint16_t *out) {
  int64_t i;
#pragma omp parallel for schedule(static)
  for (i = 0; i < numel; ++i) out[i] = is_bf16 ? fo_bf16_from_f32(x[i]) : fo_f16_from_f32(x[i]);
}

/* ---- products -------------------------------------------------------------------------- */

void fo_gemm_f32_nt(const float *a, const float *b, float *c, int m, int n, int k) {
  /* Row block of A against row blocks of B; eight interleaved partial sums per dot product so
   * that the compiler can keep them in one vector register. fp32 throughout. */
  int i;
#pragma omp parallel for schedule(dynamic, 4)
  for (i = 0; i < m; ++i) {
    const float *ar = a + (int64_t)i * k;
    int j;
    for (j = 0; j < n; ++j) {
      const float *br = b + (int64_t)j * k;
      float part[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      float sum;
      int p, q;
      for (p = 0; p + 8 <= k; p += 8) {
        for (q = 0; q < 8; ++q) part[q] += ar[p + q] * br[p + q];
      }
      sum = ((part[0] + part[4]) + (part[1] + part[5])) + ((part[2] + part[6]) + (part[3] + part[7]));
      for (; p < k; ++p) sum += ar[p] * br[p];
      c[(int64_t)i * n + j] = sum;
    }
  }
}

void fo_gemm_f64_nt(const float *a, const float *b, double *c, int m, int n, int k) {
  int i;
#pragma omp parallel for schedule(dynamic, 4)
  for (i = 0; i < m; ++i) {
    int j, p;
    for (j = 0; j < n; ++j) {
      double sum = 0.0;
      for (p = 0; p < k; ++p) sum += (double)a[(int64_t)i * k + p] * (double)b[(int64_t)j * k + p];
      c[(int64_t)i * n + j] = sum;
    }
  }
}

static inline float gelu_tanh(float x) {
  /* waifu/src/krea2/dit.rs:170-188: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) */
  const float kAlpha = 0.7978845608028654f;
  float inner = kAlpha * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + (float)tanh((double)inner));
}

void fo_epilogue(const float *acc, int m, int n, const float *row_scale, const float *col_scale,
                 int col_scale_count, float global_scale, const uint16_t *bias,
                 const uint16_t *residual, int act, int out_is_bf16, uint16_t *out) {
  int i;
#pragma omp parallel for schedule(static)
  for (i = 0; i < m; ++i) {
    int j;
    float rs = row_scale ? row_scale[i] : 1.0f;
    for (j = 0; j < n; ++j) {
      float cs = col_scale ? (col_scale_count == 1 ? col_scale[0] : col_scale[j]) : 1.0f;
      float v = acc[(int64_t)i * n + j] * (rs * cs);
      if (global_scale != 1.0f) v *= global_scale;
      if (bias) v += widen16(bias[j], out_is_bf16);
      if (act == FO_ACT_GELU_TANH) v = gelu_tanh(v);
      if (residual) v += widen16(residual[(int64_t)i * n + j], out_is_bf16);
      out[(int64_t)i * n + j] = out_is_bf16 ? fo_bf16_from_f32(v) : fo_f16_from_f32(v);
    }
  }
}
