/*
 * Seeded, counter-based tensor initialisation shared by host C code and CUDA device code.
 *
 * The reference never initialises its weights, biases, masks or inputs (bare cudaMalloc at
 * src/layer/linear.h:40,92, src/layer/bert_layer.h:45,115-118, src/layer/operator.h:29-30,
 * src/test_schedule.h:29-31), so any result check needs a generator that yields the same
 * values on the CPU and on the GPU.  Everything here is built from IEEE-754 operations that
 * are correctly rounded on both sides (add, mul, div, sqrt, fma) -- no libm transcendental --
 * so host and device agree bit for bit.
 *
 * element(seed, tensor_id, idx) -> Philox4x32-10(counter = (idx/4, 0, tensor_id, 0),
 *                                               key = (seed, 0x4c494752)) word idx%4
 *                               -> u = (k+0.5)/2^23 in (0,1) -> z = Phi^-1(u) (Acklam rational approximation)
 *                               -> mean + std * z -> rounded to fp16 (RNE).
 */
#ifndef LIGER_RNG_H
#define LIGER_RNG_H

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define LIGER_HD __host__ __device__ __forceinline__
#else
#define LIGER_HD static inline
#endif

/* ---- exact-op helpers: identical rounding on host and device --------------------------- */
#if defined(__CUDA_ARCH__)
#define LG_MUL(a, b) __fmul_rn((a), (b))
#define LG_ADD(a, b) __fadd_rn((a), (b))
#define LG_DIV(a, b) __fdiv_rn((a), (b))
#define LG_SQRT(a) __fsqrt_rn((a))
#define LG_FMA(a, b, c) __fmaf_rn((a), (b), (c))
#else
#include <math.h>
/* volatile temporaries stop the host compiler from contracting mul+add into fma */
static inline float lg_mul_(float a, float b) { volatile float r = a * b; return r; }
static inline float lg_add_(float a, float b) { volatile float r = a + b; return r; }
static inline float lg_div_(float a, float b) { volatile float r = a / b; return r; }
#define LG_MUL(a, b) lg_mul_((a), (b))
#define LG_ADD(a, b) lg_add_((a), (b))
#define LG_DIV(a, b) lg_div_((a), (b))
#define LG_SQRT(a) sqrtf((a))
#define LG_FMA(a, b, c) fmaf((a), (b), (c))
#endif

LIGER_HD uint32_t lg_mulhi32(uint32_t a, uint32_t b) {
  return (uint32_t)(((uint64_t)a * (uint64_t)b) >> 32);
}

/* Philox4x32-10 (Salmon et al., SC'11); constants are the published ones. */
LIGER_HD void lg_philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0 = lg_mulhi32(0xD2511F53u, c[0]);
    uint32_t lo0 = 0xD2511F53u * c[0];
    uint32_t hi1 = lg_mulhi32(0xCD9E8D57u, c[2]);
    uint32_t lo1 = 0xCD9E8D57u * c[2];
    uint32_t n0 = hi1 ^ c[1] ^ k0;
    uint32_t n1 = lo1;
    uint32_t n2 = hi0 ^ c[3] ^ k1;
    uint32_t n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

LIGER_HD float lg_bits_to_float(uint32_t b) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(b);
#else
  float f; memcpy(&f, &b, 4); return f;
#endif
}
LIGER_HD uint32_t lg_float_to_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t b; memcpy(&b, &f, 4); return b;
#endif
}

/* natural log of a positive normal float from exact ops only (|rel err| ~ 2e-7) */
LIGER_HD float lg_det_logf(float x) {
  uint32_t b = lg_float_to_bits(x);
  int e = (int)(b >> 23) - 127;
  float m = lg_bits_to_float((b & 0x007FFFFFu) | 0x3F800000u); /* [1,2) */
  if (m > 1.41421356f) { m = LG_MUL(m, 0.5f); e += 1; }
  float f = LG_ADD(m, -1.0f);
  float s = LG_DIV(f, LG_ADD(2.0f, f));
  float z = LG_MUL(s, s);
  float p = 0.181818182f;              /* 2/11 */
  p = LG_FMA(p, z, 0.222222222f);      /* 2/9 */
  p = LG_FMA(p, z, 0.285714286f);      /* 2/7 */
  p = LG_FMA(p, z, 0.4f);              /* 2/5 */
  p = LG_FMA(p, z, 0.666666667f);      /* 2/3 */
  float r = LG_FMA(LG_MUL(s, z), p, LG_MUL(2.0f, s));
  return LG_FMA((float)e, 0.693147181f, r);
}

/* inverse standard-normal CDF, Acklam's rational approximation evaluated in fp32 */
LIGER_HD float lg_inv_normal_cdf(float u) {
  const float a0 = -3.969683028665376e+01f, a1 = 2.209460984245205e+02f, a2 = -2.759285104469687e+02f,
              a3 = 1.383577518672690e+02f, a4 = -3.066479806614716e+01f, a5 = 2.506628277459239e+00f;
  const float b0 = -5.447609879822406e+01f, b1 = 1.615858368580409e+02f, b2 = -1.556989798598866e+02f,
              b3 = 6.680131188771972e+01f, b4 = -1.328068155288572e+01f;
  const float c0 = -7.784894002430293e-03f, c1 = -3.223964580411365e-01f, c2 = -2.400758277161838e+00f,
              c3 = -2.549732539343734e+00f, c4 = 4.374664141464968e+00f, c5 = 2.938163982698783e+00f;
  const float d0 = 7.784695709041462e-03f, d1 = 3.224671290700398e-01f, d2 = 2.445134137142996e+00f,
              d3 = 3.754408661907416e+00f;
  const float plow = 0.02425f;
  if (u < plow || u > 1.0f - plow) {
    float t = (u < plow) ? u : LG_ADD(1.0f, -u);
    float q = LG_SQRT(LG_MUL(-2.0f, lg_det_logf(t)));
    float num = c0;
    num = LG_FMA(num, q, c1); num = LG_FMA(num, q, c2); num = LG_FMA(num, q, c3);
    num = LG_FMA(num, q, c4); num = LG_FMA(num, q, c5);
    float den = d0;
    den = LG_FMA(den, q, d1); den = LG_FMA(den, q, d2); den = LG_FMA(den, q, d3);
    den = LG_FMA(den, q, 1.0f);
    float v = LG_DIV(num, den);
    return (u < plow) ? v : -v;
  }
  float q = LG_ADD(u, -0.5f);
  float r = LG_MUL(q, q);
  float num = a0;
  num = LG_FMA(num, r, a1); num = LG_FMA(num, r, a2); num = LG_FMA(num, r, a3);
  num = LG_FMA(num, r, a4); num = LG_FMA(num, r, a5);
  float den = b0;
  den = LG_FMA(den, r, b1); den = LG_FMA(den, r, b2); den = LG_FMA(den, r, b3);
  den = LG_FMA(den, r, b4); den = LG_FMA(den, r, 1.0f);
  return LG_DIV(LG_MUL(num, q), den);
}

/* fp32 -> fp16 bits, round to nearest even, with subnormals and overflow to inf */
LIGER_HD uint16_t lg_float_to_half_bits(float f) {
  uint32_t x = lg_float_to_bits(f);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t ax = x & 0x7FFFFFFFu;
  if (ax >= 0x7F800000u) return (uint16_t)(sign | (ax > 0x7F800000u ? 0x7E00u : 0x7C00u));
  if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to >= 65520 -> inf */
  if (ax < 0x33000001u) return (uint16_t)sign;               /* < 2^-25 (or == 2^-25 tie->0) */
  int e = (int)(ax >> 23) - 127;
  uint32_t man = (ax & 0x007FFFFFu) | 0x00800000u;
  int shift;
  uint32_t base;
  if (e < -14) { shift = 13 + (-14 - e); base = 0; }
  else { shift = 13; base = (uint32_t)(e + 15) << 10; man &= 0x007FFFFFu; }
  uint32_t q = man >> shift;
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q += 1;
  return (uint16_t)(sign | (base + q));
}

LIGER_HD float lg_half_bits_to_float(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1Fu;
  uint32_t m = h & 0x3FFu;
  if (e == 0) {
    if (m == 0) return lg_bits_to_float(sign);
    /* subnormal: m * 2^-24, exactly representable */
    float v = (float)m * 5.9604644775390625e-08f;
    return sign ? -v : v;
  }
  if (e == 31) return lg_bits_to_float(sign | 0x7F800000u | (m << 13));
  return lg_bits_to_float(sign | ((e + 112u) << 23) | (m << 13));
}

/* One element of tensor `tensor_id`: fp16 bits of mean + std * N(0,1). */
LIGER_HD uint16_t lg_normal_half_bits(uint32_t seed, uint32_t tensor_id, uint64_t idx, float mean, float std) {
  uint32_t c[4];
  uint64_t blk = idx >> 2;
  c[0] = (uint32_t)blk; c[1] = (uint32_t)(blk >> 32); c[2] = tensor_id; c[3] = 0u;
  lg_philox4x32_10(c, seed, 0x4c494752u);
  uint32_t w = c[idx & 3u];
  /* 23 random bits: k + 0.5 is exact in fp32 and u stays strictly inside (0,1) */
  float u = LG_MUL(LG_ADD((float)(w >> 9), 0.5f), 1.1920928955078125e-07f); /* (k+0.5)/2^23 */
  float z = lg_inv_normal_cdf(u);
  return lg_float_to_half_bits(LG_FMA(std, z, mean));
}

#endif /* LIGER_RNG_H */
