// Deterministic elementary functions shared by the host (g++) and device (nvcc) builds.
//
// Every function below is a fixed sequence of IEEE-754 binary32/binary64 operations
// (add, multiply, fused multiply-add, divide, square root, round-to-integer) and integer
// bit manipulation. All of those are correctly rounded on x86-64 and on sm_100a, so the
// two builds return the same bits for the same input. No libm / CUDA math-library
// transcendental is called anywhere on a hashed path: their results differ between
// platforms in the last place (the reference met this with torch's cos/sin,
// docs/unified-audit-results.md:24-25, and pins its own `repop.ops.exp/log/cos/sin`).
//
// Build rules that keep this true: host `-ffp-contract=off`, device `--fmad=false`; fused
// multiply-adds are always spelled `det_fmaf`/`det_fma`.
#pragma once
#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define DET_HD __host__ __device__ __forceinline__
#else
#define DET_HD inline
#endif

DET_HD float det_fmaf(float a, float b, float c) {
#if defined(__CUDA_ARCH__)
  return __fmaf_rn(a, b, c);
#else
  return fmaf(a, b, c);
#endif
}
DET_HD float det_addf(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fadd_rn(a, b);
#else
  return a + b;
#endif
}
DET_HD float det_mulf(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);
#else
  return a * b;
#endif
}
DET_HD float det_divf(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fdiv_rn(a, b);
#else
  return a / b;
#endif
}
DET_HD float det_sqrtf(float a) {
#if defined(__CUDA_ARCH__)
  return __fsqrt_rn(a);
#else
  return sqrtf(a);
#endif
}
DET_HD double det_fma(double a, double b, double c) {
#if defined(__CUDA_ARCH__)
  return __fma_rn(a, b, c);
#else
  return fma(a, b, c);
#endif
}
DET_HD float det_rintf(float a) {
#if defined(__CUDA_ARCH__)
  return rintf(a);  // cvt.rni: round to nearest even, exact
#else
  return nearbyintf(a);
#endif
}
DET_HD uint32_t det_f2u(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
#endif
}
DET_HD float det_u2f(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}

// bf16 <-> fp32 (round to nearest even; NaN kept quiet)
DET_HD uint16_t det_f2bf(float f) {
  uint32_t u = det_f2u(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
DET_HD float det_bf2f(uint16_t h) { return det_u2f(((uint32_t)h) << 16); }

// 1/sqrt(x): two correctly rounded operations.
DET_HD float det_rsqrtf(float x) { return det_divf(1.0f, det_sqrtf(x)); }

// 2^k for integer k in [-126, 127]
DET_HD float det_pow2i(int k) { return det_u2f((uint32_t)(k + 127) << 23); }

// exp(x), |rel err| about 1 ulp. Range reduction x = k ln2 + r, |r| <= ln2/2, degree-6
// polynomial in Horner form with explicit fma, result scaled by 2^k in two exact-ish steps so
// that overflow / gradual underflow follow IEEE multiplication.
DET_HD float det_expf(float x) {
  if (x != x) return x;
  if (x > 88.72284f) return det_u2f(0x7F800000u);
  if (x < -103.98f) return 0.0f;
  const float kf = det_rintf(det_mulf(x, 1.44269504088896341f));
  float r = det_fmaf(kf, -0.693359375f, x);          // ln2 high part (exact in 9 bits)
  r = det_fmaf(kf, 2.12194440e-4f, r);               // minus ln2 low part
  float p = 1.9875691500e-4f;
  p = det_fmaf(p, r, 1.3981999507e-3f);
  p = det_fmaf(p, r, 8.3334519073e-3f);
  p = det_fmaf(p, r, 4.1665795894e-2f);
  p = det_fmaf(p, r, 1.6666665459e-1f);
  p = det_fmaf(p, r, 5.0000001201e-1f);
  const float r2 = det_mulf(r, r);
  float y = det_addf(det_fmaf(p, r2, r), 1.0f);
  const int k = (int)kf;
  const int k1 = k / 2, k2 = k - k1;
  y = det_mulf(y, det_pow2i(k1));
  return det_mulf(y, det_pow2i(k2));
}

// natural log, x > 0 finite (0 -> -inf, negative -> NaN). Cephes-style: x = 2^e * m,
// m in [sqrt(1/2), sqrt(2)), polynomial in (m-1).
DET_HD float det_logf(float x) {
  if (x != x) return x;
  if (x < 0.0f) return det_u2f(0x7FC00000u);
  if (x == 0.0f) return det_u2f(0xFF800000u);
  uint32_t u = det_f2u(x);
  if (u == 0x7F800000u) return x;
  int e = 0;
  if (u < 0x00800000u) {  // subnormal: scale up by 2^23 exactly
    x = det_mulf(x, 8388608.0f);
    u = det_f2u(x);
    e = -23;
  }
  e += (int)(u >> 23) - 126;
  float m = det_u2f((u & 0x007FFFFFu) | 0x3F000000u);  // [0.5, 1)
  if (m < 0.70710678118654752f) {
    e -= 1;
    m = det_addf(det_addf(m, m), -1.0f);
  } else {
    m = det_addf(m, -1.0f);
  }
  const float z = det_mulf(m, m);
  float p = 7.0376836292e-2f;
  p = det_fmaf(p, m, -1.1514610310e-1f);
  p = det_fmaf(p, m, 1.1676998740e-1f);
  p = det_fmaf(p, m, -1.2420140846e-1f);
  p = det_fmaf(p, m, 1.4249322787e-1f);
  p = det_fmaf(p, m, -1.6668057665e-1f);
  p = det_fmaf(p, m, 2.0000714765e-1f);
  p = det_fmaf(p, m, -2.4999993993e-1f);
  p = det_fmaf(p, m, 3.3333331174e-1f);
  float y = det_mulf(det_mulf(m, z), p);
  const float ef = (float)e;
  y = det_fmaf(ef, -2.12194440e-4f, y);
  y = det_fmaf(z, -0.5f, y);
  float r = det_addf(m, y);
  r = det_fmaf(ef, 0.693359375f, r);
  return r;
}


// exp(x) for the attention kernels, x <= 0 (or -inf): same reduction and polynomial as det_expf,
// inputs below -87 return 0 so the 2^k scaling is a single exact-exponent multiply.
DET_HD float det_exp_attn(float x) {
  if (!(x >= -87.0f)) return 0.0f;
  const float kf = det_rintf(det_mulf(x, 1.44269504088896341f));
  float r = det_fmaf(kf, -0.693359375f, x);
  r = det_fmaf(kf, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = det_fmaf(p, r, 1.3981999507e-3f);
  p = det_fmaf(p, r, 8.3334519073e-3f);
  p = det_fmaf(p, r, 4.1665795894e-2f);
  p = det_fmaf(p, r, 1.6666665459e-1f);
  p = det_fmaf(p, r, 5.0000001201e-1f);
  const float r2 = det_mulf(r, r);
  const float y = det_addf(det_fmaf(p, r2, r), 1.0f);
  return det_mulf(y, det_pow2i((int)kf));
}

// 2^max(y, -126) for the attention kernels, y <= ~1. The clamp keeps the result a normal number (so the scaling is
// an exact exponent add) and makes the function branch-free; an input of -inf gives 2^-126, so MASKED scores are
// zeroed by the caller, not here. Round-to-nearest-integer by the 1.5*2^23 trick (two exact adds), r = y - k exact,
// degree-4 polynomial for 2^r on |r| <= 1/2, then k is added to the exponent field: (bits(t) << 23) is k << 23
// because the magic constant's own bits shift out.
DET_HD float det_exp2_attn(float y) {
  const float yc = fmaxf(y, -126.0f);
  const float t = det_addf(yc, 12582912.0f);
  const float kf = det_addf(t, -12582912.0f);
  const float r = det_fmaf(kf, -1.0f, yc);
  float p = 9.582852944731712e-3f;  // degree-4 minimax of 2^r on [-1/2, 1/2] with p(0) = 1: relative error 2.9e-6
  p = det_fmaf(p, r, 5.5906426161527634e-2f);
  p = det_fmaf(p, r, 2.4024099111557007e-1f);
  p = det_fmaf(p, r, 6.931241750717163e-1f);
  p = det_fmaf(p, r, 1.0f);
  return det_u2f(det_f2u(p) + (det_f2u(t) << 23));
}

// 2^max(y, -126) with a degree-6 polynomial (relative error about 1e-7): the loss kernels' exponential, where the sum
// of 128 K terms and the probabilities of the gradient want fp32 accuracy. Same construction as det_exp2_attn.
DET_HD float det_exp2_acc(float y) {
  const float yc = fmaxf(y, -126.0f);
  const float t = det_addf(yc, 12582912.0f);
  const float kf = det_addf(t, -12582912.0f);
  const float r = det_fmaf(kf, -1.0f, yc);
  float p = 1.5403530393381606e-4f;
  p = det_fmaf(p, r, 1.3333558146428443e-3f);
  p = det_fmaf(p, r, 9.6181291076284772e-3f);
  p = det_fmaf(p, r, 5.5504108664821580e-2f);
  p = det_fmaf(p, r, 2.4022650695910071e-1f);
  p = det_fmaf(p, r, 6.9314718055994531e-1f);
  p = det_fmaf(p, r, 1.0f);
  return det_u2f(det_f2u(p) + (det_f2u(t) << 23));
}

// sigmoid(x) = 1 / (1 + exp(-x))
DET_HD float det_sigmoidf(float x) { return det_divf(1.0f, det_addf(1.0f, det_expf(-x))); }

// 1 / d for a normal d >= 1: integer-seeded first guess (within 12.5 %) and three Newton steps r <- r (2 - d r), every
// step one fma and one multiply; relative error about 1e-7. Not correctly rounded, but the same bits everywhere.
DET_HD float det_recip_ge1(float d) {
  float r = det_u2f(0x7EF311C7u - det_f2u(d));
  r = det_mulf(r, det_fmaf(-d, r, 2.0f));
  r = det_mulf(r, det_fmaf(-d, r, 2.0f));
  r = det_mulf(r, det_fmaf(-d, r, 2.0f));
  return r;
}
// sigmoid for the SwiGLU kernels: e = 2^clamp(-x log2(e), -126, 126) through det_exp2_acc, then 1 / (1 + e) by
// det_recip_ge1. Branch-free, so two values go through packed fp32 instructions on the GPU.
DET_HD float det_sigmoid_fastf(float x) {
  const float y = fminf(fmaxf(det_mulf(x, -1.44269504088896341f), -126.0f), 126.0f);
  return det_recip_ge1(det_addf(1.0f, det_exp2_acc(y)));
}

// ---- double precision sin/cos for the RoPE tables (argument up to ~1e6) ---------------
// Cody-Waite reduction by pi/2 in three parts followed by Taylor polynomials; the table value
// is the double result rounded once to binary32.
DET_HD void det_sincos(double x, double* s_out, double* c_out) {
  const double two_over_pi = 0.63661977236758134308;
  const double p1 = 1.57079632673412561417e+00;  // pi/2 high 33 bits
  const double p2 = 6.07710050650619224932e-11;
  const double p3 = 2.02226624879595063154e-21;
  double kd = x * two_over_pi;
  kd = (kd >= 0.0) ? (double)(long long)(kd + 0.5) : -(double)(long long)(-kd + 0.5);
  double r = det_fma(-kd, p1, x);
  r = det_fma(-kd, p2, r);
  r = det_fma(-kd, p3, r);
  const double z = r * r;
  double sp = 1.58969099521155010221e-10;
  sp = det_fma(sp, z, -2.50507602534068634195e-08);
  sp = det_fma(sp, z, 2.75573137070700676789e-06);
  sp = det_fma(sp, z, -1.98412698298579493134e-04);
  sp = det_fma(sp, z, 8.33333333332248946124e-03);
  sp = det_fma(sp, z, -1.66666666666666324348e-01);
  const double sv = det_fma(r * z, sp, r);
  double cp = -1.13596475577881948265e-11;
  cp = det_fma(cp, z, 2.08757232129817482790e-09);
  cp = det_fma(cp, z, -2.75573143513906633035e-07);
  cp = det_fma(cp, z, 2.48015872894767294178e-05);
  cp = det_fma(cp, z, -1.38888888888741095749e-03);
  cp = det_fma(cp, z, 4.16666666666666019037e-02);
  const double cv = det_fma(z * z, cp, det_fma(z, -0.5, 1.0));
  const long long k = (long long)kd;
  switch ((int)(k & 3)) {
    case 0: *s_out = sv; *c_out = cv; break;
    case 1: *s_out = cv; *c_out = -sv; break;
    case 2: *s_out = -sv; *c_out = -cv; break;
    default: *s_out = -cv; *c_out = sv; break;
  }
}

// base^n for a non-negative integer n by binary exponentiation in double (each step one
// correctly rounded multiply): the Adam bias-correction powers.
DET_HD double det_powi(double base, long long n) {
  double result = 1.0, b = base;
  while (n > 0) {
    if (n & 1) result = result * b;
    b = b * b;
    n >>= 1;
  }
  return result;
}
