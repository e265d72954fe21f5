// CPU twins of csrc/cuda/qat_int8.cu and of the int8 tensor-core GEMM: the same operations in the same order
// (IEEE division, round-half-even, exact int32 accumulation, lane-tree row sums), so a quantised layer replays
// with identical bits on a plain CPU.
#include <float.h>
#include <math.h>
#include <stdint.h>

#include <algorithm>
#include <vector>

#include "det_math.h"
#include "det_reduce.h"

namespace {

struct BF16 { uint16_t v; };
template <typename T> inline float ld(const T* p, long i);
template <> inline float ld<float>(const float* p, long i) { return p[i]; }
template <> inline float ld<BF16>(const BF16* p, long i) { return det_bf2f(p[i].v); }
template <typename T> inline void st(T* p, long i, float f);
template <> inline void st<float>(float* p, long i, float f) { p[i] = f; }
template <> inline void st<BF16>(BF16* p, long i, float f) { p[i].v = det_f2bf(f); }

inline float clamp_q(float q, float qmax) { return std::min(std::max(q, -qmax), qmax); }

#define DISPATCH_T(is_bf16, ...)              \
  if (is_bf16) { using T = BF16; __VA_ARGS__ } \
  else { using T = float; __VA_ARGS__ }

template <typename T>
void quant_act(const T* x, long n, float step, float qmax, int8_t* q) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < n; ++i) q[i] = (int8_t)(int)clamp_q(rintf(ld(x, i) / step), qmax);
}

template <typename T, typename TO>
void quant_weight(const T* w, const float* s, long N, int K, float qmax, int8_t* q, TO* w_hat) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < N; ++r)
    for (int k = 0; k < K; ++k) {
      const float t = clamp_q(rintf(ld(w, r * K + k) / s[r]), qmax);
      q[r * K + k] = (int8_t)(int)t;
      if (w_hat) st(w_hat, r * K + k, t * s[r]);
    }
}

template <typename T>
void lsq_bwd(const float* G, const T* w, const float* s, float a, long N, int K, float qmax, float gs, float* dW,
             float* ds, int learn_step) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < N; ++r) {
    float part[32];
    for (int l = 0; l < 32; ++l) part[l] = 0.0f;
    for (int k = 0; k < K; ++k) {
      const int l = (k / 8) % 32;
      const float t = ld(w, r * K + k) / s[r];
      const float gv = G[r * K + k] * a;
      const bool inside = fabsf(t) <= qmax;
      const float term = inside ? rintf(t) - t : (t > 0.0f ? qmax : -qmax);
      part[l] = det_fmaf(gv, term, part[l]);
      if (inside) dW[r * K + k] = dW[r * K + k] + gv;
    }
    if (learn_step) ds[r] = ds[r] + det_butterfly_host(part, 32) * gs;
  }
}

template <typename T>
void row_stat(const T* w, long N, int K, int mode, float c, float floor_v, float* s) {
  const float inv_k = 1.0f / (float)K;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < N; ++r) {
    float part[32];
    for (int l = 0; l < 32; ++l) part[l] = 0.0f;
    for (int k = 0; k < K; ++k) {
      const int l = (k / 8) % 32;
      const float f = fabsf(ld(w, r * K + k));
      part[l] = mode == 0 ? part[l] + f : std::max(part[l], f);
    }
    float v;
    if (mode == 0) {
      v = det_butterfly_host(part, 32) * inv_k * c;
    } else {
      float m = 0.0f;
      for (int l = 0; l < 32; ++l) m = std::max(m, part[l]);
      v = m * c;
    }
    s[r] = std::max(v, floor_v);
  }
}

}  // namespace

extern "C" {

int otb_cpu_absmax(const void* x, long n, int dtype, float* amax) {
  float m = 0.0f;
  DISPATCH_T(dtype, for (long i = 0; i < n; ++i) m = std::max(m, fabsf(ld((const T*)x, i)));)
  amax[0] = m;
  return 0;
}

int otb_cpu_quant_act(const void* x, long n, int dtype, const float* amax, int qmax, void* qv, float* step_out) {
  const float inv = 1.0f / (float)qmax;
  const float step = std::max(amax[0] * inv, FLT_MIN);
  step_out[0] = step;
  DISPATCH_T(dtype, quant_act<T>((const T*)x, n, step, (float)qmax, (int8_t*)qv);)
  return 0;
}

int otb_cpu_quant_weight(const void* w, const float* s, long N, int K, int dtype, int qmax, void* qv, void* w_hat,
                         int out_dtype) {
  if (out_dtype) {
    DISPATCH_T(dtype, (quant_weight<T, BF16>((const T*)w, s, N, K, (float)qmax, (int8_t*)qv, (BF16*)w_hat));)
  } else {
    DISPATCH_T(dtype, (quant_weight<T, float>((const T*)w, s, N, K, (float)qmax, (int8_t*)qv, (float*)w_hat));)
  }
  return 0;
}

int otb_cpu_lsq_bwd(const float* G, const void* w, const float* s, const float* ga, long N, int K, int dtype, int qmax,
                    float gs, float* dW, float* ds, int learn_step) {
  DISPATCH_T(dtype, lsq_bwd<T>(G, (const T*)w, s, ga ? ga[0] : 1.0f, N, K, (float)qmax, gs, dW, ds, learn_step);)
  return 0;
}

int otb_cpu_row_stat(const void* w, long N, int K, int dtype, int mode, float c, float floor_v, float* s) {
  DISPATCH_T(dtype, row_stat<T>((const T*)w, N, K, mode, c, floor_v, s);)
  return 0;
}

int otb_cpu_i8_widen(const void* qv, void* out, long n, int out_dtype) {
  const int8_t* q = (const int8_t*)qv;
  if (out_dtype) for (long i = 0; i < n; ++i) st((BF16*)out, i, (float)q[i]);
  else for (long i = 0; i < n; ++i) st((float*)out, i, (float)q[i]);
  return 0;
}

// C = float(int32 sum) * (sa * sb[n]) (+ residual); epi 0 bf16-or-fp32 store per out_dtype, 3 adds residual R first.
int otb_cpu_gemm_i8(const void* Av, const void* Bv, void* C, const void* R, int M, int N, int K, long lda, long ldb,
                    long ldc, long ldr, const float* sa, const float* sb, int epi, int out_dtype) {
  const int8_t* A = (const int8_t*)Av;
  const int8_t* B = (const int8_t*)Bv;
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    for (int n = 0; n < N; ++n) {
      int32_t acc = 0;
      for (int k = 0; k < K; ++k) acc += (int32_t)A[m * lda + k] * (int32_t)B[n * ldb + k];
      float v = (float)acc * (sa[0] * sb[n]);
      if (epi == 3) v = v + (out_dtype ? ld((const BF16*)R, m * ldr + n) : ld((const float*)R, m * ldr + n));
      if (out_dtype) st((BF16*)C, m * ldc + n, v);
      else st((float*)C, m * ldc + n, v);
    }
  }
  return 0;
}

}  // extern "C"
