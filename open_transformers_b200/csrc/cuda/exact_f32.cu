// Exact fp32 family on CUDA cores: GEMM and attention whose every dot product is the single chain
//   acc = fma(a_k, b_k, acc), k ascending, acc starting at +0
// i.e. bit-identical to csrc/cpu/ref_gemm_attn.cpp. Used when activations are fp32
// (run.mixed_precision = false: the tiny reproducibility configs, the fp32 audit replay); the
// throughput path is the tcgen05 family.
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "det_math.h"

namespace {

// ------------------------------------------------------------------------------ GEMM
constexpr int GT = 64, GK = 16;
template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                const float* __restrict__ R, int M, int N, int K, long lda, long ldb, long ldc, long ldr) {
  __shared__ float sa[GK][GT + 1], sb[GK][GT + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // the accumulating epilogue continues the chain from the value already in C
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      acc[i][j] = (EPI == 2 && m < M && n < N) ? C[(long)m * ldc + n] : 0.0f;
    }
  for (int k0 = 0; k0 < K; k0 += GK) {
    for (int idx = threadIdx.x; idx < GT * GK; idx += 256) {
      int k, mn;
      if (A_MN) { mn = idx % GT; k = idx / GT; } else { k = idx % GK; mn = idx / GK; }
      const int gm = m0 + mn, gk = k0 + k;
      sa[k][mn] = (gm < M && gk < K) ? (A_MN ? A[(long)gk * lda + gm] : A[(long)gm * lda + gk]) : 0.0f;
      if (B_MN) { mn = idx % GT; k = idx / GT; } else { k = idx % GK; mn = idx / GK; }
      const int gn = n0 + mn, gk2 = k0 + k;
      sb[k][mn] = (gn < N && gk2 < K) ? (B_MN ? B[(long)gk2 * ldb + gn] : B[(long)gn * ldb + gk2]) : 0.0f;
    }
    __syncthreads();
    const int kend = min(GK, K - k0);
    for (int k = 0; k < kend; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = sa[k][ty * 4 + i]; b[i] = sb[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N) {
        float v = acc[i][j];
        if (EPI == 3) v = __fadd_rn(v, R[(long)m * ldr + n]);
        C[(long)m * ldc + n] = v;
      }
    }
}

// ------------------------------------------------------------------------- attention
__device__ __forceinline__ bool masked(int qi, int kj, int window) { return kj > qi || (window > 0 && kj <= qi - window); }

// one warp per (b, h, query)
__global__ void __launch_bounds__(128)
attn_f32_fwd_kernel(const float* __restrict__ qk, long ldqk, const float* __restrict__ qkv, long ldqkv,
                    float* __restrict__ O, long ldo, float* __restrict__ lse, int B, int T, int H, int Hkv, int D,
                    int window, float c_log2) {
  __shared__ float sq[4][128], sp[4][128];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long wid = (long)blockIdx.x * 4 + w;
  if (wid >= (long)B * H * T) return;
  const int qi = (int)(wid % T);
  const int h = (int)((wid / T) % H), b = (int)(wid / ((long)T * H));
  const int g = h / (H / Hkv);
  const long qrow = (long)b * T + qi;
  for (int d = lane; d < D; d += 32) sq[w][d] = qk[qrow * ldqk + (long)h * D + d];
  __syncwarp();
  float o[4] = {0.f, 0.f, 0.f, 0.f};
  const int q0 = (qi / 128) * 128, jmax = qi / 128;
  const int jmin = (window > 0 && q0 - window + 1 > 0) ? (q0 - window + 1) / 128 : 0;
  float m_run = -INFINITY, l_part = 0.f;  // lanes 0..3 each own one 32-key quarter
  for (int j = jmin; j <= jmax; ++j) {
    float mx = -INFINITY;
    float s[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = lane + 32 * u, kj = j * 128 + e;
      if (masked(qi, kj, window) || kj >= T) { s[u] = -INFINITY; continue; }
      const float* kr = qk + ((long)b * T + kj) * ldqk + (long)(H + g) * D;
      float acc = 0.0f;
      for (int d = 0; d < D; ++d) acc = __fmaf_rn(sq[w][d], kr[d], acc);
      s[u] = acc;
      mx = fmaxf(mx, acc);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const float m_new = fmaxf(m_run, __fmul_rn(mx, c_log2));
    const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;
    const float alpha = det_exp2_attn(__fadd_rn(m_run, -m_safe));
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      sp[w][lane + 32 * u] = (s[u] == -INFINITY) ? 0.0f : det_exp2_attn(__fmaf_rn(s[u], c_log2, -m_safe));
    }
    __syncwarp();
    if (lane < 4) {  // the four quarter-row sums: even and odd keys are ascending chains, then added
      float le = 0.0f, lo = 0.0f;
      for (int e = lane * 32; e < lane * 32 + 32; e += 2) { le = __fadd_rn(le, sp[w][e]); lo = __fadd_rn(lo, sp[w][e + 1]); }
      l_part = __fmaf_rn(l_part, alpha, __fadd_rn(le, lo));
    }
    float pv[4] = {0.f, 0.f, 0.f, 0.f};
    for (int e = 0; e < 128; ++e) {
      const int kj = j * 128 + e;
      if (kj >= T) break;
      const float p = sp[w][e];
      if (p == 0.0f) continue;
      const float* vr = qkv + ((long)b * T + kj) * ldqkv + (long)(H + Hkv + g) * D;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int d = lane + 32 * u;
        if (d < D) pv[u] = __fmaf_rn(p, vr[d], pv[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) o[u] = __fmaf_rn(o[u], alpha, pv[u]);
    m_run = m_new;
    __syncwarp();
  }
  const float l0 = __shfl_sync(0xffffffffu, l_part, 0), l1 = __shfl_sync(0xffffffffu, l_part, 1);
  const float l2 = __shfl_sync(0xffffffffu, l_part, 2), l3 = __shfl_sync(0xffffffffu, l_part, 3);
  const float l_tot = __fadd_rn(__fadd_rn(__fadd_rn(l0, l1), l2), l3);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int d = lane + 32 * u;
    if (d < D) O[qrow * ldo + (long)h * D + d] = __fdiv_rn(o[u], l_tot);
  }
  if (lane == 0) lse[((long)b * H + h) * T + qi] = __fmaf_rn(det_logf(l_tot), 1.44269504088896341f, m_run);
}

__global__ void attn_f32_delta_kernel(const float* __restrict__ dO, long lddo, const float* __restrict__ O, long ldo,
                                      float* __restrict__ delta, int B, int T, int H, int D) {
  const long wid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long)B * T * H) return;
  const long row = wid / H;
  const int h = (int)(wid - row * H);
  float acc = 0.0f;
  for (int e = 0; e < 4; ++e) {
    const int d = lane * 4 + e;
    if (d < D) acc = __fmaf_rn(dO[row * lddo + (long)h * D + d], O[row * ldo + (long)h * D + d], acc);
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
  if (lane == 0) {
    const long bb = row / T, t = row - bb * T;
    delta[(bb * H + h) * T + t] = acc;
  }
}

// p and ds of the pair (qi, kj); lane-parallel over pairs, each pair's two chains sequential in d
__device__ __forceinline__ void pair_p_ds(const float* __restrict__ qk, long ldqk, const float* __restrict__ qkv,
                                          long ldqkv, const float* __restrict__ dO, long lddo, const float* lse,
                                          const float* delta, int b, int h, int g, int qi, int kj, int T, int H, int Hkv,
                                          int D, float c_log2, float scale, float* p_out, float* ds_out) {
  const long qrow = (long)b * T + qi, krow = (long)b * T + kj;
  const float* q = qk + qrow * ldqk + (long)h * D;
  const float* k = qk + krow * ldqk + (long)(H + g) * D;
  const float* dor = dO + qrow * lddo + (long)h * D;
  const float* v = qkv + krow * ldqkv + (long)(H + Hkv + g) * D;
  float s = 0.0f, dp = 0.0f;
  for (int d = 0; d < D; ++d) s = __fmaf_rn(q[d], k[d], s);
  for (int d = 0; d < D; ++d) dp = __fmaf_rn(dor[d], v[d], dp);
  const float l2 = lse[((long)b * H + h) * T + qi], dl = delta[((long)b * H + h) * T + qi];
  const float p = det_exp2_attn(__fmaf_rn(s, c_log2, -l2));
  *p_out = p;
  *ds_out = __fmul_rn(__fmul_rn(p, __fadd_rn(dp, -dl)), scale);
}

// one warp per (b, kv head, key)
__global__ void __launch_bounds__(128)
attn_f32_bwd_kv_kernel(const float* __restrict__ qk, long ldqk, const float* __restrict__ qkv, long ldqkv,
                       const float* __restrict__ dO, long lddo, const float* __restrict__ lse,
                       const float* __restrict__ delta, float* __restrict__ dqk, long lddqk, float* __restrict__ dqkv,
                       long lddqkv, int B, int T, int H, int Hkv, int D, int window, float c_log2, float scale) {
  __shared__ float sp[4][32], sds[4][32];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long wid = (long)blockIdx.x * 4 + w;
  if (wid >= (long)B * Hkv * T) return;
  const int kj = (int)(wid % T);
  const int g = (int)((wid / T) % Hkv), b = (int)(wid / ((long)T * Hkv));
  const int G = H / Hkv;
  const int kb = kj / 128;
  int qlast = (T + 127) / 128 - 1;
  if (window > 0) qlast = min(qlast, (kb * 128 + 127 + window - 1) / 128);
  const int qend = min((qlast + 1) * 128, T);
  float dk[4] = {0.f, 0.f, 0.f, 0.f}, dv[4] = {0.f, 0.f, 0.f, 0.f};
  for (int hh = 0; hh < G; ++hh) {
    const int h = g * G + hh;
    for (int qb = kb * 128; qb < qend; qb += 32) {
      const int qi = qb + lane;
      float p = 0.0f, ds = 0.0f;
      if (qi < qend && !masked(qi, kj, window))
        pair_p_ds(qk, ldqk, qkv, ldqkv, dO, lddo, lse, delta, b, h, g, qi, kj, T, H, Hkv, D, c_log2, scale, &p, &ds);
      sp[w][lane] = p;
      sds[w][lane] = ds;
      __syncwarp();
      for (int e = 0; e < 32 && qb + e < qend; ++e) {
        if (masked(qb + e, kj, window)) continue;
        const long qrow = (long)b * T + qb + e;
        const float pe = sp[w][e], dse = sds[w][e];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int d = lane + 32 * u;
          if (d < D) {
            dv[u] = __fmaf_rn(pe, dO[qrow * lddo + (long)h * D + d], dv[u]);
            dk[u] = __fmaf_rn(dse, qk[qrow * ldqk + (long)h * D + d], dk[u]);
          }
        }
      }
      __syncwarp();
    }
  }
  const long krow = (long)b * T + kj;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int d = lane + 32 * u;
    if (d < D) {
      dqk[krow * lddqk + (long)(H + g) * D + d] = dk[u];
      dqkv[krow * lddqkv + (long)(H + Hkv + g) * D + d] = dv[u];
    }
  }
}

// one warp per (b, h, query)
__global__ void __launch_bounds__(128)
attn_f32_bwd_q_kernel(const float* __restrict__ qk, long ldqk, const float* __restrict__ qkv, long ldqkv,
                      const float* __restrict__ dO, long lddo, const float* __restrict__ lse,
                      const float* __restrict__ delta, float* __restrict__ dqk, long lddqk, int B, int T, int H, int Hkv,
                      int D, int window, float c_log2, float scale) {
  __shared__ float sds[4][32];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long wid = (long)blockIdx.x * 4 + w;
  if (wid >= (long)B * H * T) return;
  const int qi = (int)(wid % T);
  const int h = (int)((wid / T) % H), b = (int)(wid / ((long)T * H));
  const int g = h / (H / Hkv);
  const int q0 = (qi / 128) * 128;
  const int jmin = (window > 0 && q0 - window + 1 > 0) ? (q0 - window + 1) / 128 : 0;
  float dq[4] = {0.f, 0.f, 0.f, 0.f};
  for (int kb = jmin * 128; kb <= qi; kb += 32) {
    const int kj = kb + lane;
    float p = 0.0f, ds = 0.0f;
    if (kj <= qi && !masked(qi, kj, window))
      pair_p_ds(qk, ldqk, qkv, ldqkv, dO, lddo, lse, delta, b, h, g, qi, kj, T, H, Hkv, D, c_log2, scale, &p, &ds);
    sds[w][lane] = ds;
    __syncwarp();
    for (int e = 0; e < 32 && kb + e <= qi; ++e) {
      if (masked(qi, kb + e, window)) continue;
      const long krow = (long)b * T + kb + e;
      const float dse = sds[w][e];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int d = lane + 32 * u;
        if (d < D) dq[u] = __fmaf_rn(dse, qk[krow * ldqk + (long)(H + g) * D + d], dq[u]);
      }
    }
    __syncwarp();
  }
  const long qrow = (long)b * T + qi;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int d = lane + 32 * u;
    if (d < D) dqk[qrow * lddqk + (long)h * D + d] = dq[u];
  }
}

}  // namespace

extern "C" int otb_gemm_f32(const float* A, const float* B, float* C, const float* R, int M, int N, int K, long lda,
                            long ldb, long ldc, long ldr, int a_mn, int b_mn, int epi, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  dim3 grid((N + GT - 1) / GT, (M + GT - 1) / GT);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define GF(AM, BM, E) gemm_f32_kernel<AM, BM, E><<<grid, 256, 0, s>>>(A, B, C, R, M, N, K, lda, ldb, ldc, ldr)
#define GE(AM, BM)                                      \
  switch (epi) {                                         \
    case 0: case 1: GF(AM, BM, 0); break;                \
    case 2: GF(AM, BM, 2); break;                        \
    case 3: GF(AM, BM, 3); break;                        \
    default: return -3;                                  \
  }
  if (!a_mn && !b_mn) { GE(false, false) } else if (!a_mn && b_mn) { GE(false, true) }
  else if (a_mn && b_mn) { GE(true, true) } else { GE(true, false) }
#undef GE
#undef GF
  return (int)cudaGetLastError();
}

extern "C" int otb_attn_f32_fwd(const float* qk, long ldqk, const float* qkv, long ldqkv, float* O, long ldo, float* lse,
                                int B, int T, int H, int Hkv, int D, int window, float scale, void* stream) {
  if (D > 128 || H % Hkv) return -2;
  const float c_log2 = (float)((double)scale * 1.4426950408889634);
  const long warps = (long)B * H * T;
  attn_f32_fwd_kernel<<<(unsigned)((warps + 3) / 4), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      qk, ldqk, qkv, ldqkv, O, ldo, lse, B, T, H, Hkv, D, window, c_log2);
  return (int)cudaGetLastError();
}
extern "C" int otb_attn_f32_bwd(const float* qk, long ldqk, const float* qkv, long ldqkv, const float* O, long ldo,
                                const float* dO, long lddo, const float* lse, float* delta, float* dqk, long lddqk,
                                float* dqkv, long lddqkv, int B, int T, int H, int Hkv, int D, int window, float scale,
                                void* stream) {
  if (D > 128 || H % Hkv) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const float c_log2 = (float)((double)scale * 1.4426950408889634);
  const long w1 = (long)B * T * H;
  attn_f32_delta_kernel<<<(unsigned)((w1 + 7) / 8), 256, 0, s>>>(dO, lddo, O, ldo, delta, B, T, H, D);
  const long wkv = (long)B * Hkv * T;
  attn_f32_bwd_kv_kernel<<<(unsigned)((wkv + 3) / 4), 128, 0, s>>>(qk, ldqk, qkv, ldqkv, dO, lddo, lse, delta, dqk, lddqk,
                                                                   dqkv, lddqkv, B, T, H, Hkv, D, window, c_log2, scale);
  attn_f32_bwd_q_kernel<<<(unsigned)((w1 + 3) / 4), 128, 0, s>>>(qk, ldqk, qkv, ldqkv, dO, lddo, lse, delta, dqk, lddqk, B,
                                                                 T, H, Hkv, D, window, c_log2, scale);
  return (int)cudaGetLastError();
}
