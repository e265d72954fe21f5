// CPU twins of csrc/cuda/elementwise.cu: same operations in the same order, so the audit replay
// on a plain CPU reproduces the GPU bits. Compiled with -ffp-contract=off; every fused
// multiply-add is an explicit det_fmaf. Parallel loops (OpenMP) only ever split independent
// rows / columns, never a reduction.
#include <math.h>
#include <stdint.h>
#include <string.h>

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

// block_tree_sum of the CUDA side: butterfly inside each group of 32, then over the group sums.
inline float block_tree_host(float* part, int nthreads) {
  const int nw = nthreads / 32;
  float ws[32];
  for (int w = 0; w < nw; ++w) ws[w] = det_butterfly_host(part + w * 32, 32);
  if (nw == 1) return ws[0];
  return det_butterfly_host(ws, nw);
}

template <typename T>
void rmsnorm_fwd(const T* x, const T* w, T* y, float* rstd_out, long rows, int D, float inv_d, float eps) {
#pragma omp parallel for schedule(static)
  for (long row = 0; row < rows; ++row) {
    const T* xr = x + row * D;
    float part[32];
    for (int l = 0; l < 32; ++l) part[l] = 0.0f;
    for (int i = 0; i < D; ++i) {
      const int l = (i / 8) % 32;
      const float f = ld(xr, i);
      part[l] = det_fmaf(f, f, part[l]);
    }
    const float ss = det_butterfly_host(part, 32);
    const float rstd = det_rsqrtf(ss * inv_d + eps);
    rstd_out[row] = rstd;
    for (int i = 0; i < D; ++i) {
      float o = ld(xr, i) * rstd;
      if (w) o = o * ld(w, i);
      st(y + row * D, i, o);
    }
  }
}

constexpr int NORM_SLAB = 8;
template <typename T>
void rmsnorm_bwd(const T* dy, const T* x, const T* w, const float* rstd_in, T* dx, float* dgamma_partial, long rows,
                 int D, float inv_d) {
  const long slabs = (rows + NORM_SLAB - 1) / NORM_SLAB;
#pragma omp parallel for schedule(static)
  for (long slab = 0; slab < slabs; ++slab) {
    std::vector<float> dg(D, 0.0f);
    for (long row = slab * NORM_SLAB; row < (slab + 1) * NORM_SLAB && row < rows; ++row) {
      const float rstd = rstd_in[row];
      const T* xr = x + row * D;
      const T* dyr = dy + row * D;
      float part[32];
      for (int l = 0; l < 32; ++l) part[l] = 0.0f;
      for (int i = 0; i < D; ++i) {
        const int l = (i / 8) % 32;
        const float xh = ld(xr, i) * rstd;
        const float d = ld(dyr, i);
        const float gy = w ? d * ld(w, i) : d;
        part[l] = det_fmaf(gy, xh, part[l]);
        dg[i] = dg[i] + d * xh;
      }
      const float cs = det_butterfly_host(part, 32) * inv_d;
      for (int i = 0; i < D; ++i) {
        const float xh = ld(xr, i) * rstd;
        const float d = ld(dyr, i);
        const float gy = w ? d * ld(w, i) : d;
        st(dx + row * D, i, rstd * det_fmaf(-xh, cs, gy));
      }
    }
    if (dgamma_partial) memcpy(dgamma_partial + slab * D, dg.data(), sizeof(float) * D);
  }
  if (dgamma_partial) {
#pragma omp parallel for schedule(static)
    for (int c = 0; c < D; ++c) det_pair_tree_host(dgamma_partial + c, slabs, D);
  }
}

template <typename T>
void qknorm_rope_fwd(const T* in, long ld_in, T* out, long ld_out, float* rstd_out, const float* cosb, const float* sinb,
                     long rows, int heads, int D, int seq_len, int do_norm, float inv_d, float eps) {
  const int half = D / 2;
#pragma omp parallel for schedule(static)
  for (long wid = 0; wid < rows * heads; ++wid) {
    const long row = wid / heads;
    const int head = (int)(wid - row * heads);
    const int pos = (int)(row % seq_len);
    const T* p = in + row * ld_in + (long)head * D;
    float f[128];
    for (int i = 0; i < D; ++i) f[i] = ld(p, i);
    if (do_norm) {
      float part[32];
      for (int l = 0; l < 32; ++l) part[l] = 0.0f;
      for (int i = 0; i < D; ++i) part[i / 4] = det_fmaf(f[i], f[i], part[i / 4]);
      const float ss = det_butterfly_host(part, 32);
      const float rstd = det_rsqrtf(ss * inv_d + eps);
      rstd_out[wid] = rstd;
      for (int i = 0; i < D; ++i) f[i] = f[i] * rstd;
    }
    T* o = out + row * ld_out + (long)head * D;
    for (int j = 0; j < half; ++j) {
      const float c = cosb[(long)pos * half + j], s = sinb[(long)pos * half + j];
      const float xe = f[2 * j], xo = f[2 * j + 1];
      st(o, 2 * j, det_fmaf(xe, c, -(xo * s)));
      st(o, 2 * j + 1, det_fmaf(xe, s, xo * c));
    }
  }
}

template <typename T>
void qknorm_rope_bwd(const T* dout, long ld_dout, const T* in, long ld_in, const float* rstd_in, T* din, long ld_din,
                     const float* cosb, const float* sinb, long rows, int heads, int D, int seq_len, int do_norm,
                     float inv_d) {
  const int half = D / 2;
#pragma omp parallel for schedule(static)
  for (long wid = 0; wid < rows * heads; ++wid) {
    const long row = wid / heads;
    const int head = (int)(wid - row * heads);
    const int pos = (int)(row % seq_len);
    const T* p = dout + row * ld_dout + (long)head * D;
    float g[128];
    for (int j = 0; j < half; ++j) {
      const float c = cosb[(long)pos * half + j], s = sinb[(long)pos * half + j];
      const float de = ld(p, 2 * j), dd = ld(p, 2 * j + 1);
      g[2 * j] = det_fmaf(de, c, dd * s);
      g[2 * j + 1] = det_fmaf(dd, c, -(de * s));
    }
    if (do_norm) {
      const float rstd = rstd_in[wid];
      const T* xp = in + row * ld_in + (long)head * D;
      float xh[128], part[32];
      for (int l = 0; l < 32; ++l) part[l] = 0.0f;
      for (int i = 0; i < D; ++i) {
        xh[i] = ld(xp, i) * rstd;
        part[i / 4] = det_fmaf(g[i], xh[i], part[i / 4]);
      }
      const float cs = det_butterfly_host(part, 32) * inv_d;
      for (int i = 0; i < D; ++i) g[i] = rstd * det_fmaf(-xh[i], cs, g[i]);
    }
    T* o = din + row * ld_din + (long)head * D;
    for (int i = 0; i < D; ++i) st(o, i, g[i]);
  }
}

template <typename T>
void swiglu_fwd(const T* gu, T* h, long rows, int F) {
#pragma omp parallel for schedule(static)
  for (long row = 0; row < rows; ++row)
    for (int c = 0; c < F; ++c) {
      const float g = ld(gu, row * 2 * F + c), u = ld(gu, row * 2 * F + F + c);
      st(h, row * F + c, (g * det_sigmoid_fastf(g)) * u);
    }
}
template <typename T>
void swiglu_bwd(const T* gu, const T* dh, T* dgu, long rows, int F) {
#pragma omp parallel for schedule(static)
  for (long row = 0; row < rows; ++row)
    for (int c = 0; c < F; ++c) {
      const float g = ld(gu, row * 2 * F + c), u = ld(gu, row * 2 * F + F + c), d = ld(dh, row * F + c);
      const float sg = det_sigmoid_fastf(g);
      const float silu = g * sg;
      const float dsilu = sg * det_fmaf(g, 1.0f + (-sg), 1.0f);
      st(dgu, row * 2 * F + c, (d * u) * dsilu);
      st(dgu, row * 2 * F + F + c, d * silu);
    }
}

template <typename T>
void ce_zloss(T* logits, const long* labels, float* ce_out, float* lse_out, long rows, int V, float two_z, float scale,
              int write_grad) {
#pragma omp parallel for schedule(dynamic, 4)
  for (long row = 0; row < rows; ++row) {
    T* xr = logits + row * V;
    const long label = labels[row];
    if (label < 0) {
      ce_out[row] = 0.0f;
      lse_out[row] = 0.0f;
      if (write_grad) for (int i = 0; i < V; ++i) st(xr, i, 0.0f);
      continue;
    }
    const float x_label = ld(xr, label);
    float mx = -INFINITY;
    for (int i = 0; i < V; ++i) mx = fmaxf(mx, ld(xr, i));
    const float LOG2E = 1.44269504088896341f;
    const float nm = -(mx * LOG2E);
    float even[512], odd[512], part[512];
    for (int t = 0; t < 512; ++t) even[t] = odd[t] = 0.0f;
    for (int i = 0; i < V; ++i) {
      const int t = (i / 8) % 512;
      const float e = det_exp2_acc(det_fmaf(ld(xr, i), LOG2E, nm));
      if (i & 1) odd[t] = odd[t] + e; else even[t] = even[t] + e;
    }
    for (int t = 0; t < 512; ++t) part[t] = even[t] + odd[t];
    const float s = block_tree_host(part, 512);
    const float lse = det_logf(s) + mx;
    ce_out[row] = lse + (-x_label);
    lse_out[row] = lse;
    if (!write_grad) continue;
    const float k = (det_fmaf(two_z, lse, 1.0f) / s) * scale;
    for (int i = 0; i < V; ++i) {
      if (i == label) continue;
      st(xr, i, det_exp2_acc(det_fmaf(ld(xr, i), LOG2E, nm)) * k);
    }
    st(xr, label, det_fmaf(det_exp2_acc(det_fmaf(x_label, LOG2E, nm)), k, -scale));
  }
}

}  // namespace

#define DISPATCH_T(is_bf16, ...)               \
  if (is_bf16) { using T = BF16; __VA_ARGS__ }  \
  else { using T = float; __VA_ARGS__ }

extern "C" {

int otb_cpu_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long rows, int D, float inv_d, float eps,
                        int dtype) {
  DISPATCH_T(dtype, rmsnorm_fwd<T>((const T*)x, (const T*)w, (T*)y, rstd, rows, D, inv_d, eps);)
  return 0;
}
int otb_cpu_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dgamma_partial,
                        long rows, int D, float inv_d, int dtype) {
  DISPATCH_T(dtype, rmsnorm_bwd<T>((const T*)dy, (const T*)x, (const T*)w, rstd, (T*)dx, dgamma_partial, rows, D, inv_d);)
  return 0;
}
long otb_cpu_rmsnorm_slabs(long rows) { return (rows + NORM_SLAB - 1) / NORM_SLAB; }
int otb_cpu_pair_tree_cols(float* v, long n, int D) {
#pragma omp parallel for schedule(static)
  for (int c = 0; c < D; ++c) det_pair_tree_host(v + c, n, D);
  return 0;
}
int otb_cpu_qknorm_rope_fwd(const void* in, long ld_in, void* out, long ld_out, float* rstd, const float* cosb,
                            const float* sinb, long rows, int heads, int D, int seq_len, int do_norm, float inv_d,
                            float eps, int dtype) {
  if (D > 128 || D % 4) return -2;
  DISPATCH_T(dtype, qknorm_rope_fwd<T>((const T*)in, ld_in, (T*)out, ld_out, rstd, cosb, sinb, rows, heads, D, seq_len,
                                       do_norm, inv_d, eps);)
  return 0;
}
int otb_cpu_qknorm_rope_bwd(const void* dout, long ld_dout, const void* in, long ld_in, const float* rstd, void* din,
                            long ld_din, const float* cosb, const float* sinb, long rows, int heads, int D, int seq_len,
                            int do_norm, float inv_d, int dtype) {
  if (D > 128 || D % 4) return -2;
  DISPATCH_T(dtype, qknorm_rope_bwd<T>((const T*)dout, ld_dout, (const T*)in, ld_in, rstd, (T*)din, ld_din, cosb, sinb,
                                       rows, heads, D, seq_len, do_norm, inv_d);)
  return 0;
}
int otb_cpu_swiglu_fwd(const void* gu, void* h, long rows, int F, int dtype) {
  DISPATCH_T(dtype, swiglu_fwd<T>((const T*)gu, (T*)h, rows, F);)
  return 0;
}
int otb_cpu_swiglu_bwd(const void* gu, const void* dh, void* dgu, long rows, int F, int dtype) {
  DISPATCH_T(dtype, swiglu_bwd<T>((const T*)gu, (const T*)dh, (T*)dgu, rows, F);)
  return 0;
}
int otb_cpu_ce_zloss(void* logits, const long* labels, float* ce, float* lse, long rows, int V, float two_z, float scale,
                     int write_grad, int dtype) {
  DISPATCH_T(dtype, ce_zloss<T>((T*)logits, labels, ce, lse, rows, V, two_z, scale, write_grad);)
  return 0;
}
int otb_cpu_det_sum(const float* x, long n, int mode, float post_scale, float* out) {
  float part[1024];
  for (int t = 0; t < 1024; ++t) part[t] = 0.0f;
  for (long i = 0; i < n; ++i) {
    const int t = (int)(i % 1024);
    part[t] = mode ? det_fmaf(x[i], x[i], part[t]) : part[t] + x[i];
  }
  out[0] = block_tree_host(part, 1024) * post_scale;
  return 0;
}
int otb_cpu_embedding_fwd(const long* ids, const void* table, void* out, long rows, int D, int dtype) {
  const size_t es = dtype ? 2 : 4;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < rows; ++r)
    memcpy((char*)out + r * D * es, (const char*)table + ids[r] * D * es, D * es);
  return 0;
}
int otb_cpu_embedding_bwd(const void* dy, const long* sorted_ids, const long* sorted_tok, long n, float* dW, int D, int accumulate,
                          int dtype) {
#pragma omp parallel for schedule(dynamic, 64)
  for (long b = 0; b < n; ++b) {
    const long id = sorted_ids[b];
    if (b > 0 && sorted_ids[b - 1] == id) continue;  // not the head of its run
    long e = b + 1;
    while (e < n && sorted_ids[e] == id) ++e;
    float* out = dW + id * D;
    for (int c = 0; c < D; ++c) {
      float acc = 0.0f;
      for (long i = b; i < e; ++i) {
        const long tok = sorted_tok[i];
        acc = acc + (dtype ? det_bf2f(((const uint16_t*)dy)[tok * D + c]) : ((const float*)dy)[tok * D + c]);
      }
      out[c] = accumulate ? out[c] + acc : acc;
    }
  }
  return 0;
}
int otb_cpu_cast(const void* in, void* out, long n, int in_bf16, int out_bf16) {
  if (in_bf16 && !out_bf16) {
    for (long i = 0; i < n; ++i) ((float*)out)[i] = det_bf2f(((const uint16_t*)in)[i]);
  } else if (!in_bf16 && out_bf16) {
    for (long i = 0; i < n; ++i) ((uint16_t*)out)[i] = det_f2bf(((const float*)in)[i]);
  } else {
    return -2;
  }
  return 0;
}
// unit-test hooks for the shared math header
// Elementwise maps with the shared deterministic routines. op: 0 exp, 1 log, 2 sqrt, 3 1/sqrt, 4 sigmoid, 5 sin, 6 cos
// (sin / cos: double-precision evaluation rounded once to binary32, as for the RoPE tables).
int otb_cpu_map(int op, const float* x, float* y, long n) {
  if (op < 0 || op > 6) return -3;
#pragma omp parallel for schedule(static)
  for (long i = 0; i < n; ++i) {
    const float v = x[i];
    float r;
    switch (op) {
      case 0: r = det_expf(v); break;
      case 1: r = det_logf(v); break;
      case 2: r = det_sqrtf(v); break;
      case 3: r = det_rsqrtf(v); break;
      case 4: r = det_sigmoidf(v); break;
      default: {
        double sv, cv;
        det_sincos((double)v, &sv, &cv);
        r = (float)(op == 5 ? sv : cv);
      }
    }
    y[i] = r;
  }
  return 0;
}
// Canonical sums of the rows of a [rows, n] fp32 matrix (mode 1: sums of squares), each times post_scale.
int otb_cpu_row_sums(const float* x, long rows, long n, int mode, float post_scale, float* out) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < rows; ++r) otb_cpu_det_sum(x + r * n, n, mode, post_scale, out + r);
  return 0;
}
float otb_cpu_expf(float x) { return det_expf(x); }
float otb_cpu_logf(float x) { return det_logf(x); }
void otb_cpu_rope_tables(float* cosb, float* sinb, int seq_len, int half, double theta) {
  // inv_freq_j = 1 / theta^(j/half) = 1 / r^j with r = theta^(1/half); everything is built from
  // correctly rounded double operations, no libm transcendental.
  // r = theta^(1/half) by bisection on x^half = theta (x^half may overflow to +inf for large x, which
  // still compares correctly); only multiplications, comparisons and halvings: deterministic everywhere.
  double lo = 1.0, hi = theta > 1.0 ? theta : 1.0;
  for (int it = 0; it < 4000; ++it) {
    const double mid = lo + (hi - lo) * 0.5;
    if (mid <= lo || mid >= hi) break;
    if (det_powi(mid, half) > theta) hi = mid; else lo = mid;
  }
  const double r = lo;
  for (int j = 0; j < half; ++j) {
    const double inv_freq = 1.0 / det_powi(r, j);
    for (int p = 0; p < seq_len; ++p) {
      double s, c;
      det_sincos((double)p * inv_freq, &s, &c);
      cosb[(long)p * half + j] = (float)c;
      sinb[(long)p * half + j] = (float)s;
    }
  }
}
}  // extern "C"
