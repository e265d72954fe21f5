// Memory-bound kernels of the transformer block for sm_100a: RMSNorm fwd/bwd, gain-free QK-norm
// fused with RoPE fwd/bwd, SwiGLU fwd/bwd, fused cross-entropy + z-loss fwd+bwd, embedding
// gather and its deterministic backward, canonical sums.
//
// Every reduction follows csrc/common/det_reduce.h and every transcendental comes from
// csrc/common/det_math.h, so csrc/cpu/ref_ops.cpp returns the same bits.
// Activations are templated on T in {bf16, float}; arithmetic is always fp32 with one
// rounding to T at the store.
//
// Reference roles: repop rms_norm (src/pretrain/model/modules/norm_repop.py:19-22), silu
// (ffn_repop.py:52-54), apply_rope (rope.py:103-125), fused_ce_z_loss (model/fused_loss.py:40-104),
// deterministic embedding backward (embedding_repop.py:3-10).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "det_math.h"
#include "ew_common.cuh"
#include "tc05.cuh"

namespace {


// ------------------------------------------------------------------ RMSNorm
// one warp per row; lane_tree with VW = 8
template <typename T>
__global__ void rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                   float* __restrict__ rstd_out, long rows, int D, float inv_d, float eps) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + row * D;
  float acc = 0.0f;
  for (int c = lane * 8; c < D; c += 256) {
    float f[8];
    Vec8<T>::load(xr + c, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc = __fmaf_rn(f[e], f[e], acc);
  }
  const float ss = warp_butterfly(acc);
  const float rstd = det_rsqrtf(__fadd_rn(__fmul_rn(ss, inv_d), eps));
  if (lane == 0) rstd_out[row] = rstd;
  T* yr = y + row * D;
  for (int c = lane * 8; c < D; c += 256) {
    float f[8], o[8];
    Vec8<T>::load(xr + c, f);
    if (w) {
      float g[8];
      Vec8<T>::load(w + c, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = __fmul_rn(__fmul_rn(f[e], rstd), g[e]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = __fmul_rn(f[e], rstd);
    }
    Vec8<T>::store(yr + c, o);
  }
}

// One CTA of SLAB warps per slab of SLAB rows, one warp per row: the row stays in registers (as loaded, 16-byte
// vectors) between the dot product and the dx pass, so x and dy are read once. dgamma partial [slab][D] is the
// ascending-row fold inside the slab: every warp leaves its row's dy * xhat products in shared memory and, after one
// barrier, the CTA adds the SLAB rows of each column in row order (the same chain a single warp would have run).
// MAXC = max number of 8-wide column chunks per lane (D <= 256 * MAXC).
constexpr int NORM_SLAB = 8;
template <typename T, int MAXC>
__global__ void __launch_bounds__(NORM_SLAB * 32) rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                                                    const float* __restrict__ rstd_in, T* __restrict__ dx,
                                                                    float* __restrict__ dgamma_partial, long rows, int D, float inv_d) {
  extern __shared__ float prod[];  // [NORM_SLAB][MAXC * 256] when dgamma is wanted
  const long slab = blockIdx.x;
  const int lane = threadIdx.x & 31, wrow = threadIdx.x >> 5;
  const long row = slab * NORM_SLAB + wrow;
  const bool live = row < rows;
  if (live) {
    const float rstd = rstd_in[row];
    const T* xr = x + row * D;
    const T* dyr = dy + row * D;
    Raw8<T> xraw[MAXC], draw[MAXC];
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
      const int c = lane * 8 + j * 256;
      if (c < D) {
        xraw[j].load(xr + c);
        draw[j].load(dyr + c);
      }
    }
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
      const int c = lane * 8 + j * 256;
      if (c < D) {
        float xf[8], df[8], g[8];
        xraw[j].unpack(xf);
        draw[j].unpack(df);
        if (w) Vec8<T>::load(w + c, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = __fmul_rn(xf[e], rstd);
          const float gy = w ? __fmul_rn(df[e], g[e]) : df[e];
          acc = __fmaf_rn(gy, xh, acc);
          if (dgamma_partial) prod[wrow * (MAXC * 256) + j * 256 + e * 32 + lane] = __fmul_rn(df[e], xh);  // lanes side by side: no bank conflict
        }
      }
    }
    const float cs = __fmul_rn(warp_butterfly(acc), inv_d);
    T* dxr = dx + row * D;
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
      const int c = lane * 8 + j * 256;
      if (c < D) {
        float xf[8], df[8], g[8], o[8];
        xraw[j].unpack(xf);
        draw[j].unpack(df);
        if (w) Vec8<T>::load(w + c, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = __fmul_rn(xf[e], rstd);
          const float gy = w ? __fmul_rn(df[e], g[e]) : df[e];
          o[e] = __fmul_rn(rstd, __fmaf_rn(-xh, cs, gy));
        }
        Vec8<T>::store(dxr + c, o);
      }
    }
  }
  if (dgamma_partial) {
    __syncthreads();
    const int nrow = (int)((rows - slab * NORM_SLAB < NORM_SLAB) ? rows - slab * NORM_SLAB : NORM_SLAB);
    float* out = dgamma_partial + slab * D;
    for (int j = wrow; j < MAXC; j += NORM_SLAB) {  // warp j folds column chunk j; a lane owns the same 8 columns as above
      const int c = lane * 8 + j * 256;
      if (c < D) {
        float a[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float t = 0.0f;
          for (int r = 0; r < nrow; ++r) t = __fadd_rn(t, prod[r * (MAXC * 256) + j * 256 + e * 32 + lane]);
          a[e] = t;
        }
        *reinterpret_cast<float4*>(out + c) = make_float4(a[0], a[1], a[2], a[3]);
        *reinterpret_cast<float4*>(out + c + 4) = make_float4(a[4], a[5], a[6], a[7]);
      }
    }
  }
}

// pair_tree over the leading dimension of v[n][D], in place; result in row 0.
// The tree "for s = 1, 2, 4..: v[i] += v[i+s] for i multiple of 2s, i+s < n" only ever pairs rows inside a
// 2s-aligned group, so groups of 64 rows are reduced independently in shared memory (levels s = 1..32) and the
// same kernel is then applied to the 64-strided group roots (levels 64..2048), and so on: identical association,
// log-depth instead of a serial chain. Logical row j lives at v[j * row_stride * D]. A missing partner leaves the
// value untouched (never "+ 0.0", which would turn -0.0 into +0.0).
__global__ void __launch_bounds__(256) pair_tree_cols_stage_kernel(float* __restrict__ v, long n, long row_stride, int D) {
  __shared__ float sm[64][33];
  const int c = threadIdx.x & 31, r = threadIdx.x >> 5;  // 32 columns x 8 row-threads
  const int col = blockIdx.x * 32 + c;
  const long g0 = (long)blockIdx.y * 64;                // first logical row of this group
  const long rows_here = min((long)64, n - g0);
  if (col < D)
    for (int rr = r; rr < rows_here; rr += 8) sm[rr][c] = v[(g0 + rr) * row_stride * D + col];
  __syncthreads();
  for (int s = 1; s < 64; s *= 2) {
    for (int i = r * 2 * s; i + s < rows_here; i += 16 * s) sm[i][c] = __fadd_rn(sm[i][c], sm[i + s][c]);
    __syncthreads();
  }
  if (col < D && r == 0) v[g0 * row_stride * D + col] = sm[0][c];
}

inline void pair_tree_cols_launch(float* v, long n, int D, cudaStream_t s) {
  long stride = 1;
  while (n > 1) {
    const long groups = (n + 63) / 64;
    dim3 grid((D + 31) / 32, (unsigned)groups);
    pair_tree_cols_stage_kernel<<<grid, 256, 0, s>>>(v, n, stride, D);
    n = groups;
    stride *= 64;
  }
}

// --------------------------------------------------- gain-free QK-norm + RoPE
// One warp per (token, head) over the first `heads` heads of a [rows, ld_in] buffer with head
// width D (<= 128, multiple of 4): lane l holds elements 4l..4l+3 (two rotation pairs).
// out[row, head*D + i]; rstd[row*heads + head]. lane_tree with VW = 4.
template <typename T>
__global__ void qknorm_rope_fwd_kernel(const T* __restrict__ in, long ld_in, T* __restrict__ out, long ld_out,
                                       float* __restrict__ rstd_out, const float* __restrict__ cosb,
                                       const float* __restrict__ sinb, long rows, int heads, int D, int seq_len,
                                       int do_norm, float inv_d, float eps) {
  const long wid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= rows * heads) return;
  const long row = wid / heads;
  const int head = (int)(wid - row * heads);
  const int pos = (int)(row % seq_len);
  const bool active = lane * 4 < D;
  float f[4] = {0.f, 0.f, 0.f, 0.f};
  if (active) {
    const T* p = in + row * ld_in + (long)head * D + lane * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) f[e] = to_f<T>(p[e]);
  }
  float rstd = 1.0f;
  if (do_norm) {
    float acc = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc = __fmaf_rn(f[e], f[e], acc);
    const float ss = warp_butterfly(acc);
    rstd = det_rsqrtf(__fadd_rn(__fmul_rn(ss, inv_d), eps));
    if (lane == 0) rstd_out[wid] = rstd;
#pragma unroll
    for (int e = 0; e < 4; ++e) f[e] = __fmul_rn(f[e], rstd);
  }
  if (active) {
    const int half = D >> 1;
    T* o = out + row * ld_out + (long)head * D + lane * 4;
#pragma unroll
    for (int pr = 0; pr < 2; ++pr) {
      const float c = cosb[(long)pos * half + lane * 2 + pr];
      const float s = sinb[(long)pos * half + lane * 2 + pr];
      const float xe = f[2 * pr], xo = f[2 * pr + 1];
      o[2 * pr] = from_f<T>(__fmaf_rn(xe, c, -__fmul_rn(xo, s)));
      o[2 * pr + 1] = from_f<T>(__fmaf_rn(xe, s, __fmul_rn(xo, c)));
    }
  }
}

template <typename T>
__global__ void qknorm_rope_bwd_kernel(const T* __restrict__ dout, long ld_dout, const T* __restrict__ in, long ld_in,
                                       const float* __restrict__ rstd_in, T* __restrict__ din, long ld_din,
                                       const float* __restrict__ cosb, const float* __restrict__ sinb, long rows,
                                       int heads, int D, int seq_len, int do_norm, float inv_d) {
  const long wid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= rows * heads) return;
  const long row = wid / heads;
  const int head = (int)(wid - row * heads);
  const int pos = (int)(row % seq_len);
  const bool active = lane * 4 < D;
  float g[4] = {0.f, 0.f, 0.f, 0.f};
  if (active) {
    const int half = D >> 1;
    const T* p = dout + row * ld_dout + (long)head * D + lane * 4;
#pragma unroll
    for (int pr = 0; pr < 2; ++pr) {
      const float c = cosb[(long)pos * half + lane * 2 + pr];
      const float s = sinb[(long)pos * half + lane * 2 + pr];
      const float de = to_f<T>(p[2 * pr]), dd = to_f<T>(p[2 * pr + 1]);
      g[2 * pr] = __fmaf_rn(de, c, __fmul_rn(dd, s));
      g[2 * pr + 1] = __fmaf_rn(dd, c, -__fmul_rn(de, s));
    }
  }
  if (do_norm) {
    const float rstd = rstd_in[wid];
    float xh[4] = {0.f, 0.f, 0.f, 0.f};
    if (active) {
      const T* p = in + row * ld_in + (long)head * D + lane * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e) xh[e] = __fmul_rn(to_f<T>(p[e]), rstd);
    }
    float acc = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc = __fmaf_rn(g[e], xh[e], acc);
    const float cs = __fmul_rn(warp_butterfly(acc), inv_d);
#pragma unroll
    for (int e = 0; e < 4; ++e) g[e] = __fmul_rn(rstd, __fmaf_rn(-xh[e], cs, g[e]));
  }
  if (active) {
    T* o = din + row * ld_din + (long)head * D + lane * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = from_f<T>(g[e]);
  }
}

// ------------------------------------------------------------------- SwiGLU
// gate_up [rows, 2F] (gate = cols [0,F), up = cols [F,2F)) -> h [rows, F] = silu(gate) * up
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ h, long rows, int F) {
  const long idx = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (idx >= rows * F) return;
  const long row = idx / F;
  const int col = (int)(idx - row * F);
  float g[8], u[8], o[8];
  Vec8<T>::load(gu + row * 2 * F + col, g);
  Vec8<T>::load(gu + row * 2 * F + F + col, u);
#pragma unroll
  for (int e = 0; e < 8; e += 2) {
    const tc05::f2 g2 = tc05::pack2(g[e], g[e + 1]);
    tc05::unpack2(tc05::mul2(tc05::mul2(g2, tc05::sigmoid_fast2(g2)), tc05::pack2(u[e], u[e + 1])), o[e], o[e + 1]);
  }
  Vec8<T>::store(h + idx, o);
}
// d_gate_up [rows, 2F] from dh [rows, F]
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ gu, const T* __restrict__ dh, T* __restrict__ dgu, long rows,
                                  int F) {
  const long idx = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (idx >= rows * F) return;
  const long row = idx / F;
  const int col = (int)(idx - row * F);
  float g[8], u[8], d[8], og[8], ou[8];
  Vec8<T>::load(gu + row * 2 * F + col, g);
  Vec8<T>::load(gu + row * 2 * F + F + col, u);
  Vec8<T>::load(dh + idx, d);
#pragma unroll
  for (int e = 0; e < 8; e += 2) {
    using namespace tc05;
    const f2 g2 = pack2(g[e], g[e + 1]), u2 = pack2(u[e], u[e + 1]), d2 = pack2(d[e], d[e + 1]);
    const f2 sg = sigmoid_fast2(g2);
    const f2 silu = mul2(g2, sg);
    // d silu / dg = sg * (1 + g (1 - sg))
    const f2 one = pack2(1.0f, 1.0f);
    const f2 dsilu = mul2(sg, fma2(g2, add2(one, mul2(sg, pack2(-1.0f, -1.0f))), one));
    unpack2(mul2(mul2(d2, u2), dsilu), og[e], og[e + 1]);
    unpack2(mul2(d2, silu), ou[e], ou[e + 1]);
  }
  Vec8<T>::store(dgu + row * 2 * F + col, og);
  Vec8<T>::store(dgu + row * 2 * F + F + col, ou);
}

// --------------------------------------------------------- fused CE + z-loss
// One CTA of 512 threads per row of logits [rows, V] (V % 8 == 0). With m = max of the row and L = log2(e):
//   e_i = exp2(fma(x_i, L, -(m * L)))        (det_exp2_acc, evaluated two at a time with packed fp32 arithmetic)
//   s   = sum e_i: the 8-element group g = i / 8 belongs to thread g % 512; a thread keeps two ascending chains, the
//         even and the odd elements of its groups, adds them, and the 512 thread sums go through block_tree_sum
//   lse = log(s) + m,  ce[row] = lse - x[label],  lse_out[row] = lse
// and the row is overwritten with d loss / d logits = e_i * k - onehot * scale, k = ((1 + 2 z lse) / s) * scale
// (scale = 1 / (tokens * accum), host reciprocal; the label's element is fma(e, k, -scale)).
// Rows with label < 0 are ignored: zero loss, zero gradient.
constexpr int CE_THREADS = 512;
template <typename T>
__global__ void __launch_bounds__(CE_THREADS) ce_zloss_kernel(T* __restrict__ logits, const long* __restrict__ labels,
                                                              float* __restrict__ ce_out, float* __restrict__ lse_out,
                                                              long rows, int V, float two_z, float scale, int write_grad) {
  using namespace tc05;
  __shared__ float sh[32];
  constexpr int SWEEP = CE_THREADS * 8;
  const long row = blockIdx.x;
  T* xr = logits + row * V;
  const long label = labels[row];
  if (label < 0) {
    if (threadIdx.x == 0) { ce_out[row] = 0.0f; lse_out[row] = 0.0f; }
    if (write_grad) {
      float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int c = threadIdx.x * 8; c < V; c += SWEEP) Vec8<T>::store(xr + c, z);
    }
    return;
  }
  const float x_label = to_f<T>(xr[label]);
  float mx = -INFINITY;
  for (int c = threadIdx.x * 8; c < V; c += SWEEP) {
    float f[8];
    Vec8<T>::load(xr + c, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) mx = fmaxf(mx, f[e]);
  }
  mx = block_max(mx, sh);
  const float LOG2E = 1.44269504088896341f;
  const f2 l2 = pack2(LOG2E, LOG2E);
  const float nm = -__fmul_rn(mx, LOG2E);
  const f2 nm2 = pack2(nm, nm);
  f2 acc2 = pack2(0.0f, 0.0f);
  for (int c = threadIdx.x * 8; c < V; c += SWEEP) {
    float f[8];
    Vec8<T>::load(xr + c, f);
#pragma unroll
    for (int e = 0; e < 8; e += 2) acc2 = add2(acc2, exp2_acc2(fma2(pack2(f[e], f[e + 1]), l2, nm2)));
  }
  float a0, a1;
  unpack2(acc2, a0, a1);
  const float s = block_tree_sum(__fadd_rn(a0, a1), sh);
  const float lse = __fadd_rn(det_logf(s), mx);
  if (threadIdx.x == 0) {
    ce_out[row] = __fadd_rn(lse, -x_label);
    lse_out[row] = lse;
  }
  if (!write_grad) return;
  __syncthreads();  // every thread has its copy of the label logit before anyone overwrites the row
  const float k = __fmul_rn(__fdiv_rn(__fmaf_rn(two_z, lse, 1.0f), s), scale);
  const f2 k2 = pack2(k, k);
  for (int c = threadIdx.x * 8; c < V; c += SWEEP) {
    float f[8], o[8];
    Vec8<T>::load(xr + c, f);
#pragma unroll
    for (int e = 0; e < 8; e += 2) unpack2(mul2(exp2_acc2(fma2(pack2(f[e], f[e + 1]), l2, nm2)), k2), o[e], o[e + 1]);
    Vec8<T>::store(xr + c, o);
    if (label >= c && label < c + 8)  // the owner of the label's group rewrites that one element
      xr[label] = from_f<T>(__fmaf_rn(det_exp2_acc(__fmaf_rn(x_label, LOG2E, nm)), k, -scale));
  }
}

// sum (or sum of squares) of n floats: element i -> thread i % 1024, ascending fold, block_tree_sum.
// mode 0: sum x, 1: sum x*x (fma chain). out[0] = result * post_scale.
__global__ void __launch_bounds__(1024) det_sum_kernel(const float* __restrict__ x, long n, int mode, float post_scale,
                                                        float* __restrict__ out) {
  __shared__ float sh[32];
  float acc = 0.0f;
  for (long i = threadIdx.x; i < n; i += 1024) {
    const float v = x[i];
    acc = mode ? __fmaf_rn(v, v, acc) : __fadd_rn(acc, v);
  }
  const float s = block_tree_sum(acc, sh);
  if (threadIdx.x == 0) out[0] = __fmul_rn(s, post_scale);
}

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_fwd_kernel(const long* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                     long rows, int D) {
  const long row = blockIdx.x;
  const long id = ids[row];
  const uint4* src = reinterpret_cast<const uint4*>(table + id * D);
  uint4* dst = reinterpret_cast<uint4*>(out + row * D);
  const int nvec = D * (int)sizeof(T) / 16;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = src[i];
}
// sorted_ids: the n token ids in ascending order (stable sort); sorted_tok: the token position of each. One CTA per
// sorted position: the CTA at the HEAD of a run of equal ids owns that id's row, the others exit at once, so the
// launch needs no count of distinct ids (no device-to-host read of a data-dependent size).
// dW[id, :] (+)= sum over the run in ascending token position, fp32.
template <typename T>
__global__ void embedding_bwd_kernel(const T* __restrict__ dy, const long* __restrict__ sorted_ids,
                                     const long* __restrict__ sorted_tok, long n, float* __restrict__ dW, int D,
                                     int accumulate) {
  const long b = blockIdx.x;
  const long id = sorted_ids[b];
  if (b > 0 && sorted_ids[b - 1] == id) return;
  long e = b + 1;
  while (e < n && sorted_ids[e] == id) ++e;
  float* out = dW + id * D;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float acc = 0.0f;
    for (long i = b; i < e; ++i) acc = __fadd_rn(acc, to_f<T>(dy[sorted_tok[i] * D + c]));
    out[c] = accumulate ? __fadd_rn(out[c], acc) : acc;
  }
}

// elementwise helpers ---------------------------------------------------------
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, long n) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_f<TO>(to_f<TI>(in[i]));
}
template <typename T>
__global__ void add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, long n) {
  const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  float x[8], y[8], o[8];
  Vec8<T>::load(a + i, x);
  Vec8<T>::load(b + i, y);
#pragma unroll
  for (int e = 0; e < 8; ++e) o[e] = __fadd_rn(x[e], y[e]);
  Vec8<T>::store(out + i, o);
}

inline unsigned blocks_for(long n, int per) { return (unsigned)((n + per - 1) / per); }

}  // namespace

#define S(stream) reinterpret_cast<cudaStream_t>(stream)
#define DISPATCH_T(is_bf16, ...)                       \
  if (is_bf16) { using T = __nv_bfloat16; __VA_ARGS__ } \
  else { using T = float; __VA_ARGS__ }

// dtype: 1 = bf16, 0 = fp32 for every activation pointer. All row widths multiples of 8.
extern "C" int otb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long rows, int D, float inv_d,
                               float eps, int dtype, void* stream) {
  if (D % 8) return -2;
  DISPATCH_T(dtype, rmsnorm_fwd_kernel<T><<<blocks_for(rows, 8), 256, 0, S(stream)>>>(
                        (const T*)x, (const T*)w, (T*)y, rstd, rows, D, inv_d, eps);)
  return (int)cudaGetLastError();
}
extern "C" int otb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                               float* dgamma_partial, long rows, int D, float inv_d, int dtype, void* stream) {
  if (D % 8 || D > 256 * 16) return -2;
  const long slabs = (rows + NORM_SLAB - 1) / NORM_SLAB;
#define RB(MAXC)                                                                                                          \
  DISPATCH_T(dtype, {                                                                                                     \
    static int attr = cudaFuncSetAttribute(rmsnorm_bwd_kernel<T, MAXC>, cudaFuncAttributeMaxDynamicSharedMemorySize, NORM_SLAB * 256 * MAXC * 4); \
    if (attr) return attr;                                                                                                \
    rmsnorm_bwd_kernel<T, MAXC><<<(unsigned)slabs, NORM_SLAB * 32, dgamma_partial ? NORM_SLAB * 256 * MAXC * 4 : 0, S(stream)>>>((const T*)dy, (const T*)x, (const T*)w, rstd, (T*)dx, \
                                                                                     dgamma_partial, rows, D, inv_d);     \
  })
  if (D <= 256) { RB(1) } else if (D <= 1024) { RB(4) } else if (D <= 2048) { RB(8) } else { RB(16) }
#undef RB
  if (dgamma_partial) pair_tree_cols_launch(dgamma_partial, slabs, D, S(stream));
  return (int)cudaGetLastError();
}
extern "C" long otb_rmsnorm_slabs(long rows) { return (rows + NORM_SLAB - 1) / NORM_SLAB; }

extern "C" int otb_pair_tree_cols(float* v, long n, int D, void* stream) {
  pair_tree_cols_launch(v, n, D, S(stream));
  return (int)cudaGetLastError();
}

extern "C" int otb_qknorm_rope_fwd(const void* in, long ld_in, void* out, long ld_out, float* rstd, const float* cosb,
                                   const float* sinb, long rows, int heads, int D, int seq_len, int do_norm,
                                   float inv_d, float eps, int dtype, void* stream) {
  if (D % 4 || D > 128) return -2;
  DISPATCH_T(dtype, qknorm_rope_fwd_kernel<T><<<blocks_for(rows * heads, 8), 256, 0, S(stream)>>>(
                        (const T*)in, ld_in, (T*)out, ld_out, rstd, cosb, sinb, rows, heads, D, seq_len, do_norm, inv_d,
                        eps);)
  return (int)cudaGetLastError();
}
extern "C" int otb_qknorm_rope_bwd(const void* dout, long ld_dout, const void* in, long ld_in, const float* rstd,
                                   void* din, long ld_din, const float* cosb, const float* sinb, long rows, int heads,
                                   int D, int seq_len, int do_norm, float inv_d, int dtype, void* stream) {
  if (D % 4 || D > 128) return -2;
  DISPATCH_T(dtype, qknorm_rope_bwd_kernel<T><<<blocks_for(rows * heads, 8), 256, 0, S(stream)>>>(
                        (const T*)dout, ld_dout, (const T*)in, ld_in, rstd, (T*)din, ld_din, cosb, sinb, rows, heads, D,
                        seq_len, do_norm, inv_d);)
  return (int)cudaGetLastError();
}
extern "C" int otb_swiglu_fwd(const void* gu, void* h, long rows, int F, int dtype, void* stream) {
  if (F % 8) return -2;
  DISPATCH_T(dtype, swiglu_fwd_kernel<T><<<blocks_for(rows * F / 8, 256), 256, 0, S(stream)>>>((const T*)gu, (T*)h,
                                                                                                 rows, F);)
  return (int)cudaGetLastError();
}
extern "C" int otb_swiglu_bwd(const void* gu, const void* dh, void* dgu, long rows, int F, int dtype, void* stream) {
  if (F % 8) return -2;
  DISPATCH_T(dtype, swiglu_bwd_kernel<T><<<blocks_for(rows * F / 8, 256), 256, 0, S(stream)>>>(
                        (const T*)gu, (const T*)dh, (T*)dgu, rows, F);)
  return (int)cudaGetLastError();
}
extern "C" int otb_ce_zloss(void* logits, const long* labels, float* ce, float* lse, long rows, int V, float two_z,
                            float scale, int write_grad, int dtype, void* stream) {
  if (V % 8) return -2;
  DISPATCH_T(dtype, ce_zloss_kernel<T><<<(unsigned)rows, CE_THREADS, 0, S(stream)>>>((T*)logits, labels, ce, lse, rows, V,
                                                                               two_z, scale, write_grad);)
  return (int)cudaGetLastError();
}
extern "C" int otb_det_sum(const float* x, long n, int mode, float post_scale, float* out, void* stream) {
  det_sum_kernel<<<1, 1024, 0, S(stream)>>>(x, n, mode, post_scale, out);
  return (int)cudaGetLastError();
}
extern "C" int otb_embedding_fwd(const long* ids, const void* table, void* out, long rows, int D, int dtype,
                                 void* stream) {
  if (D % 8) return -2;
  DISPATCH_T(dtype, embedding_fwd_kernel<T><<<(unsigned)rows, 128, 0, S(stream)>>>(ids, (const T*)table, (T*)out, rows,
                                                                                    D);)
  return (int)cudaGetLastError();
}
extern "C" int otb_embedding_bwd(const void* dy, const long* sorted_ids, const long* sorted_tok, long n, float* dW, int D,
                                 int accumulate, int dtype, void* stream) {
  if (n <= 0) return 0;
  DISPATCH_T(dtype, embedding_bwd_kernel<T><<<(unsigned)n, 256, 0, S(stream)>>>((const T*)dy, sorted_ids, sorted_tok, n, dW, D,
                                                                               accumulate);)
  return (int)cudaGetLastError();
}
extern "C" int otb_cast(const void* in, void* out, long n, int in_bf16, int out_bf16, void* stream) {
  const unsigned g = blocks_for(n, 256);
  if (in_bf16 && !out_bf16) cast_kernel<__nv_bfloat16, float><<<g, 256, 0, S(stream)>>>((const __nv_bfloat16*)in, (float*)out, n);
  else if (!in_bf16 && out_bf16) cast_kernel<float, __nv_bfloat16><<<g, 256, 0, S(stream)>>>((const float*)in, (__nv_bfloat16*)out, n);
  else return -2;
  return (int)cudaGetLastError();
}
extern "C" int otb_add(const void* a, const void* b, void* out, long n, int dtype, void* stream) {
  if (n % 8) return -2;
  DISPATCH_T(dtype, add_kernel<T><<<blocks_for(n / 8, 256), 256, 0, S(stream)>>>((const T*)a, (const T*)b, (T*)out, n);)
  return (int)cudaGetLastError();
}
