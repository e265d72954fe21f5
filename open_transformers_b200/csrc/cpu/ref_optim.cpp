// CPU twins of csrc/cuda/optim_reduce.cu (same chunking, same association, same AdamW operation
// order) plus the deterministic host helpers for hyper-parameters.
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#include "det_math.h"
#include "det_reduce.h"

namespace {
constexpr int CHUNK = 8192;
inline float block_tree_256(float* part) {
  float ws[8];
  for (int w = 0; w < 8; ++w) ws[w] = det_butterfly_host(part + w * 32, 32);
  return det_butterfly_host(ws, 8);
}
inline float chunk_sos(const float* x, int len) {
  float part[256];
  for (int t = 0; t < 256; ++t) part[t] = 0.0f;
  for (int i = 0; i < len; ++i) {
    const int t = (i % 2048) / 8;
    part[t] = det_fmaf(x[i], x[i], part[t]);
  }
  return block_tree_256(part);
}
}  // namespace

extern "C" {

// Thread count of the OpenMP loops of this library (every twin gives the same bytes at any count). Launchers that start
// one process per GPU set OMP_NUM_THREADS=1 for all of them; the start-up work that runs on the host (the Philox
// initialisation of every weight) may ask for more for its own duration. Returns the previous count.
int otb_cpu_set_threads(int n) {
#ifdef _OPENMP
  const int before = omp_get_max_threads();
  if (n > 0) omp_set_num_threads(n);
  return before;
#else
  (void)n;
  return 1;
#endif
}

int otb_cpu_chunk_size() { return CHUNK; }

int otb_cpu_grad_reduce(const void* const* srcs, int S, int R, const long* chunk_start, const int* chunk_len, int nchunks,
                        float* out, float* chunk_sos_out) {
  const float inv_s = 1.0f / (float)S, inv_r = 1.0f / (float)R;
#pragma omp parallel for schedule(static)
  for (int c = 0; c < nchunks; ++c) {
    const long base = chunk_start[c];
    const int len = chunk_len[c];
    float rep[16];
    for (int i = 0; i < len; ++i) {
      for (int r = 0; r < R; ++r) {
        float in = ((const float*)srcs[r * S])[base + i];
        for (int s = 1; s < S; ++s) in = in + ((const float*)srcs[r * S + s])[base + i];
        rep[r] = in * inv_s;
      }
#define OTB_REP_ADD(a, b) rep[a] = rep[a] + rep[b]
      DET_BLOCKS_FOLD(R, OTB_REP_ADD);  // binary blocks over the replicas
#undef OTB_REP_ADD
      out[base + i] = rep[0] * inv_r;
    }
    chunk_sos_out[c] = chunk_sos(out + base, len);
  }
  return 0;
}
// The same fold over the chunks listed in `chunk_ids` (one bucket of the reduction that runs under the backward pass).
int otb_cpu_grad_reduce_ids(const void* const* srcs, int S, int R, const long* chunk_start, const int* chunk_len,
                            const int* chunk_ids, int nids, float* out, float* chunk_sos_out) {
  const float inv_s = 1.0f / (float)S, inv_r = 1.0f / (float)R;
#pragma omp parallel for schedule(static)
  for (int k = 0; k < nids; ++k) {
    const int c = chunk_ids[k];
    const long base = chunk_start[c];
    const int len = chunk_len[c];
    float rep[16];
    for (int i = 0; i < len; ++i) {
      for (int r = 0; r < R; ++r) {
        float in = ((const float*)srcs[r * S])[base + i];
        for (int s = 1; s < S; ++s) in = in + ((const float*)srcs[r * S + s])[base + i];
        rep[r] = in * inv_s;
      }
#define OTB_REP_ADD(a, b) rep[a] = rep[a] + rep[b]
      DET_BLOCKS_FOLD(R, OTB_REP_ADD);  // binary blocks over the replicas
#undef OTB_REP_ADD
      out[base + i] = rep[0] * inv_r;
    }
    chunk_sos_out[c] = chunk_sos(out + base, len);
  }
  return 0;
}
// Sharded state: the reduced gradient goes to `out + chunk_out_start[c]` (a packed buffer of the owned segments).
int otb_cpu_grad_reduce_ex(const void* const* srcs, int S, int R, const long* chunk_start, const int* chunk_len,
                           const int* chunk_ids, int nids, const long* chunk_out_start, float* out, float* chunk_sos_out) {
  const float inv_s = 1.0f / (float)S, inv_r = 1.0f / (float)R;
#pragma omp parallel for schedule(static)
  for (int k = 0; k < nids; ++k) {
    const int c = chunk_ids ? chunk_ids[k] : k;
    const long base = chunk_start[c];
    const int len = chunk_len[c];
    const long obase = chunk_out_start ? chunk_out_start[c] : base;
    float rep[16];
    for (int i = 0; i < len; ++i) {
      for (int r = 0; r < R; ++r) {
        float in = ((const float*)srcs[r * S])[base + i];
        for (int s = 1; s < S; ++s) in = in + ((const float*)srcs[r * S + s])[base + i];
        rep[r] = in * inv_s;
      }
#define OTB_REP_ADD(a, b) rep[a] = rep[a] + rep[b]
      DET_BLOCKS_FOLD(R, OTB_REP_ADD);  // binary blocks over the replicas
#undef OTB_REP_ADD
      out[obase + i] = rep[0] * inv_r;
    }
    chunk_sos_out[c] = chunk_sos(out + obase, len);
  }
  return 0;
}
int otb_cpu_chunk_sos(const float* x, const long* chunk_start, const int* chunk_len, int nchunks, float* chunk_sos_out) {
#pragma omp parallel for schedule(static)
  for (int c = 0; c < nchunks; ++c) chunk_sos_out[c] = chunk_sos(x + chunk_start[c], chunk_len[c]);
  return 0;
}
int otb_cpu_seg_pair_tree(float* chunk_sos_io, const int* seg_first, int nseg, float* seg_out) {
  for (int i = 0; i < nseg; ++i) {
    float* v = chunk_sos_io + seg_first[i];
    const int n = seg_first[i + 1] - seg_first[i];
    det_pair_tree_host(v, n);
    seg_out[i] = n > 0 ? v[0] : 0.0f;
  }
  return 0;
}
// hyper layout as in otb_adamw_push. dsts: compute-weight buffers to refresh (bf16 or fp32).
int otb_cpu_adamw_push(const float* hyper, const long* chunk_start, const int* chunk_len, const int* chunk_group,
                       int nchunks, float* master, float* grad, float* m1, float* m2, const void* const* dsts, int ndst,
                       int dst_bf16) {
  const float clip = hyper[0], beta1 = hyper[3], beta2 = hyper[4], omb1 = hyper[5], omb2 = hyper[6], eps = hyper[7],
              step_size = hyper[8], sqrt_bc2 = hyper[9];
#pragma omp parallel for schedule(static)
  for (int c = 0; c < nchunks; ++c) {
    const long base = chunk_start[c];
    const float keep = hyper[1 + chunk_group[c]];
    for (int j = 0; j < chunk_len[c]; ++j) {
      const long i = base + j;
      const float g = grad[i] * clip;
      grad[i] = g;
      float p = master[i] * keep;
      const float m = det_fmaf(m1[i], beta1, g * omb1);
      const float v = det_fmaf(m2[i], beta2, (g * g) * omb2);
      m1[i] = m;
      m2[i] = v;
      const float denom = det_sqrtf(v) / sqrt_bc2 + eps;
      p = det_fmaf(-step_size, m / denom, p);
      master[i] = p;
      for (int d = 0; d < ndst; ++d) {
        if (dst_bf16) ((uint16_t*)dsts[d])[i] = det_f2bf(p);
        else if ((float*)dsts[d] != master) ((float*)dsts[d])[i] = p;
      }
    }
  }
  return 0;
}
// Sharded state: gradient and moments are addressed by `chunk_state_start`, master weights and destinations by `chunk_start`.
int otb_cpu_adamw_push_ex(const float* hyper, const long* chunk_start, const long* chunk_state_start, const int* chunk_len, const int* chunk_group,
                       int nchunks, float* master, float* grad, float* m1, float* m2, const void* const* dsts, int ndst,
                       int dst_bf16) {
  const float clip = hyper[0], beta1 = hyper[3], beta2 = hyper[4], omb1 = hyper[5], omb2 = hyper[6], eps = hyper[7],
              step_size = hyper[8], sqrt_bc2 = hyper[9];
#pragma omp parallel for schedule(static)
  for (int c = 0; c < nchunks; ++c) {
    const long base = chunk_start[c];
    const float keep = hyper[1 + chunk_group[c]];
    for (int j = 0; j < chunk_len[c]; ++j) {
      const long i = base + j;
      const long si = (chunk_state_start ? chunk_state_start[c] : base) + j;  // gradient and moments: packed buffers
      const float g = grad[si] * clip;
      grad[si] = g;
      float p = master[i] * keep;
      const float m = det_fmaf(m1[si], beta1, g * omb1);
      const float v = det_fmaf(m2[si], beta2, (g * g) * omb2);
      m1[si] = m;
      m2[si] = v;
      const float denom = det_sqrtf(v) / sqrt_bc2 + eps;
      p = det_fmaf(-step_size, m / denom, p);
      master[i] = p;
      for (int d = 0; d < ndst; ++d) {
        if (dst_bf16) ((uint16_t*)dsts[d])[i] = det_f2bf(p);
        else if ((float*)dsts[d] != master) ((float*)dsts[d])[i] = p;
      }
    }
  }
  return 0;
}
// The same update dividing by the running element-wise maximum of the second moment (amsgrad).
int otb_cpu_adamw_push_amsgrad(const float* hyper, const long* chunk_start, const int* chunk_len, const int* chunk_group,
                       int nchunks, float* master, float* grad, float* m1, float* m2, float* vmax, const void* const* dsts, int ndst,
                       int dst_bf16) {
  const float clip = hyper[0], beta1 = hyper[3], beta2 = hyper[4], omb1 = hyper[5], omb2 = hyper[6], eps = hyper[7],
              step_size = hyper[8], sqrt_bc2 = hyper[9];
#pragma omp parallel for schedule(static)
  for (int c = 0; c < nchunks; ++c) {
    const long base = chunk_start[c];
    const float keep = hyper[1 + chunk_group[c]];
    for (int j = 0; j < chunk_len[c]; ++j) {
      const long i = base + j;
      const float g = grad[i] * clip;
      grad[i] = g;
      float p = master[i] * keep;
      const float m = det_fmaf(m1[i], beta1, g * omb1);
      const float v = det_fmaf(m2[i], beta2, (g * g) * omb2);
      m1[i] = m;
      m2[i] = v;
      const float vd = fmaxf(vmax[i], v);  // running maximum of the second moment (IEEE maxNum on both sides)
      vmax[i] = vd;
      const float denom = det_sqrtf(vd) / sqrt_bc2 + eps;
      p = det_fmaf(-step_size, m / denom, p);
      master[i] = p;
      for (int d = 0; d < ndst; ++d) {
        if (dst_bf16) ((uint16_t*)dsts[d])[i] = det_f2bf(p);
        else if ((float*)dsts[d] != master) ((float*)dsts[d])[i] = p;
      }
    }
  }
  return 0;
}
int otb_cpu_push_cast(const long* chunk_start, const int* chunk_len, int nchunks, const float* master,
                      const void* const* dsts, int ndst, int dst_bf16) {
#pragma omp parallel for schedule(static)
  for (int c = 0; c < nchunks; ++c)
    for (int j = 0; j < chunk_len[c]; ++j) {
      const long i = chunk_start[c] + j;
      for (int d = 0; d < ndst; ++d) {
        if (dst_bf16) ((uint16_t*)dsts[d])[i] = det_f2bf(master[i]);
        else if ((const float*)dsts[d] != master) ((float*)dsts[d])[i] = master[i];
      }
    }
  return 0;
}

// Hyper-parameters of one AdamW step as the fp32 values both devices use.
//   out[0] clip (filled by caller), out[1] 1 - lr*wd, out[2] 1.0, out[3] beta1, out[4] beta2, out[5] 1-beta1,
//   out[6] 1-beta2, out[7] eps, out[8] lr / (1 - beta1^step), out[9] sqrt(1 - beta2^step)
void otb_cpu_adamw_hyper(double lr, double beta1, double beta2, double eps, double wd, long step, float clip, float* out) {
  const float lrf = (float)lr, b1 = (float)beta1, b2 = (float)beta2;
  const float bc1 = (float)(1.0 - det_powi((double)b1, step));
  const float bc2 = (float)(1.0 - det_powi((double)b2, step));
  out[0] = clip;
  out[1] = 1.0f - lrf * (float)wd;
  out[2] = 1.0f;
  out[3] = b1;
  out[4] = b2;
  out[5] = 1.0f - b1;
  out[6] = 1.0f - b2;
  out[7] = (float)eps;
  out[8] = lrf / bc1;
  out[9] = det_sqrtf(bc2);
}

// ---- Philox4x32-10 truncated normal ------------------------------------------------------------
static inline void philox_round(uint32_t* c, const uint32_t* k) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
  const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k[0], n1 = (uint32_t)p1;
  const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k[1], n3 = (uint32_t)p0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
static inline void philox4x32(uint64_t ctr, uint64_t key, uint32_t* out) {
  uint32_t c[4] = {(uint32_t)ctr, (uint32_t)(ctr >> 32), 0u, 0u};
  uint32_t k[2] = {(uint32_t)key, (uint32_t)(key >> 32)};
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k);
    k[0] += 0x9E3779B9u;
    k[1] += 0xBB67AE85u;
  }
  memcpy(out, c, 16);
}
static inline float erfinv_central(float x) {  // |x| <= 0.96; Giles' single-precision polynomial
  float w = -det_logf(det_mulf(1.0f - x, 1.0f + x));
  w = w - 2.5f;
  float p = 2.81022636e-08f;
  p = det_fmaf(p, w, 3.43273939e-07f);
  p = det_fmaf(p, w, -3.5233877e-06f);
  p = det_fmaf(p, w, -4.39150654e-06f);
  p = det_fmaf(p, w, 0.00021858087f);
  p = det_fmaf(p, w, -0.00125372503f);
  p = det_fmaf(p, w, -0.00417768164f);
  p = det_fmaf(p, w, 0.246640727f);
  p = det_fmaf(p, w, 1.50140941f);
  return p * x;
}
// out[i] = std * z_i, z_i standard normal truncated to [-2, 2]; element i uses the 32-bit word
// (offset + i) of the Philox stream keyed by `seed`: the value of an element depends only on
// (seed, its index in the stream), never on how the work is split.
void otb_cpu_trunc_normal(float* out, long n, float std, uint64_t seed, uint64_t offset) {
  const float span = 0.95449973610364158f;  // erf(2/sqrt(2)) = P(|z| <= 2)
  // one Philox block yields the four words 4b .. 4b+3; walk whole blocks and drop the words outside [offset, offset + n)
  const uint64_t first = offset, end = offset + (uint64_t)n;
  const long b0 = (long)(first >> 2), b1 = (long)((end + 3) >> 2);
#pragma omp parallel for schedule(static)
  for (long b = b0; b < b1; ++b) {
    uint32_t r[4];
    philox4x32((uint64_t)b, seed, r);
    for (int j = 0; j < 4; ++j) {
      const uint64_t w = ((uint64_t)b << 2) + (uint64_t)j;
      if (w < first || w >= end) continue;
      // uniform in (-1, 1), 24 bits, symmetric about 0
      const float u = ((float)(r[j] >> 8) + 0.5f) * (1.0f / 8388608.0f) - 1.0f;
      float z = 1.41421356237309505f * erfinv_central(u * span);
      if (z > 2.0f) z = 2.0f;
      if (z < -2.0f) z = -2.0f;
      out[w - first] = z * std;
    }
  }
}
}  // extern "C"
