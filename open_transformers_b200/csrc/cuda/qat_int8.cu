// Quantisation-aware training (W8A8) support kernels for sm_100a. The int8 x int8 -> int32 product itself runs on
// the tensor cores in gemm_tc05.cu (otb_gemm_i8); this file holds everything around it:
//
//   absmax            amax = max |x|                      (order-free, so any grid gives the same bits)
//   quant_act         step = max(amax / qmax, FLT_MIN);  q = clamp(rint(x / step), +-qmax)       per tensor
//   quant_weight      q = clamp(rint(w / s[n]), +-qmax);  w_hat = q * s[n]                        per output channel
//   lsq_bwd           straight-through backward of the learned step size:
//                       dW[n,k] += |w/s| <= qmax ? G[n,k] * ga : 0
//                       ds[n]   += gs * sum_k G[n,k] * ga * ( |t| <= qmax ? rint(t) - t : sign(t) * qmax ),  t = w/s
//                     with G = dL/dw_hat of this micro-batch, ga a device scalar (the activation step the integer
//                     activations were scaled by), and the k-sum taken as the lane tree of det_reduce.h
//   row_absmean       s[n] = max(c * mean_k |w[n,k]|, floor)   (step-size initialisation and periodic refresh)
//   row_absmax        s[n] = max(amax_k |w[n,k]| / qmax, floor) (fixed-scale "absmax" layers)
//   i8_to_float       exact widening of the saved integer activations for the weight-gradient GEMM
//
// Divisions are IEEE (the library is built without fast-math), rint is round-half-even, so csrc/cpu/ref_qat.cpp
// returns the same bits.
//
// Reference roles: repop.qat.lsq.LSQQuantizedLinear / refresh_lsq_weight_scales / QuantizedLinear as called from
// src/pretrain/model/modules/_linear.py:31-65, src/pretrain/model/init.py:150-199 and
// src/pretrain/train/loop.py:1069-1084 (docs/MODEL_OP_DTYPE_TRACE.md:78,104,113-116,129).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "common.cuh"
#include "ew_common.cuh"

namespace {

inline unsigned blocks_for(long n, int per) { return (unsigned)((n + per - 1) / per); }

constexpr int AMAX_BLOCKS = 592;  // 4 per SM; partial maxima, then one block folds them

template <typename T>
__global__ void absmax_partial_kernel(const T* __restrict__ x, long n, float* __restrict__ partial) {
  __shared__ float sh[32];
  float m = 0.0f;
  const long n8 = n / 8;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float f[8];
    Vec8<T>::load(x + i * 8, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(f[e]));
  }
  for (long i = n8 * 8 + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(to_f<T>(x[i])));
  m = block_max(m, sh);
  if (threadIdx.x == 0) partial[blockIdx.x] = m;
}
__global__ void absmax_final_kernel(const float* __restrict__ partial, int n, float* __restrict__ out) {
  __shared__ float sh[32];
  float m = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, partial[i]);
  m = block_max(m, sh);
  if (threadIdx.x == 0) out[0] = m;
}

__device__ __forceinline__ float clamp_q(float q, float qmax) { return fminf(fmaxf(q, -qmax), qmax); }

template <typename T>
__global__ void quant_act_kernel(const T* __restrict__ x, long n, const float* __restrict__ amax, float inv_qmax,
                                 float qmax, int8_t* __restrict__ q, float* __restrict__ step_out) {
  const float step = fmaxf(__fmul_rn(amax[0], inv_qmax), FLT_MIN);
  if (blockIdx.x == 0 && threadIdx.x == 0) step_out[0] = step;
  const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i + 8 <= n) {
    float f[8];
    Vec8<T>::load(x + i, f);
    uint32_t w[2] = {0, 0};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int v = (int)clamp_q(rintf(__fdiv_rn(f[e], step)), qmax);
      w[e >> 2] |= (uint32_t)(v & 0xFF) << (8 * (e & 3));
    }
    *reinterpret_cast<uint2*>(q + i) = make_uint2(w[0], w[1]);
  } else {
    for (long j = i; j < n; ++j) q[j] = (int8_t)(int)clamp_q(rintf(__fdiv_rn(to_f<T>(x[j]), step)), qmax);
  }
}

// one warp per row
template <typename T, typename TO>
__global__ void quant_weight_kernel(const T* __restrict__ w, const float* __restrict__ s, long N, int K, float qmax,
                                    int8_t* __restrict__ q, TO* __restrict__ w_hat) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= N) return;
  const float sr = s[row];
  for (int c = lane * 8; c < K; c += 256) {
    float f[8], h[8];
    Vec8<T>::load(w + row * K + c, f);
    uint32_t pk[2] = {0, 0};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float qv = clamp_q(rintf(__fdiv_rn(f[e], sr)), qmax);
      h[e] = __fmul_rn(qv, sr);
      pk[e >> 2] |= (uint32_t)((int)qv & 0xFF) << (8 * (e & 3));
    }
    *reinterpret_cast<uint2*>(q + row * K + c) = make_uint2(pk[0], pk[1]);
    if (w_hat) Vec8<TO>::store(w_hat + row * K + c, h);
  }
}

// one warp per row; G fp32 [N,K] (this micro-batch's dL/dw_hat before the activation step is applied)
template <typename T>
__global__ void lsq_bwd_kernel(const float* __restrict__ G, const T* __restrict__ w, const float* __restrict__ s,
                               const float* __restrict__ ga, long N, int K, float qmax, float gs,
                               float* __restrict__ dW, float* __restrict__ ds, int learn_step) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= N) return;
  const float sr = s[row];
  const float a = ga ? ga[0] : 1.0f;
  float acc = 0.0f;
  for (int c = lane * 8; c < K; c += 256) {
    float f[8];
    Vec8<T>::load(w + row * K + c, f);
    float g[8], d[8];
    Vec8<float>::load(G + row * K + c, g);
    Vec8<float>::load(dW + row * K + c, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float t = __fdiv_rn(f[e], sr);
      const float gv = __fmul_rn(g[e], a);
      const bool inside = fabsf(t) <= qmax;
      const float term = inside ? __fsub_rn(rintf(t), t) : (t > 0.0f ? qmax : -qmax);
      acc = __fmaf_rn(gv, term, acc);
      d[e] = inside ? __fadd_rn(d[e], gv) : d[e];
    }
    Vec8<float>::store(dW + row * K + c, d);
  }
  if (learn_step) {
    const float tot = warp_butterfly(acc);
    if (lane == 0) ds[row] = __fadd_rn(ds[row], __fmul_rn(tot, gs));
  }
}

// mode 0: s = max(c * (sum_k |w|) * inv_k, floor);  mode 1: s = max(amax_k |w| * c, floor)
template <typename T>
__global__ void row_stat_kernel(const T* __restrict__ w, long N, int K, int mode, float c, float inv_k, float floor_v,
                                float* __restrict__ s) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= N) return;
  float acc = 0.0f;
  for (int cidx = lane * 8; cidx < K; cidx += 256) {
    float f[8];
    Vec8<T>::load(w + row * K + cidx, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc = mode == 0 ? __fadd_rn(acc, fabsf(f[e])) : fmaxf(acc, fabsf(f[e]));
  }
  float r;
  if (mode == 0) r = __fmul_rn(__fmul_rn(warp_butterfly(acc), inv_k), c);
  else r = __fmul_rn(warp_max(acc), c);
  if (lane == 0) s[row] = fmaxf(r, floor_v);
}

template <typename TO>
__global__ void i8_widen_kernel(const int8_t* __restrict__ q, TO* __restrict__ out, long n) {
  const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i + 8 <= n) {
    const uint2 v = *reinterpret_cast<const uint2*>(q + i);
    const uint32_t w[2] = {v.x, v.y};
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = (float)(int8_t)((w[e >> 2] >> (8 * (e & 3))) & 0xFF);
    Vec8<TO>::store(out + i, f);
  } else {
    for (long j = i; j < n; ++j) out[j] = from_f<TO>((float)q[j]);
  }
}

}  // namespace

#define S(stream) reinterpret_cast<cudaStream_t>(stream)
#define DISPATCH_T(is_bf16, ...)                       \
  if (is_bf16) { using T = __nv_bfloat16; __VA_ARGS__ } \
  else { using T = float; __VA_ARGS__ }

extern "C" int otb_absmax_scratch_floats() { return AMAX_BLOCKS; }

// amax[0] = max |x|; scratch: otb_absmax_scratch_floats() device floats. dtype: 1 bf16, 0 fp32. x 16-byte aligned.
extern "C" int otb_absmax(const void* x, long n, int dtype, float* scratch, float* amax, void* stream) {
  DISPATCH_T(dtype, absmax_partial_kernel<T><<<AMAX_BLOCKS, 256, 0, S(stream)>>>((const T*)x, n, scratch);)
  absmax_final_kernel<<<1, 256, 0, S(stream)>>>(scratch, AMAX_BLOCKS, amax);
  return (int)cudaGetLastError();
}
extern "C" int otb_quant_act(const void* x, long n, int dtype, const float* amax, int qmax, void* q, float* step,
                             void* stream) {
  if (n <= 0) return 0;
  DISPATCH_T(dtype, quant_act_kernel<T><<<blocks_for(n, 8 * 256), 256, 0, S(stream)>>>(
                        (const T*)x, n, amax, 1.0f / (float)qmax, (float)qmax, (int8_t*)q, step);)
  return (int)cudaGetLastError();
}
// w [N,K] (dtype), s [N] fp32 -> q int8 [N,K] and, when w_hat is not null, w_hat = q*s in out_dtype. K % 8 == 0.
extern "C" int otb_quant_weight(const void* w, const float* s, long N, int K, int dtype, int qmax, void* q, void* w_hat,
                                int out_dtype, void* stream) {
  if (K % 8) return -2;
  if (out_dtype) {
    DISPATCH_T(dtype, quant_weight_kernel<T, __nv_bfloat16><<<blocks_for(N, 8), 256, 0, S(stream)>>>(
                          (const T*)w, s, N, K, (float)qmax, (int8_t*)q, (__nv_bfloat16*)w_hat);)
  } else {
    DISPATCH_T(dtype, quant_weight_kernel<T, float><<<blocks_for(N, 8), 256, 0, S(stream)>>>(
                          (const T*)w, s, N, K, (float)qmax, (int8_t*)q, (float*)w_hat);)
  }
  return (int)cudaGetLastError();
}
extern "C" int otb_lsq_bwd(const float* G, const void* w, const float* s, const float* ga, long N, int K, int dtype,
                           int qmax, float gs, float* dW, float* ds, int learn_step, void* stream) {
  if (K % 8) return -2;
  DISPATCH_T(dtype, lsq_bwd_kernel<T><<<blocks_for(N, 8), 256, 0, S(stream)>>>(G, (const T*)w, s, ga, N, K, (float)qmax,
                                                                               gs, dW, ds, learn_step);)
  return (int)cudaGetLastError();
}
extern "C" int otb_row_stat(const void* w, long N, int K, int dtype, int mode, float c, float floor_v, float* s,
                            void* stream) {
  if (K % 8) return -2;
  DISPATCH_T(dtype, row_stat_kernel<T><<<blocks_for(N, 8), 256, 0, S(stream)>>>((const T*)w, N, K, mode, c,
                                                                                1.0f / (float)K, floor_v, s);)
  return (int)cudaGetLastError();
}
extern "C" int otb_i8_widen(const void* q, void* out, long n, int out_dtype, void* stream) {
  if (n <= 0) return 0;
  if (out_dtype) i8_widen_kernel<__nv_bfloat16><<<blocks_for(n, 8 * 256), 256, 0, S(stream)>>>((const int8_t*)q, (__nv_bfloat16*)out, n);
  else i8_widen_kernel<float><<<blocks_for(n, 8 * 256), 256, 0, S(stream)>>>((const int8_t*)q, (float*)out, n);
  return (int)cudaGetLastError();
}
