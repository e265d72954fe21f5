// Allocation-free RMSNorm backward: see rmsnorm_bwd_noalloc.h for who needs it and the rules of use.
// Same arithmetic and the same reduction order as the regular backward in elementwise.cu (one warp per
// slab of 8 rows, ascending-row fold inside the slab, pair tree over slabs), with the slab partials kept
// in a fixed device array instead of a caller-provided buffer.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "rmsnorm_bwd_noalloc.h"

// The work buffer: part of the library image, one copy per GPU that loads it. In host code this name is
// only a handle for cudaGetSymbolAddress - it is NOT a device address and must never be passed to a kernel.
static __device__ __align__(256) float g_noalloc_partials[OTB_RMSNORM_NOALLOC_MAX_FLOATS];

namespace {

constexpr int SLAB = 8;
constexpr int MAX_DEVICES = 64;

template <typename T> struct V8;
template <> struct V8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 b = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&b);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct V8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
};

template <typename T, int MAXC>
__global__ void rmsnorm_bwd_noalloc_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                           const float* __restrict__ rstd_in, T* __restrict__ dx, float* __restrict__ partials,
                                           long rows, int D, float inv_d) {
  const long slab = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const long r0 = slab * SLAB;
  if (r0 >= rows) return;
  float dg[MAXC][8];
#pragma unroll
  for (int j = 0; j < MAXC; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) dg[j][e] = 0.0f;
  for (long row = r0; row < r0 + SLAB && row < rows; ++row) {
    const float rstd = rstd_in[row];
    const T* xr = x + row * D;
    const T* dyr = dy + row * D;
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
      const int c = lane * 8 + j * 256;
      if (c < D) {
        float xf[8], df[8], g[8];
        V8<T>::load(xr + c, xf);
        V8<T>::load(dyr + c, df);
        if (w) V8<T>::load(w + c, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = __fmul_rn(xf[e], rstd);
          const float gy = w ? __fmul_rn(df[e], g[e]) : df[e];
          acc = __fmaf_rn(gy, xh, acc);
          dg[j][e] = __fadd_rn(dg[j][e], __fmul_rn(df[e], xh));
        }
      }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
    const float cs = __fmul_rn(acc, inv_d);
    T* dxr = dx + row * D;
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
      const int c = lane * 8 + j * 256;
      if (c < D) {
        float xf[8], df[8], g[8], o[8];
        V8<T>::load(xr + c, xf);
        V8<T>::load(dyr + c, df);
        if (w) V8<T>::load(w + c, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = __fmul_rn(xf[e], rstd);
          const float gy = w ? __fmul_rn(df[e], g[e]) : df[e];
          o[e] = __fmul_rn(rstd, __fmaf_rn(-xh, cs, gy));
        }
        V8<T>::store(dxr + c, o);
      }
    }
  }
  // every (slab, column) entry that the tree below reads is written here, whatever the array held before
  float* out = partials + slab * D;
#pragma unroll
  for (int j = 0; j < MAXC; ++j) {
    const int c = lane * 8 + j * 256;
    if (c < D) {
      *reinterpret_cast<float4*>(out + c) = make_float4(dg[j][0], dg[j][1], dg[j][2], dg[j][3]);
      *reinterpret_cast<float4*>(out + c + 4) = make_float4(dg[j][4], dg[j][5], dg[j][6], dg[j][7]);
    }
  }
}

// pair tree over the slabs, then the total goes to the caller's dgamma
__global__ void noalloc_tree_kernel(float* __restrict__ v, long n, int D, float* __restrict__ dgamma) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= D) return;
  for (long s = 1; s < n; s *= 2)
    for (long i = 0; i + s < n; i += 2 * s) v[i * D + col] = __fadd_rn(v[i * D + col], v[(i + s) * D + col]);
  dgamma[col] = v[col];
}

// device address of the work buffer, looked up once per device
float* g_scratch_addr[MAX_DEVICES] = {nullptr};
std::mutex g_scratch_mutex;

int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return (int)cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partials);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return (int)cudaErrorInvalidSymbol;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

template <typename T>
int launch(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dgamma, float* partials, long rows,
           int D, float inv_d, cudaStream_t s) {
  const long slabs = (rows + SLAB - 1) / SLAB;
  const unsigned grid = (unsigned)((slabs + 3) / 4);
#define RB(MAXC)                                                                                                        \
  rmsnorm_bwd_noalloc_kernel<T, MAXC><<<grid, 128, 0, s>>>((const T*)dy, (const T*)x, (const T*)w, rstd, (T*)dx, partials, rows, D, inv_d)
  if (D <= 256) RB(1); else if (D <= 1024) RB(4); else if (D <= 2048) RB(8); else RB(16);
#undef RB
  if (w != nullptr && dgamma != nullptr) noalloc_tree_kernel<<<(D + 127) / 128, 128, 0, s>>>(partials, slabs, D, dgamma);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" int otb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dgamma,
                                       long rows, int D, float inv_d, int dtype, void* stream) {
  if (rows <= 0 || D <= 0 || (D % 8) != 0 || D > 4096) return OTB_NOALLOC_BAD_SHAPE;
  const long slabs = (rows + SLAB - 1) / SLAB;
  if ((unsigned long long)slabs * (unsigned long long)D > (unsigned long long)OTB_RMSNORM_NOALLOC_MAX_FLOATS) return OTB_NOALLOC_TOO_LARGE;
  float* partials = nullptr;
  const int rc = scratch_for_current_device(&partials);
  if (rc != 0) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype) return launch<__nv_bfloat16>(dy, x, w, rstd, dx, dgamma, partials, rows, D, inv_d, s);
  return launch<float>(dy, x, w, rstd, dx, dgamma, partials, rows, D, inv_d, s);
}
