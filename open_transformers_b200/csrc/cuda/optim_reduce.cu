// Deterministic gradient reduction fused with its neighbours, and the AdamW update fused with the
// parameter all-gather. Both kernels move their inter-GPU traffic themselves with plain peer
// loads / stores over NVLink (pointers obtained by CUDA IPC); no NCCL call and no in-switch
// reduction: every sum is formed by this kernel in a fixed order.
//
//  grad_reduce  (pull reduce-scatter + replica tree + squared-norm partials)
//     For every element this GPU owns:
//        inner_r = (((g[r,0] + g[r,1]) + ...) + g[r,S-1]) * (1/S)       ascending shard rank
//        outer   = blocks_fold(inner_0 .. inner_{R-1})   * (1/R)          binary blocks over replicas (det_reduce.h)
//     g[r,s] is virtual rank (r*S+s)'s fp32 gradient buffer, local or a peer's. The same pass
//     writes `outer` and folds it into the squared-norm partial of its 8192-element chunk
//     (thread t takes elements j*2048 + t*8 .. +7, fma chain, block_tree_sum).
//     Reference roles: DeterministicReduceScatter + DeterministicReplicateAllReduce +
//     deterministic_per_tensor_and_global_norm (src/pretrain/parallel/deterministic_reduce.py:77-117,
//     223-290, 717-777).
//
//  adamw_push   (clip + AdamW + cast + all-gather by peer stores)
//     g *= clip; decoupled weight decay; fp32 moments; bias corrections passed in as fp32
//     (computed by det_powi); the updated parameter is written to the fp32 master and, as the
//     compute dtype, into the weight buffer of every GPU.
//     Reference roles: global_clip.py:47-55, optim/adamw_repop.py:45-120, FSDP all-gather.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "det_math.h"
#include "det_reduce.h"

namespace {

constexpr int CHUNK = 8192;
constexpr int MAX_SRC = 64;
constexpr int MAX_DST = 16;

struct ReduceSrc {
  const float* p[MAX_SRC];
};
struct PushDst {
  void* p[MAX_DST];
};

__device__ __forceinline__ float block_tree_sum_256(float v, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float w = (lane < 8) ? sh[lane] : 0.0f;
#pragma unroll
  for (int off = 4; off >= 1; off >>= 1) w = __fadd_rn(w, __shfl_xor_sync(0xffffffffu, w, off));
  return __shfl_sync(0xffffffffu, w, 0);
}

// chunk table: chunk c covers flat elements [chunk_start[c], chunk_start[c] + chunk_len[c]) (len <= 8192,
// start 16-byte aligned). One CTA per chunk.
__global__ void __launch_bounds__(256)
grad_reduce_kernel(ReduceSrc src, int S, int R, int TPN, float inv_s, float inv_r, const long* __restrict__ chunk_start,
                   const int* __restrict__ chunk_len, const int* __restrict__ chunk_ids, float* __restrict__ out,
                   float* __restrict__ chunk_sos, const long* __restrict__ chunk_out_start = nullptr) {
  __shared__ float sh[32];
  // a launch covers either the first gridDim.x chunks of the table or, with `chunk_ids`, the listed ones (one bucket)
  const int c = chunk_ids ? chunk_ids[blockIdx.x] : (int)blockIdx.x;
  const long base = chunk_start[c];
  const int len = chunk_len[c];
  float acc = 0.0f;
  for (int j = threadIdx.x * 8; j < len; j += 2048) {
    float o[8];
    const bool vec = (j + 8 <= len);
    float rep[16][8];
    for (int r = 0; r < R; ++r) {
      float in[8];
      for (int s = 0; s < S; ++s) {
        const float* p = src.p[(r * S + s) * TPN] + base + j;
        float v[8];
        if (vec) {
          const float4 a = *reinterpret_cast<const float4*>(p);
          const float4 b = *reinterpret_cast<const float4*>(p + 4);
          v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = (j + e < len) ? p[e] : 0.0f;
        }
        // Tensor-parallel group of TPN processes: each wrote only its own slices of this virtual rank's gradient and
        // left +0.0 elsewhere, so at most one of the TPN buffers holds a non-zero bit pattern per element and the
        // integer sum of the patterns is that pattern, exactly (no floating-point addition, no order).
        for (int t = 1; t < TPN; ++t) {
          const float* pt = src.p[(r * S + s) * TPN + t] + base + j;
          if (vec) {
            const uint4 a = *reinterpret_cast<const uint4*>(pt);
            const uint4 b = *reinterpret_cast<const uint4*>(pt + 4);
            const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(__float_as_uint(v[e]) + w[e]);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (j + e < len) v[e] = __uint_as_float(__float_as_uint(v[e]) + __float_as_uint(pt[e]));
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) in[e] = (s == 0) ? v[e] : __fadd_rn(in[e], v[e]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) rep[r][e] = __fmul_rn(in[e], inv_s);
    }
    // binary blocks over the replicas (det_reduce.h): balanced trees inside the power-of-two blocks of R, block sums added
    // left to right
#define OTB_REP_ADD(a, b)                                                            \
  _Pragma("unroll") for (int e = 0; e < 8; ++e) rep[a][e] = __fadd_rn(rep[a][e], rep[b][e])
    DET_BLOCKS_FOLD(R, OTB_REP_ADD);
#undef OTB_REP_ADD
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      o[e] = __fmul_rn(rep[0][e], inv_r);
      if (j + e < len) acc = __fmaf_rn(o[e], o[e], acc);
    }
    // the reduced gradient may live in a packed buffer that holds this process's segments only (sharded state)
    float* q = out + (chunk_out_start ? chunk_out_start[c] : base) + j;
    if (vec) {
      *reinterpret_cast<float4*>(q) = make_float4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<float4*>(q + 4) = make_float4(o[4], o[5], o[6], o[7]);
    } else {
      for (int e = 0; e < 8 && j + e < len; ++e) q[e] = o[e];
    }
  }
  const float s = block_tree_sum_256(acc, sh);
  if (threadIdx.x == 0) chunk_sos[c] = s;
}

// Readiness flags of the overlapped reduction. Every GPU owns an array of `buckets x P` words in peer-mapped memory;
// word [b * P + r] takes the step's epoch when rank r's gradients of bucket b are final. A signal is one release store
// per destination at system scope; a wait is a bounded acquire poll (no trap, no endless loop: when the budget runs
// out the kernel records which word it gave up on in `status` and returns, and the host raises after its next sync).
struct FlagDst {
  uint32_t* p[MAX_DST];
};
__global__ void flag_signal_kernel(FlagDst dst, int ndst, int idx, uint32_t val) {
  const int d = threadIdx.x;
  if (d < ndst) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst.p[d] + idx), "r"(val) : "memory");
  }
}
__global__ void flag_wait_kernel(const uint32_t* flags, int first, int count, uint32_t val, unsigned long long budget_ns,
                                 uint32_t* status, uint32_t code) {
  const int t = threadIdx.x;
  if (t >= count) return;
  const uint32_t* f = flags + first + t;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t i = 0;; ++i) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if (v == val) return;
    if ((i & 15u) == 15u) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > budget_ns) break;
    }
    __nanosleep(200);
  }
  if (status) {
    atomicExch(status, code);
    atomicExch(status + 1, (uint32_t)(first + t));
  }
}

// Squared-norm partials only (same chunk order), for tensors that are not reduced by this kernel.
__global__ void __launch_bounds__(256)
chunk_sos_kernel(const float* __restrict__ x, const long* __restrict__ chunk_start, const int* __restrict__ chunk_len,
                 float* __restrict__ chunk_sos) {
  __shared__ float sh[32];
  const long base = chunk_start[blockIdx.x];
  const int len = chunk_len[blockIdx.x];
  float acc = 0.0f;
  for (int j = threadIdx.x * 8; j < len; j += 2048)
    for (int e = 0; e < 8 && j + e < len; ++e) {
      const float v = x[base + j + e];
      acc = __fmaf_rn(v, v, acc);
    }
  const float s = block_tree_sum_256(acc, sh);
  if (threadIdx.x == 0) chunk_sos[blockIdx.x] = s;
}

// segment sums: seg i = pair_tree over chunk_sos[seg_first[i] .. seg_first[i+1]), in place. One CTA per segment;
// every level of the tree is a parallel sweep (the association is the stride tree of det_reduce.h).
__global__ void __launch_bounds__(256) seg_pair_tree_kernel(float* __restrict__ chunk_sos, const int* __restrict__ seg_first,
                                                            int nseg, float* __restrict__ seg_out) {
  const int i = blockIdx.x;
  if (i >= nseg) return;
  float* v = chunk_sos + seg_first[i];
  const int n = seg_first[i + 1] - seg_first[i];
  for (int s = 1; s < n; s *= 2) {
    for (int k = threadIdx.x * 2 * s; k + s < n; k += 512 * s) v[k] = __fadd_rn(v[k], v[k + s]);
    __syncthreads();
  }
  if (threadIdx.x == 0) seg_out[i] = n > 0 ? v[0] : 0.0f;
}

struct AdamArgs {
  float clip, lr_wd_keep[2];  // keep factor 1 - lr*wd for group 0 (decay) and 1 (no decay = 1.0)
  float beta1, beta2, one_m_b1, one_m_b2, eps, step_size, sqrt_bc2;
};

// AMSGRAD: `vmax` keeps the running element-wise maximum of the second moment and the update divides by it
// (max_exp_avg_sq of torch.optim.AdamW(amsgrad=True); reference src/pretrain/optim/adamw_repop.py:105-118).
template <bool DST_BF16, bool AMSGRAD = false>
__global__ void __launch_bounds__(256)
adamw_push_kernel(AdamArgs a, const long* __restrict__ chunk_start, const int* __restrict__ chunk_len,
                  const int* __restrict__ chunk_group, float* __restrict__ master, float* __restrict__ grad,
                  float* __restrict__ m1, float* __restrict__ m2, PushDst dst, int ndst, float* __restrict__ vmax = nullptr,
                  const long* __restrict__ chunk_state_start = nullptr) {
  const long base = chunk_start[blockIdx.x];
  const int len = chunk_len[blockIdx.x];
  // sharded state: gradient and moments sit in packed buffers of this process's segments (their own offsets), the master
  // weights and the destinations keep the full layout
  const long sdelta = chunk_state_start ? chunk_state_start[blockIdx.x] - base : 0;
  grad += sdelta;
  m1 += sdelta;
  m2 += sdelta;
  if (AMSGRAD) vmax += sdelta;
  const float keep = a.lr_wd_keep[chunk_group[blockIdx.x]];
  for (int j = threadIdx.x * 8; j < len; j += 2048) {
    float pn[8];
    const long i0 = base + j;
    if (j + 8 <= len) {
      float gv[8], pv[8], mv[8], vv[8];
      *reinterpret_cast<float4*>(gv) = *reinterpret_cast<const float4*>(grad + i0);
      *reinterpret_cast<float4*>(gv + 4) = *reinterpret_cast<const float4*>(grad + i0 + 4);
      *reinterpret_cast<float4*>(pv) = *reinterpret_cast<const float4*>(master + i0);
      *reinterpret_cast<float4*>(pv + 4) = *reinterpret_cast<const float4*>(master + i0 + 4);
      *reinterpret_cast<float4*>(mv) = *reinterpret_cast<const float4*>(m1 + i0);
      *reinterpret_cast<float4*>(mv + 4) = *reinterpret_cast<const float4*>(m1 + i0 + 4);
      *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(m2 + i0);
      *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(m2 + i0 + 4);
      float xv[8];
      if (AMSGRAD) {
        *reinterpret_cast<float4*>(xv) = *reinterpret_cast<const float4*>(vmax + i0);
        *reinterpret_cast<float4*>(xv + 4) = *reinterpret_cast<const float4*>(vmax + i0 + 4);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float g = __fmul_rn(gv[e], a.clip);
        gv[e] = g;
        float p = __fmul_rn(pv[e], keep);
        const float m = __fmaf_rn(mv[e], a.beta1, __fmul_rn(g, a.one_m_b1));
        const float v = __fmaf_rn(vv[e], a.beta2, __fmul_rn(__fmul_rn(g, g), a.one_m_b2));
        mv[e] = m;
        vv[e] = v;
        float vd = v;
        if (AMSGRAD) {
          vd = fmaxf(xv[e], v);
          xv[e] = vd;
        }
        const float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(vd), a.sqrt_bc2), a.eps);
        p = __fmaf_rn(-a.step_size, __fdiv_rn(m, denom), p);
        pv[e] = p;
        pn[e] = p;
      }
      *reinterpret_cast<float4*>(grad + i0) = *reinterpret_cast<float4*>(gv);
      *reinterpret_cast<float4*>(grad + i0 + 4) = *reinterpret_cast<float4*>(gv + 4);
      *reinterpret_cast<float4*>(master + i0) = *reinterpret_cast<float4*>(pv);
      *reinterpret_cast<float4*>(master + i0 + 4) = *reinterpret_cast<float4*>(pv + 4);
      *reinterpret_cast<float4*>(m1 + i0) = *reinterpret_cast<float4*>(mv);
      *reinterpret_cast<float4*>(m1 + i0 + 4) = *reinterpret_cast<float4*>(mv + 4);
      *reinterpret_cast<float4*>(m2 + i0) = *reinterpret_cast<float4*>(vv);
      *reinterpret_cast<float4*>(m2 + i0 + 4) = *reinterpret_cast<float4*>(vv + 4);
      if (AMSGRAD) {
        *reinterpret_cast<float4*>(vmax + i0) = *reinterpret_cast<float4*>(xv);
        *reinterpret_cast<float4*>(vmax + i0 + 4) = *reinterpret_cast<float4*>(xv + 4);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (j + e < len) {
          const long i = base + j + e;
          const float g = __fmul_rn(grad[i], a.clip);
          grad[i] = g;
          float p = __fmul_rn(master[i], keep);
          const float m = __fmaf_rn(m1[i], a.beta1, __fmul_rn(g, a.one_m_b1));
          const float v = __fmaf_rn(m2[i], a.beta2, __fmul_rn(__fmul_rn(g, g), a.one_m_b2));
          m1[i] = m;
          m2[i] = v;
          float vd = v;
          if (AMSGRAD) {
            vd = fmaxf(vmax[i], v);
            vmax[i] = vd;
          }
          const float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(vd), a.sqrt_bc2), a.eps);
          p = __fmaf_rn(-a.step_size, __fdiv_rn(m, denom), p);
          master[i] = p;
          pn[e] = p;
        } else {
          pn[e] = 0.0f;
        }
      }
    }
    const bool vec = (j + 8 <= len);
    for (int d = 0; d < ndst; ++d) {
      if (DST_BF16) {
        __nv_bfloat16* q = reinterpret_cast<__nv_bfloat16*>(dst.p[d]) + base + j;
        if (vec) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 b = __floats2bfloat162_rn(pn[2 * e], pn[2 * e + 1]);
            w[e] = *reinterpret_cast<uint32_t*>(&b);
          }
          *reinterpret_cast<uint4*>(q) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
          for (int e = 0; e < 8 && j + e < len; ++e) q[e] = __float2bfloat16_rn(pn[e]);
        }
      } else {
        float* q = reinterpret_cast<float*>(dst.p[d]) + base + j;
        if (q == master + base + j) continue;  // the master itself is the local fp32 compute weight
        for (int e = 0; e < 8 && j + e < len; ++e) q[e] = pn[e];
      }
    }
  }
}

// fp32 -> compute dtype copy of whole chunks into every destination (initial broadcast of the weights)
template <bool DST_BF16>
__global__ void __launch_bounds__(256)
push_cast_kernel(const long* __restrict__ chunk_start, const int* __restrict__ chunk_len, const float* __restrict__ master,
                 PushDst dst, int ndst) {
  const long base = chunk_start[blockIdx.x];
  const int len = chunk_len[blockIdx.x];
  for (int j = threadIdx.x; j < len; j += 256) {
    const float p = master[base + j];
    for (int d = 0; d < ndst; ++d) {
      if (DST_BF16) reinterpret_cast<__nv_bfloat16*>(dst.p[d])[base + j] = __float2bfloat16_rn(p);
      else if (reinterpret_cast<float*>(dst.p[d]) != master) reinterpret_cast<float*>(dst.p[d])[base + j] = p;
    }
  }
}

}  // namespace

extern "C" int otb_chunk_size() { return CHUNK; }

// srcs: nsrc = S*R device pointers (fp32 flat gradient buffers, replica-major). Chunks must start at
// 16-byte aligned element offsets.
extern "C" int otb_grad_reduce(const void* const* srcs, int S, int R, const long* chunk_start, const int* chunk_len,
                               int nchunks, float* out, float* chunk_sos, void* stream) {
  if (S * R > MAX_SRC || R > 16 || S < 1 || R < 1) return -2;
  if (nchunks <= 0) return 0;
  ReduceSrc rs;
  for (int i = 0; i < S * R; ++i) rs.p[i] = reinterpret_cast<const float*>(srcs[i]);
  const float inv_s = 1.0f / (float)S, inv_r = 1.0f / (float)R;
  grad_reduce_kernel<<<nchunks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(rs, S, R, 1, inv_s, inv_r, chunk_start,
                                                                                  chunk_len, nullptr, out, chunk_sos);
  return (int)cudaGetLastError();
}
// The same reduction over the chunks listed in `chunk_ids` (indices into the chunk table; `chunk_sos` is indexed by
// them as well): one bucket of the reduction that runs under the backward pass.
extern "C" int otb_grad_reduce_ids(const void* const* srcs, int S, int R, const long* chunk_start, const int* chunk_len,
                                   const int* chunk_ids, int nids, float* out, float* chunk_sos, void* stream) {
  if (S * R > MAX_SRC || R > 16 || S < 1 || R < 1 || !chunk_ids) return -2;
  if (nids <= 0) return 0;
  ReduceSrc rs;
  for (int i = 0; i < S * R; ++i) rs.p[i] = reinterpret_cast<const float*>(srcs[i]);
  const float inv_s = 1.0f / (float)S, inv_r = 1.0f / (float)R;
  grad_reduce_kernel<<<nids, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(rs, S, R, 1, inv_s, inv_r, chunk_start, chunk_len,
                                                                               chunk_ids, out, chunk_sos);
  return (int)cudaGetLastError();
}
// Tensor-parallel groups: srcs holds S*R*tp pointers, [virtual rank][tensor-parallel rank]; the tp partial buffers of a
// virtual rank (disjoint slices, zeros elsewhere) are assembled by integer addition of their bit patterns, then the
// same shard fold and replica tree run. `chunk_ids` may be null (the first `n` chunks of the table).
extern "C" int otb_grad_reduce_tp(const void* const* srcs, int S, int R, int tp, const long* chunk_start, const int* chunk_len,
                                  const int* chunk_ids, int n, float* out, float* chunk_sos, void* stream) {
  if (tp < 1 || S * R * tp > MAX_SRC || R > 16 || S < 1 || R < 1) return -2;
  if (n <= 0) return 0;
  ReduceSrc rs;
  for (int i = 0; i < S * R * tp; ++i) rs.p[i] = reinterpret_cast<const float*>(srcs[i]);
  const float inv_s = 1.0f / (float)S, inv_r = 1.0f / (float)R;
  grad_reduce_kernel<<<n, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(rs, S, R, tp, inv_s, inv_r, chunk_start, chunk_len, chunk_ids,
                                                                            out, chunk_sos);
  return (int)cudaGetLastError();
}
// Writes `val` into word `idx` of every destination flag array (this GPU's and the peers'), after everything queued
// before it on `stream`.
extern "C" int otb_flag_signal(void* const* dsts, int ndst, int idx, unsigned val, void* stream) {
  if (ndst < 1 || ndst > MAX_DST || idx < 0) return -2;
  FlagDst fd{};
  for (int i = 0; i < ndst; ++i) fd.p[i] = reinterpret_cast<uint32_t*>(dsts[i]);
  flag_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(fd, ndst, idx, val);
  return (int)cudaGetLastError();
}
// Holds `stream` until words [first, first + count) of this GPU's flag array equal `val`, for at most `budget_ns`; a
// wait that runs out writes `code` to status[0] and the word's index to status[1] and lets the stream go on.
extern "C" int otb_flag_wait(const void* flags, int first, int count, unsigned val, unsigned long long budget_ns,
                             uint32_t* status, unsigned code, void* stream) {
  if (count < 1 || count > 32 || first < 0) return -2;
  flag_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const uint32_t*>(flags), first, count,
                                                                         val, budget_ns, status, code);
  return (int)cudaGetLastError();
}
extern "C" int otb_chunk_sos(const float* x, const long* chunk_start, const int* chunk_len, int nchunks, float* chunk_sos,
                             void* stream) {
  if (nchunks <= 0) return 0;
  chunk_sos_kernel<<<nchunks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, chunk_start, chunk_len, chunk_sos);
  return (int)cudaGetLastError();
}
extern "C" int otb_seg_pair_tree(float* chunk_sos, const int* seg_first, int nseg, float* seg_out, void* stream) {
  if (nseg <= 0) return 0;
  seg_pair_tree_kernel<<<nseg, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(chunk_sos, seg_first, nseg,
                                                                                             seg_out);
  return (int)cudaGetLastError();
}
// hyper: [clip, keep_decay, keep_nodecay, beta1, beta2, 1-beta1, 1-beta2, eps, step_size, sqrt_bc2] (fp32, host-computed
// with the shared deterministic helpers). dsts: ndst pointers to weight buffers (this GPU's and the peers').
extern "C" int otb_adamw_push(const float* hyper, const long* chunk_start, const int* chunk_len, const int* chunk_group,
                              int nchunks, float* master, float* grad, float* m1, float* m2, const void* const* dsts,
                              int ndst, int dst_bf16, void* stream) {
  if (ndst > MAX_DST) return -2;
  if (nchunks <= 0) return 0;
  AdamArgs a;
  a.clip = hyper[0]; a.lr_wd_keep[0] = hyper[1]; a.lr_wd_keep[1] = hyper[2]; a.beta1 = hyper[3]; a.beta2 = hyper[4];
  a.one_m_b1 = hyper[5]; a.one_m_b2 = hyper[6]; a.eps = hyper[7]; a.step_size = hyper[8]; a.sqrt_bc2 = hyper[9];
  PushDst pd;
  for (int i = 0; i < ndst; ++i) pd.p[i] = const_cast<void*>(dsts[i]);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dst_bf16) adamw_push_kernel<true><<<nchunks, 256, 0, s>>>(a, chunk_start, chunk_len, chunk_group, master, grad, m1, m2, pd, ndst);
  else adamw_push_kernel<false><<<nchunks, 256, 0, s>>>(a, chunk_start, chunk_len, chunk_group, master, grad, m1, m2, pd, ndst);
  return (int)cudaGetLastError();
}
// The same update with the running maximum of the second moment (`vmax`, fp32, same layout as m2).
extern "C" int otb_adamw_push_amsgrad(const float* hyper, const long* chunk_start, const int* chunk_len, const int* chunk_group,
                                      int nchunks, float* master, float* grad, float* m1, float* m2, float* vmax,
                                      const void* const* dsts, int ndst, int dst_bf16, void* stream) {
  if (ndst > MAX_DST || !vmax) return -2;
  if (nchunks <= 0) return 0;
  AdamArgs a;
  a.clip = hyper[0]; a.lr_wd_keep[0] = hyper[1]; a.lr_wd_keep[1] = hyper[2]; a.beta1 = hyper[3]; a.beta2 = hyper[4];
  a.one_m_b1 = hyper[5]; a.one_m_b2 = hyper[6]; a.eps = hyper[7]; a.step_size = hyper[8]; a.sqrt_bc2 = hyper[9];
  PushDst pd;
  for (int i = 0; i < ndst; ++i) pd.p[i] = const_cast<void*>(dsts[i]);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dst_bf16) adamw_push_kernel<true, true><<<nchunks, 256, 0, s>>>(a, chunk_start, chunk_len, chunk_group, master, grad, m1, m2, pd, ndst, vmax);
  else adamw_push_kernel<false, true><<<nchunks, 256, 0, s>>>(a, chunk_start, chunk_len, chunk_group, master, grad, m1, m2, pd, ndst, vmax);
  return (int)cudaGetLastError();
}
// Sharded state: the reduced gradient goes to `out + chunk_out_start[c]` (a packed buffer of the owned segments).
// `tp` >= 1 partial buffers per virtual rank; `chunk_ids` may be null.
extern "C" int otb_grad_reduce_ex(const void* const* srcs, int S, int R, int tp, const long* chunk_start, const int* chunk_len,
                                  const int* chunk_ids, int n, const long* chunk_out_start, float* out, float* chunk_sos, void* stream) {
  if (tp < 1 || S * R * tp > MAX_SRC || R > 16 || S < 1 || R < 1) return -2;
  if (n <= 0) return 0;
  ReduceSrc rs;
  for (int i = 0; i < S * R * tp; ++i) rs.p[i] = reinterpret_cast<const float*>(srcs[i]);
  const float inv_s = 1.0f / (float)S, inv_r = 1.0f / (float)R;
  grad_reduce_kernel<<<n, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(rs, S, R, tp, inv_s, inv_r, chunk_start, chunk_len, chunk_ids,
                                                                            out, chunk_sos, chunk_out_start);
  return (int)cudaGetLastError();
}
// Sharded state: gradient and moments are addressed by `chunk_state_start`, master weights and destinations by `chunk_start`.
extern "C" int otb_adamw_push_ex(const float* hyper, const long* chunk_start, const long* chunk_state_start, const int* chunk_len,
                                 const int* chunk_group, int nchunks, float* master, float* grad, float* m1, float* m2,
                                 const void* const* dsts, int ndst, int dst_bf16, void* stream) {
  if (ndst > MAX_DST) return -2;
  if (nchunks <= 0) return 0;
  AdamArgs a;
  a.clip = hyper[0]; a.lr_wd_keep[0] = hyper[1]; a.lr_wd_keep[1] = hyper[2]; a.beta1 = hyper[3]; a.beta2 = hyper[4];
  a.one_m_b1 = hyper[5]; a.one_m_b2 = hyper[6]; a.eps = hyper[7]; a.step_size = hyper[8]; a.sqrt_bc2 = hyper[9];
  PushDst pd;
  for (int i = 0; i < ndst; ++i) pd.p[i] = const_cast<void*>(dsts[i]);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dst_bf16) adamw_push_kernel<true><<<nchunks, 256, 0, s>>>(a, chunk_start, chunk_len, chunk_group, master, grad, m1, m2, pd, ndst, nullptr, chunk_state_start);
  else adamw_push_kernel<false><<<nchunks, 256, 0, s>>>(a, chunk_start, chunk_len, chunk_group, master, grad, m1, m2, pd, ndst, nullptr, chunk_state_start);
  return (int)cudaGetLastError();
}
extern "C" int otb_push_cast(const long* chunk_start, const int* chunk_len, int nchunks, const float* master,
                             const void* const* dsts, int ndst, int dst_bf16, void* stream) {
  if (ndst > MAX_DST) return -2;
  if (nchunks <= 0) return 0;
  PushDst pd;
  for (int i = 0; i < ndst; ++i) pd.p[i] = const_cast<void*>(dsts[i]);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dst_bf16) push_cast_kernel<true><<<nchunks, 256, 0, s>>>(chunk_start, chunk_len, master, pd, ndst);
  else push_cast_kernel<false><<<nchunks, 256, 0, s>>>(chunk_start, chunk_len, master, pd, ndst);
  return (int)cudaGetLastError();
}

// ---- CUDA IPC helpers (peer-mapped flat buffers) ---------------------------------------------
extern "C" int otb_ipc_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  OTB_CUDA_CHECK_RET(cudaMalloc(ptr, bytes));
  OTB_CUDA_CHECK_RET(cudaMemset(*ptr, 0, bytes));
  cudaIpcMemHandle_t h;
  OTB_CUDA_CHECK_RET(cudaIpcGetMemHandle(&h, *ptr));
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int otb_ipc_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  OTB_CUDA_CHECK_RET(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
extern "C" int otb_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
extern "C" int otb_ipc_free(void* ptr) { return (int)cudaFree(ptr); }
