// BLAKE2b tree digest on the GPU: one thread per 4096-byte leaf, one launch per tree level, a
// single thread for the final node. Byte-identical to otb_cpu_tree_digest (csrc/cpu/hash.cpp) and
// to hashlib.blake2b applied leaf by leaf. Used for the per-tensor digests of the state hash when
// `train.state_hash.tensor_digest = tree`: hashing the fp32 master weights, both moments and the
// post-clip gradients of a 1.6 B-parameter model stays on the device instead of crossing PCIe
// into a serial host hash (reference src/pretrain/train/state_hash.py:102-103).
#include <cuda_runtime.h>
#include <stdint.h>

#include "blake2b.h"
#include "common.cuh"

namespace {
__global__ void tree_level_kernel(const uint8_t* __restrict__ data, uint64_t n, uint8_t* __restrict__ out, uint64_t leaves) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= leaves) return;
  const uint64_t off = i * OTB_TREE_LEAF;
  const uint64_t l = (n - off < OTB_TREE_LEAF) ? n - off : OTB_TREE_LEAF;
  uint8_t d[32];
  b2_hash(data + off, l, d, 32);
  for (int k = 0; k < 32; ++k) out[i * 32 + k] = d[k];
}
__global__ void tree_final_kernel(const uint8_t* __restrict__ data, uint64_t n, uint64_t total_len, uint8_t* __restrict__ out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  __shared__ uint64_t buf[(OTB_TREE_LEAF + 16) / 8];
  uint8_t* b = reinterpret_cast<uint8_t*>(buf);
  for (uint64_t i = 0; i < n; ++i) b[i] = data[i];
  for (int k = 0; k < 8; ++k) b[n + k] = (uint8_t)(total_len >> (8 * k));
  uint8_t d[32];
  b2_hash(b, n + 8, d, 32);
  for (int k = 0; k < 32; ++k) out[k] = d[k];
}
}  // namespace

// bytes of scratch needed for a message of `len` bytes
extern "C" uint64_t otb_tree_digest_scratch(uint64_t len) {
  uint64_t total = 0, n = len;
  while (n > OTB_TREE_LEAF) {
    n = ((n + OTB_TREE_LEAF - 1) / OTB_TREE_LEAF) * 32;
    total += (n + 255) & ~uint64_t(255);
  }
  return total + 256;
}
// data: device pointer (8-byte aligned), out32: device pointer to 32 bytes.
extern "C" int otb_tree_digest(const void* data, uint64_t len, void* scratch, uint64_t scratch_bytes, void* out32,
                               void* stream) {
  if (scratch_bytes < otb_tree_digest_scratch(len)) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const uint8_t* p = reinterpret_cast<const uint8_t*>(data);
  uint8_t* sc = reinterpret_cast<uint8_t*>(scratch);
  uint64_t n = len;
  while (n > OTB_TREE_LEAF) {
    const uint64_t leaves = (n + OTB_TREE_LEAF - 1) / OTB_TREE_LEAF;
    tree_level_kernel<<<(unsigned)((leaves + 63) / 64), 64, 0, s>>>(p, n, sc, leaves);
    p = sc;
    n = leaves * 32;
    sc += (n + 255) & ~uint64_t(255);
  }
  tree_final_kernel<<<1, 32, 0, s>>>(p, n, len, reinterpret_cast<uint8_t*>(out32));
  return (int)cudaGetLastError();
}

// ---- batched variant: many messages, one launch per tree level ---------------------------------
namespace {
struct BatchLevel {
  const uint8_t* const* src;  // [n] message pointers at this level
  const uint64_t* len;        // [n] message lengths at this level
  const uint64_t* leaf_prefix;  // [n+1] first global leaf of each message (messages already <= one leaf contribute 0)
  uint8_t* const* dst;        // [n] where this level's leaf digests go
};
__global__ void tree_level_batch_kernel(BatchLevel lv, int n, uint64_t total_leaves) {
  const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= total_leaves) return;
  int lo = 0, hi = n;  // last message with leaf_prefix <= gid
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (lv.leaf_prefix[mid] <= gid) lo = mid; else hi = mid;
  }
  const uint64_t leaf = gid - lv.leaf_prefix[lo];
  const uint64_t nbytes = lv.len[lo];
  const uint64_t off = leaf * OTB_TREE_LEAF;
  const uint64_t l = (nbytes - off < OTB_TREE_LEAF) ? nbytes - off : OTB_TREE_LEAF;
  uint8_t d[32];
  b2_hash(lv.src[lo] + off, l, d, 32);
  uint8_t* o = lv.dst[lo] + leaf * 32;
  for (int k = 0; k < 32; ++k) o[k] = d[k];
}
__global__ void tree_final_batch_kernel(const uint8_t* const* src, const uint64_t* len, const uint64_t* total_len, int n,
                                        uint8_t* out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint64_t buf[(OTB_TREE_LEAF + 16) / 8];
  uint8_t* b = reinterpret_cast<uint8_t*>(buf);
  const uint64_t m = len[i];
  for (uint64_t k = 0; k < m; ++k) b[k] = src[i][k];
  for (int k = 0; k < 8; ++k) b[m + k] = (uint8_t)(total_len[i] >> (8 * k));
  uint8_t d[32];
  b2_hash(b, m + 8, d, 32);
  for (int k = 0; k < 32; ++k) out[(size_t)i * 32 + k] = d[k];
}
}  // namespace

// Tree digests of n messages (device pointers `data[i]`, `lens[i]` bytes; host arrays). `work` is a device
// buffer of at least otb_tree_digest_batch_work(lens, n) bytes; out: device, n*32 bytes.
extern "C" uint64_t otb_tree_digest_batch_work(const uint64_t* lens, int n) {
  uint64_t total = 0;
  for (int i = 0; i < n; ++i) total += otb_tree_digest_scratch(lens[i]);
  return total + (uint64_t)n * 8 * 16 + 4096;  // + pointer/length tables (rebuilt per level)
}
extern "C" int otb_tree_digest_batch(const void* const* data, const uint64_t* lens, int n, void* work, uint64_t work_bytes,
                                     void* out, void* stream) {
  if (n <= 0) return 0;
  if (work_bytes < otb_tree_digest_batch_work(lens, n)) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  uint8_t* w = reinterpret_cast<uint8_t*>(work);
  // device tables at the front of `work`: src[n], dst[n], len[n], prefix[n+1], total[n]  (8 bytes each)
  const size_t tab_bytes = ((size_t)n * 5 + 1) * 8;
  uint64_t* dtab = reinterpret_cast<uint64_t*>(w);
  uint8_t* pool = w + ((tab_bytes + 255) & ~size_t(255));
  static thread_local uint64_t* htab = nullptr;
  static thread_local size_t htab_cap = 0;
  if (htab_cap < tab_bytes) {
    if (htab) cudaFreeHost(htab);
    if (cudaMallocHost(&htab, tab_bytes) != cudaSuccess) return -4;
    htab_cap = tab_bytes;
  }
  uint64_t* h_src = htab;
  uint64_t* h_dst = htab + n;
  uint64_t* h_len = htab + 2 * (size_t)n;
  uint64_t* h_pre = htab + 3 * (size_t)n;          // n+1
  uint64_t* h_tot = htab + 4 * (size_t)n + 1;
  for (int i = 0; i < n; ++i) { h_src[i] = reinterpret_cast<uint64_t>(data[i]); h_len[i] = lens[i]; h_tot[i] = lens[i]; }
  uint64_t pool_off = 0;
  for (;;) {
    uint64_t total_leaves = 0;
    for (int i = 0; i < n; ++i) {
      h_pre[i] = total_leaves;
      if (h_len[i] > OTB_TREE_LEAF) {
        const uint64_t leaves = (h_len[i] + OTB_TREE_LEAF - 1) / OTB_TREE_LEAF;
        h_dst[i] = reinterpret_cast<uint64_t>(pool + pool_off);
        pool_off += (leaves * 32 + 255) & ~uint64_t(255);
        total_leaves += leaves;
      } else {
        h_dst[i] = 0;
      }
    }
    h_pre[n] = total_leaves;
    if (total_leaves == 0) break;
    OTB_CUDA_CHECK_RET(cudaMemcpyAsync(dtab, htab, tab_bytes, cudaMemcpyHostToDevice, s));
    BatchLevel lv{reinterpret_cast<const uint8_t* const*>(dtab), dtab + 2 * (size_t)n, dtab + 3 * (size_t)n,
                  reinterpret_cast<uint8_t* const*>(dtab + n)};
    tree_level_batch_kernel<<<(unsigned)((total_leaves + 63) / 64), 64, 0, s>>>(lv, n, total_leaves);
    OTB_CUDA_CHECK_RET(cudaStreamSynchronize(s));  // the host table is rewritten for the next level
    for (int i = 0; i < n; ++i)
      if (h_len[i] > OTB_TREE_LEAF) {
        h_src[i] = h_dst[i];
        h_len[i] = ((h_len[i] + OTB_TREE_LEAF - 1) / OTB_TREE_LEAF) * 32;
      }
  }
  OTB_CUDA_CHECK_RET(cudaMemcpyAsync(dtab, htab, tab_bytes, cudaMemcpyHostToDevice, s));
  tree_final_batch_kernel<<<(n + 31) / 32, 32, 0, s>>>(reinterpret_cast<const uint8_t* const*>(dtab), dtab + 2 * (size_t)n,
                                                       dtab + 4 * (size_t)n + 1, n, reinterpret_cast<uint8_t*>(out));
  OTB_CUDA_CHECK_RET(cudaStreamSynchronize(s));
  return (int)cudaGetLastError();
}
