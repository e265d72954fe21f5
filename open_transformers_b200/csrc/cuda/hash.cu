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
