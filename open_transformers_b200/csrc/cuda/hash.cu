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
// Device version of the compression function with the twelve rounds written out, so the message words and the
// permutation are compile-time register choices (the shared host/device b2_compress indexes the message through the
// sigma table, which the device compiler can only do through local memory). Same function, same bytes.
#define B2D_G(a, b, c, d, x, y)                              \
  v[a] = v[a] + v[b] + (x); v[d] = b2_rotr(v[d] ^ v[a], 32); \
  v[c] = v[c] + v[d];       v[b] = b2_rotr(v[b] ^ v[c], 24); \
  v[a] = v[a] + v[b] + (y); v[d] = b2_rotr(v[d] ^ v[a], 16); \
  v[c] = v[c] + v[d];       v[b] = b2_rotr(v[b] ^ v[c], 63);
#define B2D_ROUND(s0, s1, s2, s3, s4, s5, s6, s7, s8, s9, s10, s11, s12, s13, s14, s15)  \
  B2D_G(0, 4, 8, 12, m[s0], m[s1]) B2D_G(1, 5, 9, 13, m[s2], m[s3])                      \
  B2D_G(2, 6, 10, 14, m[s4], m[s5]) B2D_G(3, 7, 11, 15, m[s6], m[s7])                    \
  B2D_G(0, 5, 10, 15, m[s8], m[s9]) B2D_G(1, 6, 11, 12, m[s10], m[s11])                  \
  B2D_G(2, 7, 8, 13, m[s12], m[s13]) B2D_G(3, 4, 9, 14, m[s14], m[s15])
__device__ __forceinline__ void b2d_compress(uint64_t (&h)[8], const uint64_t (&m)[16], uint64_t t, bool last) {
  uint64_t v[16];
  v[0] = h[0]; v[1] = h[1]; v[2] = h[2]; v[3] = h[3]; v[4] = h[4]; v[5] = h[5]; v[6] = h[6]; v[7] = h[7];
  v[8] = 0x6a09e667f3bcc908ULL; v[9] = 0xbb67ae8584caa73bULL; v[10] = 0x3c6ef372fe94f82bULL; v[11] = 0xa54ff53a5f1d36f1ULL;
  v[12] = 0x510e527fade682d1ULL ^ t; v[13] = 0x9b05688c2b3e6c1fULL;
  v[14] = last ? ~0x1f83d9abfb41bd6bULL : 0x1f83d9abfb41bd6bULL; v[15] = 0x5be0cd19137e2179ULL;
  B2D_ROUND(0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15)
  B2D_ROUND(14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3)
  B2D_ROUND(11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4)
  B2D_ROUND(7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8)
  B2D_ROUND(9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13)
  B2D_ROUND(2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9)
  B2D_ROUND(12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11)
  B2D_ROUND(13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10)
  B2D_ROUND(6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5)
  B2D_ROUND(10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0)
  B2D_ROUND(0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15)
  B2D_ROUND(14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3)
#pragma unroll
  for (int i = 0; i < 8; ++i) h[i] ^= v[i] ^ v[i + 8];
}
#undef B2D_ROUND
#undef B2D_G

// 32-byte digest of one leaf (len <= OTB_TREE_LEAF bytes at a 16-byte aligned address) into out (8-byte aligned).
// Whole 128-byte blocks come in as 16-byte loads; a ragged tail goes through the shared byte-wise routine.
__device__ __forceinline__ void leaf_digest(const uint8_t* __restrict__ data, uint64_t len, uint8_t* __restrict__ out) {
  if (len == 0 || (len & 127) != 0 || (reinterpret_cast<uintptr_t>(data) & 15) != 0) {
    uint8_t d[32];
    b2_hash(data, len, d, 32);
    for (int k = 0; k < 32; ++k) out[k] = d[k];
    return;
  }
  uint64_t h[8] = {0x6a09e667f3bcc908ULL ^ 0x01010020ULL, 0xbb67ae8584caa73bULL, 0x3c6ef372fe94f82bULL, 0xa54ff53a5f1d36f1ULL,
                   0x510e527fade682d1ULL, 0x9b05688c2b3e6c1fULL, 0x1f83d9abfb41bd6bULL, 0x5be0cd19137e2179ULL};
  const ulonglong2* src = reinterpret_cast<const ulonglong2*>(data);
  const uint64_t blocks = len >> 7;
#pragma unroll 1
  for (uint64_t blk = 0; blk < blocks; ++blk) {
    uint64_t m[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const ulonglong2 w = src[blk * 8 + i];
      m[2 * i] = w.x;
      m[2 * i + 1] = w.y;
    }
    b2d_compress(h, m, (blk + 1) << 7, blk + 1 == blocks);
  }
  uint64_t* o = reinterpret_cast<uint64_t*>(out);
  o[0] = h[0]; o[1] = h[1]; o[2] = h[2]; o[3] = h[3];
}

__global__ void tree_level_kernel(const uint8_t* __restrict__ data, uint64_t n, uint8_t* __restrict__ out, uint64_t leaves) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= leaves) return;
  const uint64_t off = i * OTB_TREE_LEAF;
  const uint64_t l = (n - off < OTB_TREE_LEAF) ? n - off : OTB_TREE_LEAF;
  leaf_digest(data + off, l, out + i * 32);
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
  leaf_digest(lv.src[lo] + off, l, lv.dst[lo] + leaf * 32);
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

// ---- planned variant: the level tables are built once, the launches never synchronise ----------------------------
// A plan covers n messages of fixed addresses and lengths (the state tensors of a training run never move). Table
// layout, 8-byte words, one block of (4n + 1) words per tree level: src[n] dst[n] len[n] prefix[n + 1]; then the final
// block: src[n] len[n] total[n]. otb_tree_plan fills the HOST copy of the table and the per-level leaf counts and
// returns the number of levels (or a negative error); the caller copies the table to the device once and then calls
// otb_tree_run on any stream, as often as it likes, with no host synchronisation inside.
extern "C" uint64_t otb_tree_plan_words(int n) { return (uint64_t)8 * (4 * (uint64_t)n + 1) + 3 * (uint64_t)n; }
extern "C" long otb_tree_plan(const void* const* data, const uint64_t* lens, int n, void* work, uint64_t work_bytes, uint64_t* tab,
                              uint64_t tab_words, uint64_t* level_leaves, int max_levels) {
  if (n <= 0) return 0;
  if (tab_words < otb_tree_plan_words(n) || max_levels > 8) return -2;
  uint64_t need = 0;
  for (int i = 0; i < n; ++i) need += otb_tree_digest_scratch(lens[i]);
  if (work_bytes < need) return -3;
  uint8_t* pool = reinterpret_cast<uint8_t*>(work);
  uint64_t pool_off = 0;
  const size_t blk = 4 * (size_t)n + 1;
  uint64_t* cur_src = new uint64_t[n];
  uint64_t* cur_len = new uint64_t[n];
  for (int i = 0; i < n; ++i) { cur_src[i] = reinterpret_cast<uint64_t>(data[i]); cur_len[i] = lens[i]; }
  int levels = 0;
  for (;;) {
    uint64_t total_leaves = 0;
    uint64_t* t = tab + (size_t)levels * blk;
    bool any = false;
    for (int i = 0; i < n; ++i) any = any || cur_len[i] > OTB_TREE_LEAF;
    if (!any) break;
    if (levels >= max_levels) { delete[] cur_src; delete[] cur_len; return -4; }
    for (int i = 0; i < n; ++i) {
      t[i] = cur_src[i];
      t[2 * (size_t)n + i] = cur_len[i];
      t[3 * (size_t)n + i] = total_leaves;
      if (cur_len[i] > OTB_TREE_LEAF) {
        const uint64_t leaves = (cur_len[i] + OTB_TREE_LEAF - 1) / OTB_TREE_LEAF;
        t[(size_t)n + i] = reinterpret_cast<uint64_t>(pool + pool_off);
        pool_off += (leaves * 32 + 255) & ~uint64_t(255);
        total_leaves += leaves;
      } else {
        t[(size_t)n + i] = 0;
        t[2 * (size_t)n + i] = 0;  // takes no part in this level (zero leaves)
      }
    }
    t[4 * (size_t)n] = total_leaves;
    level_leaves[levels] = total_leaves;
    for (int i = 0; i < n; ++i)
      if (cur_len[i] > OTB_TREE_LEAF) {
        cur_src[i] = t[(size_t)n + i];
        cur_len[i] = ((cur_len[i] + OTB_TREE_LEAF - 1) / OTB_TREE_LEAF) * 32;
      }
    ++levels;
  }
  uint64_t* f = tab + (size_t)levels * blk;
  for (int i = 0; i < n; ++i) { f[i] = cur_src[i]; f[(size_t)n + i] = cur_len[i]; f[2 * (size_t)n + i] = lens[i]; }
  delete[] cur_src;
  delete[] cur_len;
  return levels;
}
extern "C" int otb_tree_run(const uint64_t* tab_dev, int n, int levels, const uint64_t* level_leaves, void* out, void* stream) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const size_t blk = 4 * (size_t)n + 1;
  for (int l = 0; l < levels; ++l) {
    const uint64_t* t = tab_dev + (size_t)l * blk;
    BatchLevel lv{reinterpret_cast<const uint8_t* const*>(t), t + 2 * (size_t)n, t + 3 * (size_t)n,
                  reinterpret_cast<uint8_t* const*>(t + n)};
    tree_level_batch_kernel<<<(unsigned)((level_leaves[l] + 63) / 64), 64, 0, s>>>(lv, n, level_leaves[l]);
  }
  const uint64_t* f = tab_dev + (size_t)levels * blk;
  tree_final_batch_kernel<<<(n + 31) / 32, 32, 0, s>>>(reinterpret_cast<const uint8_t* const*>(f), f + n, f + 2 * (size_t)n, n,
                                                       reinterpret_cast<uint8_t*>(out));
  return (int)cudaGetLastError();
}
