// BLAKE2b (RFC 7693), unkeyed, variable digest length; compiles for host and device.
// `tree digest` of a byte string: split into 4096-byte leaves, hash each to 32 bytes, concatenate,
// repeat until at most 4096 bytes remain, then hash those bytes followed by the original length as
// 8 little-endian bytes. Leaves are independent, so a GPU hashes them in parallel.
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define B2_HD __host__ __device__ __forceinline__
#else
#define B2_HD inline
#endif

#define OTB_TREE_LEAF 4096

B2_HD uint64_t b2_rotr(uint64_t x, int n) { return (x >> n) | (x << (64 - n)); }

B2_HD void b2_compress(uint64_t* h, const uint64_t* m, uint64_t t, bool last) {
  const uint64_t iv[8] = {0x6a09e667f3bcc908ULL, 0xbb67ae8584caa73bULL, 0x3c6ef372fe94f82bULL, 0xa54ff53a5f1d36f1ULL,
                          0x510e527fade682d1ULL, 0x9b05688c2b3e6c1fULL, 0x1f83d9abfb41bd6bULL, 0x5be0cd19137e2179ULL};
  const uint8_t sigma[12][16] = {
      {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15}, {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3},
      {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4}, {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8},
      {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13}, {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9},
      {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11}, {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10},
      {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5}, {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0},
      {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15}, {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3}};
  uint64_t v[16];
  for (int i = 0; i < 8; ++i) { v[i] = h[i]; v[i + 8] = iv[i]; }
  v[12] ^= t;
  if (last) v[14] = ~v[14];
#define B2_G(a, b, c, d, x, y)                \
  v[a] = v[a] + v[b] + (x); v[d] = b2_rotr(v[d] ^ v[a], 32); \
  v[c] = v[c] + v[d];       v[b] = b2_rotr(v[b] ^ v[c], 24); \
  v[a] = v[a] + v[b] + (y); v[d] = b2_rotr(v[d] ^ v[a], 16); \
  v[c] = v[c] + v[d];       v[b] = b2_rotr(v[b] ^ v[c], 63);
#if defined(__CUDA_ARCH__)
#pragma unroll 1
#endif
  for (int r = 0; r < 12; ++r) {
    const uint8_t* s = sigma[r];
    B2_G(0, 4, 8, 12, m[s[0]], m[s[1]]) B2_G(1, 5, 9, 13, m[s[2]], m[s[3]])
    B2_G(2, 6, 10, 14, m[s[4]], m[s[5]]) B2_G(3, 7, 11, 15, m[s[6]], m[s[7]])
    B2_G(0, 5, 10, 15, m[s[8]], m[s[9]]) B2_G(1, 6, 11, 12, m[s[10]], m[s[11]])
    B2_G(2, 7, 8, 13, m[s[12]], m[s[13]]) B2_G(3, 4, 9, 14, m[s[14]], m[s[15]])
  }
#undef B2_G
  for (int i = 0; i < 8; ++i) h[i] ^= v[i] ^ v[i + 8];
}

// One-shot hash of `len` bytes at `data` (8-byte aligned when len >= 128) into out[outlen], outlen <= 64.
B2_HD void b2_hash(const uint8_t* data, uint64_t len, uint8_t* out, int outlen) {
  uint64_t h[8] = {0x6a09e667f3bcc908ULL, 0xbb67ae8584caa73bULL, 0x3c6ef372fe94f82bULL, 0xa54ff53a5f1d36f1ULL,
                   0x510e527fade682d1ULL, 0x9b05688c2b3e6c1fULL, 0x1f83d9abfb41bd6bULL, 0x5be0cd19137e2179ULL};
  h[0] ^= 0x01010000ULL ^ (uint64_t)outlen;
  uint64_t off = 0;
  uint64_t m[16];
  while (len - off > 128) {
    const uint64_t* src = reinterpret_cast<const uint64_t*>(data + off);
    for (int i = 0; i < 16; ++i) m[i] = src[i];
    off += 128;
    b2_compress(h, m, off, false);
  }
  uint8_t* mb = reinterpret_cast<uint8_t*>(m);
  for (int i = 0; i < 16; ++i) m[i] = 0;
  for (uint64_t i = 0; i < len - off; ++i) mb[i] = data[off + i];
  b2_compress(h, m, len, true);
  const uint8_t* hb = reinterpret_cast<const uint8_t*>(h);
  for (int i = 0; i < outlen; ++i) out[i] = hb[i];
}
