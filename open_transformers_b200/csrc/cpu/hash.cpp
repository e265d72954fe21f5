// Host BLAKE2b: one-shot digest and the parallel tree digest used for large tensors.
#include <stdint.h>
#include <string.h>

#include <vector>

#include "blake2b.h"

extern "C" {

void otb_cpu_blake2b(const uint8_t* data, uint64_t len, uint8_t* out, int outlen) {
  if (len >= 128 && (reinterpret_cast<uintptr_t>(data) & 7)) {
    std::vector<uint64_t> tmp((len + 7) / 8);
    memcpy(tmp.data(), data, len);
    b2_hash(reinterpret_cast<const uint8_t*>(tmp.data()), len, out, outlen);
  } else {
    b2_hash(data, len, out, outlen);
  }
}

// 32-byte tree digest (see blake2b.h). `data` 8-byte aligned.
void otb_cpu_tree_digest(const uint8_t* data, uint64_t len, uint8_t* out32) {
  std::vector<uint8_t> cur, next;
  const uint8_t* p = data;
  uint64_t n = len;
  while (n > OTB_TREE_LEAF) {
    const uint64_t leaves = (n + OTB_TREE_LEAF - 1) / OTB_TREE_LEAF;
    next.assign(leaves * 32, 0);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)leaves; ++i) {
      const uint64_t off = (uint64_t)i * OTB_TREE_LEAF;
      const uint64_t l = (n - off < OTB_TREE_LEAF) ? n - off : OTB_TREE_LEAF;
      b2_hash(p + off, l, next.data() + i * 32, 32);
    }
    cur.swap(next);
    p = cur.data();
    n = cur.size();
  }
  std::vector<uint64_t> fin((n + 8 + 7) / 8 + 1, 0);
  memcpy(fin.data(), p, n);
  uint64_t le = len;
  memcpy(reinterpret_cast<uint8_t*>(fin.data()) + n, &le, 8);
  b2_hash(reinterpret_cast<const uint8_t*>(fin.data()), n + 8, out32, 32);
}
}
