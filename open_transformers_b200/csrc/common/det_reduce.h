// Canonical (fixed-order) reductions. The same association is used by the CUDA kernels and by
// the CPU twins, so a sum has the same bits on both.
//
//  lane_tree: element i of a row goes to "lane" (i / VW) % LANES; every lane folds its elements
//  in ascending i with one rounded operation per element; the LANES partials are then combined
//  by an XOR butterfly (offsets LANES/2, ..., 1), which is the tree
//      level 0: p[l] + p[l ^ LANES/2],  level 1: ... , down to offset 1.
//  A butterfly adds commutative pairs, so every lane ends with the same bits.
//
//  pair_tree: n values combined by the lower-index-left balanced tree with strides 1, 2, 4...:
//      for (s = 1; s < n; s *= 2) for (i = 0; i + s < n; i += 2 s) v[i] += v[i + s];
//  For n a power of two this is the perfect binary tree; any aligned power-of-two sub-range is a
//  sub-tree, which is what lets a token- or K-range be split over ranks without changing bits.
//  (Same shape as the reference's binary-blocks `tree_reduce_sum`,
//  src/pretrain/parallel/deterministic_reduce.py:162-186, for power-of-two counts.)
//
//  binary blocks (the fold over data-parallel replicas): n values are cut into power-of-two blocks, one per set bit of
//  n, largest first (7 = 4 + 2 + 1); a block is summed by the balanced lower-index-left tree; the block sums are added
//  left to right. In the strided form: a pair (i, i + s) is added at stride s only while its whole aligned group
//  [i, i + 2s) lies below n (then the group is inside one block), which leaves every block's sum at the block's first
//  index; the second pass adds those to v[0] in ascending order. Equal to pair_tree while n has at most two set bits.
//  `DET_BLOCKS_FOLD(n, ADD)` runs both passes; ADD(i, j) must perform v[i] = v[i] + v[j].
#pragma once
#include "det_math.h"

#define DET_BLOCKS_FOLD(n, ADD)                                               \
  do {                                                                        \
    const int det_n_ = (n);                                                   \
    for (int det_s_ = 1; 2 * det_s_ <= det_n_; det_s_ *= 2)                   \
      for (int det_i_ = 0; det_i_ + 2 * det_s_ <= det_n_; det_i_ += 2 * det_s_) { ADD(det_i_, det_i_ + det_s_); } \
    int det_top_ = 1;                                                         \
    while (2 * det_top_ <= det_n_) det_top_ *= 2;                             \
    for (int det_at_ = det_top_, det_rest_ = det_n_ - det_top_; det_rest_ > 0;) { \
      int det_b_ = 1;                                                         \
      while (2 * det_b_ <= det_rest_) det_b_ *= 2;                            \
      ADD(0, det_at_);                                                        \
      det_at_ += det_b_;                                                      \
      det_rest_ -= det_b_;                                                    \
    }                                                                         \
  } while (0)

#if !defined(__CUDACC__)
#include <vector>
// Host model of the butterfly over `lanes` partials (lanes a power of two).
inline float det_butterfly_host(float* p, int lanes) {
  for (int off = lanes / 2; off >= 1; off >>= 1) {
    for (int l = 0; l < lanes; ++l) {
      if ((l & off) == 0) {
        const float s = p[l] + p[l ^ off];
        p[l] = s;
        p[l ^ off] = s;
      }
    }
  }
  return p[0];
}
inline void det_pair_tree_host(float* v, long n, long stride_elems = 1) {
  for (long s = 1; s < n; s *= 2)
    for (long i = 0; i + s < n; i += 2 * s) v[i * stride_elems] = v[i * stride_elems] + v[(i + s) * stride_elems];
}
inline double det_pair_tree_host_d(double* v, long n) {
  for (long s = 1; s < n; s *= 2)
    for (long i = 0; i + s < n; i += 2 * s) v[i] = v[i] + v[i + s];
  return n > 0 ? v[0] : 0.0;
}
#endif
