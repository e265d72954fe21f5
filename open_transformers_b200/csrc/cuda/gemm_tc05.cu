// Persistent, warp-specialised bf16 GEMM for sm_100a:  C[M,N] = op(A) * op(B)^T (+ epilogue)
//
//   * operands are staged by TMA (cp.async.bulk.tensor, 128-byte swizzle; each CTA fetches its own tiles)
//     into a STAGES-deep shared-memory ring,
//   * one elected thread issues tcgen05.mma (M=128, N=BN, K=16 per instruction) with the
//     fp32 accumulator in tensor memory, double-buffered so the epilogue of tile i overlaps
//     the main loop of tile i+1,
//   * four epilogue warps read the accumulator with tcgen05.ld (one row per thread), convert it,
//     stage 32-row x 128-byte slices in swizzled shared memory and hand them to TMA
//     (cp.async.bulk.tensor store; cp.reduce.async.bulk.tensor .add for the fp32 accumulate
//     epilogue, one add per element, so still a fixed order).
//
// Reduction order (the hashed contract): every output element is the tensor-core fp32
// accumulation of its K products taken in ascending k, 16 at a time, with NO split-K and no
// atomics, so the result does not depend on the grid, the tile schedule or the GPU count.
//
// Operand majorness: "K-major" means the reduction index is the contiguous one
// (A given as [M,K] row-major, B given as [N,K] row-major); "MN-major" means the operand is
// stored transposed ([K,M] / [K,N] row-major). The three training GEMMs are
//   forward  y  = x W^T         A K-major , B K-major
//   dgrad    dx = dy W          A K-major , B MN-major
//   wgrad    dW = dy^T x        A MN-major, B MN-major
//
// The same kernel runs the W8A8 forward of the quantisation-aware layers (I8 = true): int8 operands, both K-major,
// tcgen05.mma kind::i8 (K = 32 per instruction, 128 int8 = one swizzle row per k-block), exact int32 accumulation
// in tensor memory, and an epilogue that dequantises  float(acc) * (sa[0] * sb[col])  before the usual stores.
//
// Role of this file in the reference's terms: the `repop.nn.linear` / `mmacc` entry points
// (reference docs/MODEL_OP_DTYPE_TRACE.md:82,100).
#include "tc05.cuh"
#include "common.cuh"

using namespace tc05;

namespace {

constexpr int BM = 128;
constexpr int BK_BYTES = 128;  // one 128-byte swizzle row per k-block: 64 bf16 or 128 int8
constexpr int UMMA_K_BYTES = 32;  // one MMA consumes 32 bytes of K: 16 bf16 or 32 int8
constexpr int NUM_THREADS = 192;  // warp0: TMA, warp1: MMA, warps 2..5: epilogue

enum Epi : int {
  EPI_BF16 = 0,      // C(bf16)  = acc
  EPI_F32 = 1,       // C(fp32)  = acc
  EPI_F32_ACC = 2,   // C(fp32) += acc
  EPI_BF16_RES = 3,  // C(bf16)  = bf16(acc + float(R))
};

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK_BYTES;
  static constexpr int B_BYTES = BN * BK_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;       // 4 warps x 2 buffers x [32 rows][128 B]
  static constexpr int EPI_BYTES = 4 * 2 * 4096;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // + barriers + alignment slack
};

template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI, bool I8>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, void* __restrict__ Cv,
                 const __nv_bfloat16* __restrict__ R, int M, int N, int K, long ldc, long ldr, int group_m,
                 const float* __restrict__ scale_a, const float* __restrict__ scale_b, uint32_t* __restrict__ status) {
  static_assert(!I8 || (!A_MN && !B_MN), "the int8 path takes K-major operands only");
  constexpr int BK = I8 ? BK_BYTES : BK_BYTES / 2;  // elements of K per k-block
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;  // [2]
  uint64_t* tempty_bar = tfull_bar + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN >= 512 ? 512 : (2 * BN <= 32 ? 32 : 2 * BN);

  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);  // one arrive per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (m, n): groups of `group_m` row-tiles sweep all column tiles, so that the A rows of
  // a group and the B columns being swept stay L2-resident across the CTAs working on them.
  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int per_group = group_m * tiles_n;
    const int g = t / per_group;
    const int first_m = g * group_m;
    const int gsz = min(group_m, tiles_m - first_m);
    const int r = t - g * per_group;
    tm = first_m + r % gsz;
    tn = r / gsz;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coord(t, tm, tn);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(sa, &tmA, &full_bar[s], kb * BK, tm * BM);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * 8192, &tmA, &full_bar[s], tm * BM + c * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmB, &full_bar[s], kb * BK, tn * BN);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * 8192, &tmB, &full_bar[s], tn * BN + c * 64, kb * BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = I8 ? make_idesc(BM, BN, 0, 0, 2, 1) : make_idesc(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++lt) {
        const uint32_t buf = lt & 1;
        const uint32_t bph = (lt >> 1) & 1;
        if (!mbar_wait(&tempty_bar[buf], bph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK_BYTES / UMMA_K_BYTES; ++kk) {
            const uint64_t ad = A_MN ? make_smem_desc(sa + kk * 2048, 8192, 1024) : make_smem_desc(sa + kk * 32, 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(sb + kk * 2048, 8192, 1024) : make_smem_desc(sb + kk * 32, 16, 1024);
            if (I8) mma_i8_ss(d_tmem, ad, bd, idesc, (kb | kk) != 0);
            else mma_f16_ss(d_tmem, ad, bd, idesc, (kb | kk) != 0);
          }
          mma_commit(&empty_bar[s]);  // smem stage reusable once these MMAs have read it
        }
        if (ok) mma_commit(&tfull_bar[buf]);  // accumulator complete
      }
    }
  } else {
    // --------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may touch
    uint32_t lt = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++lt) {
      int tm, tn;
      tile_coord(t, tm, tn);
      const uint32_t buf = lt & 1;
      const uint32_t bph = (lt >> 1) & 1;
      if (!mbar_wait(&tfull_bar[buf], bph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const long row = (long)tm * BM + q * 32 + lane;
      const int col0 = tn * BN;
      // Software pipeline over 32-column chunks with two register buffers: the TMEM load of the next chunk is
      // in flight while the current one is converted and written to this warp's staging slice
      // ([32 rows][128 B], 128-byte swizzle = 64 bf16 or 32 fp32 columns), which TMA then stores.
      const uint32_t tbase = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
      uint8_t* stage0 = smem + L::EPI_OFFSET + q * 8192;
      constexpr bool OUT_BF16 = (EPI == EPI_BF16 || EPI == EPI_BF16_RES);
      constexpr int COLS_PER_SLICE = OUT_BF16 ? 64 : 32;
      auto emit_slice = [&](int slice, int col) {
        // staging writes (generic proxy) -> visible to TMA (async proxy), then one elected lane issues the store
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const uint32_t src = smem_u32(stage0 + (slice & 1) * 4096);
          const int y = tm * BM + q * 32;
          if (EPI == EPI_F32_ACC) {
            asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                             reinterpret_cast<uint64_t>(&tmC)),
                         "r"(src), "r"(col), "r"(y)
                         : "memory");
          } else {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                             reinterpret_cast<uint64_t>(&tmC)),
                         "r"(src), "r"(col), "r"(y)
                         : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      };
      auto slice_free = [&]() {
        // the slice written two stores ago has been read by TMA
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        __syncwarp();
      };
      int slice = 0;
      const float sa0 = I8 ? scale_a[0] : 0.0f;
      auto store_chunk = [&](uint32_t (&v)[32], int c) {
        const int col = col0 + c;
        if (I8) {
          // dequantise: the int32 sum is exact; float(acc) rounds once, then one multiply by sa * sb[col]
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float sb = col + j < N ? __ldg(scale_b + col + j) : 0.0f;
            v[j] = __float_as_uint(__fmul_rn(__int2float_rn((int)v[j]), __fmul_rn(sa0, sb)));
          }
        }
        if (OUT_BF16) {
          const int part = (c >> 5) & 1;  // which 64-byte half of the 128-byte staging row
          if (part == 0) slice_free();
          uint8_t* st = stage0 + (slice & 1) * 4096;
          uint32_t p[16];
          if (EPI == EPI_BF16_RES) {
            if (row < M && col + 32 <= N) {
              const uint4* rr = reinterpret_cast<const uint4*>(R + row * ldr + col);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint4 r4 = rr[j];
                const uint32_t rw[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float r0 = __uint_as_float(rw[e] << 16);
                  const float r1 = __uint_as_float(rw[e] & 0xFFFF0000u);
                  p[j * 4 + e] = pack_bf16(__fadd_rn(__uint_as_float(v[j * 8 + e * 2]), r0),
                                           __fadd_rn(__uint_as_float(v[j * 8 + e * 2 + 1]), r1));
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float x0 = __uint_as_float(v[2 * j]), x1 = __uint_as_float(v[2 * j + 1]);
                if (row < M && col + 2 * j < N) x0 = __fadd_rn(x0, __bfloat162float(R[row * ldr + col + 2 * j]));
                if (row < M && col + 2 * j + 1 < N) x1 = __fadd_rn(x1, __bfloat162float(R[row * ldr + col + 2 * j + 1]));
                p[j] = pack_bf16(x0, x1);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) p[j] = pack_bf16(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(st + lane * 128 + (((part * 4 + j) ^ (lane & 7)) << 4)) =
                make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
          if (part == 1) {
            emit_slice(slice, col - 32);
            ++slice;
          }
        } else {
          slice_free();
          uint8_t* st = stage0 + (slice & 1) * 4096;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(st + lane * 128 + ((j ^ (lane & 7)) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          emit_slice(slice, col);
          ++slice;
        }
      };
      uint32_t va[32], vb[32];
      tmem_ld_32x32b_x32(tbase, va);
      tmem_ld_wait();
#pragma unroll 1
      for (int c = 0; c < BN; c += 64) {
        tmem_ld_32x32b_x32(tbase + c + 32, vb);
        store_chunk(va, c);
        tmem_ld_wait();
        if (c + 64 < BN) tmem_ld_32x32b_x32(tbase + c + 64, va);
        store_chunk(vb, c + 32);
        tmem_ld_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every TMA store of this warp has completed
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && status) atomicExch(status, 1u);  // a bounded wait ran out
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
struct TmapKey {
  const void* ptr;
  uint64_t d0, d1, ld;
  uint32_t b0, b1;
};

// elem_bytes: 2 bf16, 4 fp32, 1 int8 (moved as bytes)
CUresult encode_2d(CUtensorMap* out, const void* ptr, uint64_t dim0, uint64_t dim1, uint64_t ld_elems, uint32_t box0,
                   uint32_t box1, int elem_bytes = 2) {
  static PFN_encodeTiled fn = get_encode_tiled();
  if (!fn) return CUDA_ERROR_NOT_SUPPORTED;
  cuuint64_t dims[2] = {dim0, dim1};
  cuuint64_t strides[1] = {ld_elems * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  return fn(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI, bool I8 = false>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, void* C, const void* R, int M, int N, int K, long ldc, long ldr,
           uint32_t* status, int max_ctas, cudaStream_t stream, const float* scale_a = nullptr, const float* scale_b = nullptr) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = gemm_tc05_kernel<BN, STAGES, A_MN, B_MN, EPI, I8>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = tiles < max_ctas ? tiles : max_ctas;
  if (grid < 1) grid = 1;
  const int group_m = 8;
  kern<<<grid, NUM_THREADS, L::TOTAL, stream>>>(ta, tb, tc, C, reinterpret_cast<const __nv_bfloat16*>(R), M, N, K, ldc, ldr,
                                                group_m, scale_a, scale_b, status);
  return (int)cudaGetLastError();
}

template <int BN, int STAGES, int EPI>
int launch_major(int a_mn, int b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, void* C, const void* R, int M, int N,
                 int K, long ldc, long ldr, uint32_t* status, int max_ctas, cudaStream_t s) {
  if (!a_mn && !b_mn) return launch<BN, STAGES, false, false, EPI>(ta, tb, tc, C, R, M, N, K, ldc, ldr, status, max_ctas, s);
  if (!a_mn && b_mn) return launch<BN, STAGES, false, true, EPI>(ta, tb, tc, C, R, M, N, K, ldc, ldr, status, max_ctas, s);
  if (a_mn && b_mn) return launch<BN, STAGES, true, true, EPI>(ta, tb, tc, C, R, M, N, K, ldc, ldr, status, max_ctas, s);
  return launch<BN, STAGES, true, false, EPI>(ta, tb, tc, C, R, M, N, K, ldc, ldr, status, max_ctas, s);
}

}  // namespace

// C[M,N] = op(A) op(B)^T with bf16 operands and fp32 tensor-core accumulation.
//   a_mn = 0: A is [M,K] row-major with leading dimension lda;  a_mn = 1: A is [K,M] row-major.
//   b_mn = 0: B is [N,K] row-major with leading dimension ldb;  b_mn = 1: B is [K,N] row-major.
//   epi: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate into C, 3 bf16 store of acc + R (bf16 residual, ldr).
// Leading dimensions are in elements and must be multiples of 8 (16-byte TMA strides); all base
// pointers 16-byte aligned. `status` (device word, may be null) is set to 1 if a bounded wait gave up.
// Returns 0 or a CUDA/driver error code; never allocates.
extern "C" int otb_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K, long lda,
                             long ldb, long ldc, long ldr, int a_mn, int b_mn, int epi, uint32_t* status,
                             int max_ctas, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  const bool bf16_out = (epi == EPI_BF16 || epi == EPI_BF16_RES);
  if ((bf16_out && (ldc & 7)) || (!bf16_out && (ldc & 3)) || (epi == EPI_BF16_RES && (ldr & 7))) return -2;
  if (max_ctas <= 0) max_ctas = otb_sm_count();
  // Tile width: the 256-wide tile is the more efficient one per tile; the 128-wide one wins when
  // it fills the last wave of CTAs noticeably better.
  int BN = 128;
  if (N >= 256) {
    const long t256 = (long)((M + 127) / 128) * ((N + 255) / 256);
    const long t128 = (long)((M + 127) / 128) * ((N + 127) / 128);
    const double e256 = (double)t256 / (double)(((t256 + max_ctas - 1) / max_ctas) * max_ctas) *
                        ((double)N / (double)(((N + 255) / 256) * 256));
    const double e128 = 0.88 * (double)t128 / (double)(((t128 + max_ctas - 1) / max_ctas) * max_ctas) *
                        ((double)N / (double)(((N + 127) / 128) * 128));
    BN = e256 >= e128 ? 256 : 128;
  }
  CUtensorMap ta, tb;
  CUresult r;
  constexpr int BK = BK_BYTES / 2;
  r = a_mn ? encode_2d(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK)
           : encode_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = b_mn ? encode_2d(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK)
           : encode_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, (uint32_t)BN);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  CUtensorMap tc;
  r = bf16_out ? encode_2d(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 64, 32, 2)
               : encode_2d(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 32, 32, 4);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  if (reinterpret_cast<uintptr_t>(C) & 15) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define OTB_DISPATCH(BN_, ST_)                                                                                      \
  switch (epi) {                                                                                                    \
    case EPI_BF16: return launch_major<BN_, ST_, EPI_BF16>(a_mn, b_mn, ta, tb, tc, C, R, M, N, K, ldc, ldr, status, max_ctas, s); \
    case EPI_F32: return launch_major<BN_, ST_, EPI_F32>(a_mn, b_mn, ta, tb, tc, C, R, M, N, K, ldc, ldr, status, max_ctas, s);   \
    case EPI_F32_ACC: return launch_major<BN_, ST_, EPI_F32_ACC>(a_mn, b_mn, ta, tb, tc, C, R, M, N, K, ldc, ldr, status, max_ctas, s); \
    case EPI_BF16_RES: return launch_major<BN_, ST_, EPI_BF16_RES>(a_mn, b_mn, ta, tb, tc, C, R, M, N, K, ldc, ldr, status, max_ctas, s); \
    default: return -3;                                                                                             \
  }
  if (BN == 256) {
    OTB_DISPATCH(256, 4)
  } else {
    OTB_DISPATCH(128, 6)
  }
#undef OTB_DISPATCH
}

// W8A8 forward of a quantised linear layer:  C[M,N] = dequant( A_q[M,K] * B_q[N,K]^T ),  int8 operands (K-major,
// leading dimensions multiples of 16), exact int32 accumulation on the tensor cores, then
//   C = float(acc) * (scale_a[0] * scale_b[n])        (+ bf16 residual R for epi 3)
// scale_a: one device float (per-tensor activation step); scale_b: N device floats (per-channel weight step).
// epi: 0 bf16 store, 1 fp32 store, 3 bf16 store with residual. Never allocates.
extern "C" int otb_gemm_i8(const void* A, const void* B, void* C, const void* R, int M, int N, int K, long lda, long ldb,
                           long ldc, long ldr, const float* scale_a, const float* scale_b, int epi, uint32_t* status,
                           int max_ctas, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 15) || (ldb & 15) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15))
    return -2;
  if (epi != EPI_BF16 && epi != EPI_F32 && epi != EPI_BF16_RES) return -3;
  const bool bf16_out = epi != EPI_F32;
  if ((bf16_out && (ldc & 7)) || (!bf16_out && (ldc & 3)) || (epi == EPI_BF16_RES && (ldr & 7))) return -2;
  if (!scale_a || !scale_b) return -2;
  if (max_ctas <= 0) max_ctas = otb_sm_count();
  const int BN = N > 128 ? 256 : 128;
  CUtensorMap ta, tb, tc;
  CUresult r = encode_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK_BYTES, BM, 1);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = encode_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK_BYTES, (uint32_t)BN, 1);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = bf16_out ? encode_2d(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 64, 32, 2)
               : encode_2d(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 32, 32, 4);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define OTB_I8(BN_, ST_, EPI_) \
  return launch<BN_, ST_, false, false, EPI_, true>(ta, tb, tc, C, R, M, N, K, ldc, ldr, status, max_ctas, s, scale_a, scale_b);
  if (BN == 256) {
    if (epi == EPI_BF16) { OTB_I8(256, 4, EPI_BF16) }
    if (epi == EPI_F32) { OTB_I8(256, 4, EPI_F32) }
    OTB_I8(256, 4, EPI_BF16_RES)
  } else {
    if (epi == EPI_BF16) { OTB_I8(128, 6, EPI_BF16) }
    if (epi == EPI_F32) { OTB_I8(128, 6, EPI_F32) }
    OTB_I8(128, 6, EPI_BF16_RES)
  }
#undef OTB_I8
}
