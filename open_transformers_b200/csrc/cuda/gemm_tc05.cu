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
// Tensor-parallel variants (TP template parameter), each ONE kernel that moves data over NVLink peer pointers
// while the tensor cores work, with no library collective involved:
//   TP = 1  all-gather -> GEMM.  The A operand is token-sharded over P ranks. A few extra CTAs of the same launch
//           push this rank's rows into every peer's full-size A buffer (plain 16-byte peer stores) and then set a
//           per-128-row flag on that peer; the GEMM CTAs start with the rows that are already local and, before
//           the TMA loads of a row block owned by a peer, wait (bounded) for that block's flag.
//   TP = 2  GEMM -> ordered reduction over ranks (row-parallel layer: K is split over the P ranks). The partial
//           sums are NOT added after the fact: rank r receives the fp32 accumulator tile of rank r-1 in its inbox,
//           loads it into tensor memory (tcgen05.st), continues the SAME ascending-k accumulation chain over its own
//           K slice, and TMA-stores the tile into rank r+1's inbox (the last rank: into the buffer of the rank that
//           owns those rows) followed by a release flag per 32-row quarter. The result is therefore bit-identical
//           to the unsplit GEMM on one GPU, and ranks work on different tiles at the same time (a pipeline).
// Every wait on a peer is bounded (two seconds of %globaltimer); when it runs out the kernel raises the abort
// flag, drains its own copies, frees its tensor memory and reports through the status word.
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

struct TpNone {};
struct TpArgs {
  CUtensorMap tmOut[8];        // TP 2: [0] = next rank's inbox, or (last rank) the fp32 result buffer of each row owner
  uint32_t* flags_out[8];      // TP 2: flag arrays matching tmOut
  const float* inbox;          // TP 2: this rank's inbox (fp32 [M, ld_in]) and its flags [tiles * 4]
  const uint32_t* flags_in;    // TP 1: this rank's row-block flags [P * tiles_per_shard]
  long ld_in;
  const uint4* ag_src;         // TP 1: this rank's own rows inside its full-size A buffer
  uint4* ag_dst[8];            // TP 1: the same rows inside every peer's A buffer (null for this rank)
  uint32_t* ag_flags[8];       // TP 1: every peer's row-block flags
  long ag_block_u4;            // 16-byte units per 128-row block
  uint32_t seq;                // value a flag takes when its data of THIS call has landed
  int rank, P, tiles_per_shard, gemm_ctas;
  // TP 3 (parameter gather): B [N,K] is a weight whose rows are spread over the P processes. Every process keeps a
  // full-size buffer of the same layout in which only its own rows are current; the rows of the others are pulled
  // from their buffers (plain peer loads) into the local one by four extra warps of the GEMM's own CTAs.
  const uint4* pg_src[8];      // row 0 of this weight in every process's buffer ([rank] is the local buffer)
  uint4* pg_dst;               // row 0 of this weight in the local buffer (what tmB reads)
  uint32_t* pg_flags;          // local counters: word [tn] counts the copy units of B tile tn (BN rows) that have landed,
                               // word [tiles_n] all units of the weight; they only grow: after call number `seq` of this
                               // weight a complete tile reads seq x (its units)
  int pg_seg_begin[4];         // B is up to 3 row-concatenated parameters: first row of each, then N
  int pg_rows_per_owner[3];    // rows of parameter j per process (process p holds rows [p*rpo, (p+1)*rpo) of it)
  int pg_nseg, pg_rot;         // number of parameters; B tile the tile order starts from (this process's rows first)
  int pg_unit_rows;            // rows per copy unit (divides 128): small weights are cut finer so that every CTA copies
  int pg_row_u4, pg_ld_u4;     // 16-byte units per row that are copied / between rows
};

// Which process holds row `row` of a gathered weight.
__device__ __forceinline__ int pg_owner(const TpArgs& tp, int row) {
  int j = 0;
  if (tp.pg_nseg > 1 && row >= tp.pg_seg_begin[1]) j = 1;
  if (tp.pg_nseg > 2 && row >= tp.pg_seg_begin[2]) j = 2;
  const int o = (row - tp.pg_seg_begin[j]) / tp.pg_rows_per_owner[j];
  return o < tp.P ? o : tp.P - 1;
}

// Launch-order permutation for the race tests: CTA b works as CTA (b + g_cta_rotation) mod (number of GEMM CTAs). Every
// output tile is owned by one CTA and summed in ascending k whatever CTA that is, so any rotation must give the same bytes
// (otb_set_cta_rotation; 0 in production).
__device__ int g_cta_rotation = 0;

// How long a kernel of this file waits for a peer's flag before it gives up, sets its status word and returns
// (nanoseconds of %globaltimer; otb_set_peer_wait_ns changes it for the current device).
__device__ unsigned long long g_peer_wait_ns = 2000000000ull;

// Counter words of the parameter gather: relaxed/acquire at GPU scope (copiers and consumers are CTAs of one launch).
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_count(const uint32_t* word, uint32_t target, volatile uint32_t* abort_flag) {
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t i = 0;; ++i) {
    if (ld_acquire_gpu(word) == target) return true;
    if (*abort_flag) return false;
    if ((i & 63u) == 63u) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > g_peer_wait_ns) break;
    }
    __nanosleep(100);
  }
  *abort_flag = 1;
  return false;
}

// Bounded wait for a flag written by a peer GPU (release at system scope on their side).
__device__ __forceinline__ bool wait_peer_flag(const uint32_t* flag, uint32_t seq, volatile uint32_t* abort_flag) {
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t i = 0;; ++i) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v == seq) return true;
    if (*abort_flag) return false;
    if ((i & 63u) == 63u) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > g_peer_wait_ns) break;
    }
    __nanosleep(100);
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void release_peer_flag(uint32_t* flag, uint32_t seq) {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(seq) : "memory");
}

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

template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI, bool I8, int TP, typename TPA>
__global__ void __launch_bounds__(TP >= 2 ? NUM_THREADS + 128 : NUM_THREADS, 1)
gemm_tc05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, void* __restrict__ Cv,
                 const __nv_bfloat16* __restrict__ R, int M, int N, int K, long ldc, long ldr, int group_m,
                 const float* __restrict__ scale_a, const float* __restrict__ scale_b, uint32_t* __restrict__ status,
                 const __grid_constant__ TPA tp) {
  static_assert(!I8 || (!A_MN && !B_MN), "the int8 path takes K-major operands only");
  static_assert(TP == 0 || !I8, "the tensor-parallel variants are bf16");
  static_assert(TP != 2 || EPI == EPI_F32, "the chained GEMM hands fp32 accumulator tiles on");
  int nctas = gridDim.x;
  if constexpr (TP == 1) {
    nctas = tp.gemm_ctas;
    if ((int)blockIdx.x >= nctas) {
      // ---------------------------------------------------- all-gather pusher CTAs (no tensor cores, no barriers)
      const int copiers = gridDim.x - nctas;
      for (int blk = blockIdx.x - nctas; blk < tp.tiles_per_shard; blk += copiers) {
        const uint4* src = tp.ag_src + (long)blk * tp.ag_block_u4;
        for (int p = 0; p < tp.P; ++p) {
          if (p == tp.rank) continue;
          uint4* dst = tp.ag_dst[p] + (long)blk * tp.ag_block_u4;
          // 16 independent 16-byte loads per thread in flight (48 KB per CTA), then the peer stores
          for (long i = threadIdx.x; i < tp.ag_block_u4; i += 16 * blockDim.x) {
            uint4 v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u)
              if (i + u * blockDim.x < tp.ag_block_u4) v[u] = __ldg(src + i + u * blockDim.x);
#pragma unroll
            for (int u = 0; u < 16; ++u)
              if (i + u * blockDim.x < tp.ag_block_u4) dst[i + u * blockDim.x] = v[u];
          }
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < tp.P && (int)threadIdx.x != tp.rank)
          release_peer_flag(tp.ag_flags[threadIdx.x] + tp.rank * tp.tiles_per_shard + blk, tp.seq);
        __syncthreads();
      }
      return;
    }
  }
  constexpr int BK = I8 ? BK_BYTES : BK_BYTES / 2;  // elements of K per k-block
  const int cta = ((int)blockIdx.x + g_cta_rotation) % nctas;  // which persistent worker this CTA is
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;  // [2]
  uint64_t* tempty_bar = tfull_bar + 2;      // [2]
  uint64_t* tloaded_bar = tempty_bar + 2;    // [2] (chained GEMM: incoming accumulator is in tensor memory)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tloaded_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  bool chain_in = false;
  if constexpr (TP == 2) chain_in = tp.rank > 0;

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
      mbar_init(&tloaded_bar[b], 4);  // one arrive per accumulator-loading warp
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
    if constexpr (TP == 1) tm = (tm + tp.rank * tp.tiles_per_shard) % tiles_m;  // own rows first, then the peers' in ring order
    if constexpr (TP == 3) tn = (tn + tp.pg_rot) % tiles_n;                        // weight rows of this process first
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      [[maybe_unused]] bool pg_all = false;
      for (int t = cta; t < num_tiles && ok; t += nctas) {
        int tm, tn;
        tile_coord(t, tm, tn);
        if constexpr (TP == 1) {
          const int owner = tm / tp.tiles_per_shard;
          if (owner != tp.rank) {
            if (!wait_peer_flag(tp.flags_in + owner * tp.tiles_per_shard + tm % tp.tiles_per_shard, tp.seq, abort_flag)) { ok = false; break; }
            asm volatile("fence.proxy.async;" ::: "memory");  // the peer's generic stores, then our TMA (async proxy) reads
          }
        }
        if constexpr (TP == 3) {
          // the rows of this B tile must be complete in the local buffer. Until the whole weight has arrived that is one
          // look at the weight's counter and, if it is not there yet, a wait for the tile's own counter; afterwards nothing.
          if (!pg_all) {
            const int units_row = (N + tp.pg_unit_rows - 1) / tp.pg_unit_rows;
            if (ld_acquire_gpu(tp.pg_flags + tiles_n) == tp.seq * (uint32_t)units_row) {
              pg_all = true;
            } else {
              const int rows_here = min(BN, N - tn * BN);
              const uint32_t units_here = (uint32_t)((rows_here + tp.pg_unit_rows - 1) / tp.pg_unit_rows);
              if (!wait_count(tp.pg_flags + tn, tp.seq * units_here, abort_flag)) { ok = false; break; }
            }
            asm volatile("fence.proxy.async;" ::: "memory");  // the copiers' generic stores, then our TMA (async proxy) reads
          }
        }
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
      for (int t = cta; t < num_tiles && ok; t += nctas, ++lt) {
        const uint32_t buf = lt & 1;
        const uint32_t bph = (lt >> 1) & 1;
        if (chain_in) {  // the loading warps waited for the buffer to be free and filled it with the incoming partial sum
          if (!mbar_wait(&tloaded_bar[buf], bph, abort_flag)) { ok = false; break; }
        } else {
          if (!mbar_wait(&tempty_bar[buf], bph ^ 1, abort_flag)) { ok = false; break; }
        }
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
            else mma_f16_ss(d_tmem, ad, bd, idesc, ((kb | kk) != 0) || chain_in);
          }
          mma_commit(&empty_bar[s]);  // smem stage reusable once these MMAs have read it
        }
        if (ok) mma_commit(&tfull_bar[buf]);  // accumulator complete
      }
    }
  } else if (TP == 3 && warp >= 6) {
    // ------------------------------------------ parameter gather: pull the other processes' rows of B into the local buffer
    if constexpr (TP == 3) {
      const int ct = threadIdx.x - 6 * 32;                  // 0..127 among the copier threads of this CTA
      const int ur = tp.pg_unit_rows;
      const int units = (N + ur - 1) / ur;
      const int rot_units = tp.pg_rot * (BN / ur);
      for (int j = cta; j < units; j += nctas) {
        const int unit = (j + rot_units) % units;           // the order in which the tiles want them
        const int row0 = unit * ur;
        const int row1 = min(N, row0 + ur);
        // walk the unit in runs of rows that have one owner; runs of this process's own rows cost nothing
        for (int r = row0; r < row1;) {
          int sj = 0;
          if (tp.pg_nseg > 1 && r >= tp.pg_seg_begin[1]) sj = 1;
          if (tp.pg_nseg > 2 && r >= tp.pg_seg_begin[2]) sj = 2;
          const int sb = tp.pg_seg_begin[sj], se = tp.pg_seg_begin[sj + 1], rpo = tp.pg_rows_per_owner[sj];
          int own = (r - sb) / rpo;
          if (own > tp.P - 1) own = tp.P - 1;
          int run_end = own == tp.P - 1 ? se : min(se, sb + (own + 1) * rpo);
          run_end = min(run_end, row1);
          if (own != tp.rank) {
            const bool flat = tp.pg_ld_u4 == tp.pg_row_u4;   // rows adjacent in memory: the run is one span
            const int spans = flat ? 1 : run_end - r;
            const int span_u4 = flat ? (run_end - r) * tp.pg_row_u4 : tp.pg_row_u4;
            for (int sp = 0; sp < spans; ++sp) {
              const long base = (long)(r + sp) * tp.pg_ld_u4;
              const uint4* __restrict__ src = tp.pg_src[own] + base;
              uint4* __restrict__ dst = tp.pg_dst + base;
              for (int i0 = ct; i0 < span_u4; i0 += 32 * 128) {
                // 32 independent 16-byte peer loads in flight per thread (64 KB per CTA): a loaded link answers in
                // microseconds, so the bytes in flight decide the rate
                uint4 v[32];
#pragma unroll
                for (int u = 0; u < 32; ++u)
                  if (i0 + u * 128 < span_u4) v[u] = src[i0 + u * 128];
#pragma unroll
                for (int u = 0; u < 32; ++u)
                  if (i0 + u * 128 < span_u4) dst[i0 + u * 128] = v[u];
              }
            }
          }
          r = run_end;
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");     // the four copier warps only
        if (ct == 0) {                                      // (fence, then relaxed adds: a release of the unit's rows)
          atomicAdd(tp.pg_flags + row0 / BN, 1u);
          atomicAdd(tp.pg_flags + tiles_n, 1u);
        }
      }
    }
  } else if (TP == 2 && warp >= 6) {
    // ------------------------------------------ chained GEMM: incoming fp32 accumulator tile -> tensor memory
    if constexpr (TP == 2) {
      if (chain_in) {
        const int q = warp & 3;
        uint32_t lt = 0;
        bool ok = true;
        for (int t = cta; t < num_tiles && ok; t += nctas, ++lt) {
          int tm, tn;
          tile_coord(t, tm, tn);
          const uint32_t buf = lt & 1;
          const uint32_t bph = (lt >> 1) & 1;
          if (!mbar_wait(&tempty_bar[buf], bph ^ 1, abort_flag)) { ok = false; break; }
          uint32_t got = 1;
          if (lane == 0) got = wait_peer_flag(tp.flags_in + ((long)tm * tiles_n + tn) * 4 + q, tp.seq, abort_flag) ? 1u : 0u;
          got = __shfl_sync(0xffffffffu, got, 0);
          if (!got) { ok = false; break; }
          tc_fence_after();
          const long row = (long)tm * BM + q * 32 + lane;
          const float* src = tp.inbox + row * tp.ld_in + (long)tn * BN;
          const uint32_t tdst = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
#pragma unroll 1
          for (int c = 0; c < BN; c += 64) {
            uint32_t v[2][32];  // 16 independent 16-byte loads in flight per thread
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 f = make_float4(0.0f, 0.0f, 0.0f, 0.0f);  // columns past N (N % 4 == 0) are never stored
                if (tn * BN + c + u * 32 + 4 * j + 4 <= N)
                  f = __ldcg(reinterpret_cast<const float4*>(src + c + u * 32) + j);  // L2 only: written by a peer GPU
                v[u][4 * j] = __float_as_uint(f.x); v[u][4 * j + 1] = __float_as_uint(f.y);
                v[u][4 * j + 2] = __float_as_uint(f.z); v[u][4 * j + 3] = __float_as_uint(f.w);
              }
            tmem_st_32x32b_x32(tdst + c, v[0]);
            tmem_st_32x32b_x32(tdst + c + 32, v[1]);
          }
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tloaded_bar[buf]);
        }
      }
    }
  } else {
    // --------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may touch
    uint32_t lt = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += nctas, ++lt) {
      int tm, tn;
      tile_coord(t, tm, tn);
      const CUtensorMap* tmc = &tmC;
      int out_sel = 0;
      if constexpr (TP == 2) {
        out_sel = tp.rank == tp.P - 1 ? tm / tp.tiles_per_shard : 0;
        tmc = &tp.tmOut[out_sel];
      }
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
                             reinterpret_cast<uint64_t>(tmc)),
                         "r"(src), "r"(col), "r"(y)
                         : "memory");
          } else {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                             reinterpret_cast<uint64_t>(tmc)),
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
      if constexpr (TP == 2) {
        // this warp's 32 rows of the tile have been written into the next rank's memory: tell it
        if (lane == 0) {
          asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
          asm volatile("fence.proxy.async;" ::: "memory");
          release_peer_flag(tp.flags_out[out_sel] + ((long)tm * tiles_n + tn) * 4 + q, tp.seq);
        }
        __syncwarp();
      }
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
  auto kern = gemm_tc05_kernel<BN, STAGES, A_MN, B_MN, EPI, I8, 0, TpNone>;
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
                                                group_m, scale_a, scale_b, status, TpNone{});
  return (int)cudaGetLastError();
}

template <int BN, int STAGES, bool B_MN, int EPI, int TP>
int launch_tp(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, void* C, const void* R, int M, int N, int K, long ldc,
              long ldr, uint32_t* status, int grid, const TpArgs& tp, cudaStream_t stream, int group_m = 8) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = gemm_tc05_kernel<BN, STAGES, false, B_MN, EPI, false, TP, TpArgs>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  kern<<<grid, TP >= 2 ? NUM_THREADS + 128 : NUM_THREADS, L::TOTAL, stream>>>(
      ta, tb, tc, C, reinterpret_cast<const __nv_bfloat16*>(R), M, N, K, ldc, ldr, group_m, nullptr, nullptr, status, tp);
  return (int)cudaGetLastError();
}

// y[rows of this rank] = bf16( acc (+ R) ) once the last rank of the chain has delivered the tile quarter
__global__ void tp_finish_kernel(const float* __restrict__ acc, const uint32_t* __restrict__ flags, uint32_t seq,
                                 const __nv_bfloat16* __restrict__ R, __nv_bfloat16* __restrict__ y, int rows_per_rank,
                                 int N, int BN, int rank, long ld_acc, long ldr, long ldy, uint32_t* __restrict__ status) {
  __shared__ uint32_t ok_sh;
  __shared__ uint32_t abort_sh;
  const int tn = blockIdx.x;
  const int rb = blockIdx.y;                       // 32-row block inside this rank's rows
  const long row0 = (long)rank * rows_per_rank + (long)rb * 32;
  const int tm = (int)(row0 / BM), q = (int)((row0 % BM) / 32);
  const int tiles_n = (N + BN - 1) / BN;
  if (threadIdx.x == 0) {
    abort_sh = 0;
    ok_sh = wait_peer_flag(flags + ((long)tm * tiles_n + tn) * 4 + q, seq, &abort_sh) ? 1u : 0u;
    if (!ok_sh && status) atomicExch(status, 2u);
  }
  __syncthreads();
  if (!ok_sh) return;
  const int col0 = tn * BN;
  const int vec_per_row = BN / 8;
  for (int i = threadIdx.x; i < 32 * vec_per_row; i += blockDim.x) {
    const int r = i / vec_per_row, c = col0 + (i % vec_per_row) * 8;
    if (c >= N) continue;
    const long row = row0 + r;
    const long lrow = (long)rb * 32 + r;           // row inside this rank's shard (R and y are shard-local)
    const float4 a0 = __ldcg(reinterpret_cast<const float4*>(acc + row * ld_acc + c));
    const float4 a1 = __ldcg(reinterpret_cast<const float4*>(acc + row * ld_acc + c) + 1);
    float f[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    if (R) {
      const uint4 rv = *reinterpret_cast<const uint4*>(R + lrow * ldr + c);
      const uint32_t w[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        f[2 * e] = __fadd_rn(f[2 * e], __uint_as_float(w[e] << 16));
        f[2 * e + 1] = __fadd_rn(f[2 * e + 1], __uint_as_float(w[e] & 0xFFFF0000u));
      }
    }
    uint4 o;
    o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]); o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
    *reinterpret_cast<uint4*>(y + lrow * ldy + c) = o;
  }
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

namespace {
struct PtrTable8 { uint32_t* p[8]; };
__global__ void peer_barrier_tab_kernel(PtrTable8 slots, int rank, int P, uint32_t seq, uint32_t* status) {
  __shared__ uint32_t abort_sh;
  if (threadIdx.x == 0) abort_sh = 0;
  __syncthreads();
  const int p = threadIdx.x;
  if (p < P) {
    release_peer_flag(slots.p[p] + rank, seq);
    if (!wait_peer_flag(slots.p[rank] + p, seq, &abort_sh) && status) atomicExch(status, 3u);
  }
}
inline int tp_chain_bn(int N) { return N >= 256 ? 256 : 128; }
}  // namespace

// Budget of every bounded peer wait of the tensor-parallel kernels and of otb_peer_barrier on the current device
// (default 2 s). A wait that runs out makes its kernel write its status word (1 all-gather->GEMM, 2 chained GEMM /
// otb_tp_finish, 3 otb_peer_barrier) and return normally.
extern "C" int otb_set_cta_rotation(int rotation) {
  if (rotation < 0) return -2;
  return (int)cudaMemcpyToSymbol(g_cta_rotation, &rotation, sizeof(rotation));
}
extern "C" int otb_set_peer_wait_ns(unsigned long long ns) {
  if (ns == 0) return -2;
  return (int)cudaMemcpyToSymbol(g_peer_wait_ns, &ns, sizeof(ns));
}

// Cross-GPU barrier on the stream: slots[p] is rank p's array of P words (peer pointers); seq must grow by one per call.
extern "C" int otb_peer_barrier(void* const* slots, int rank, int P, unsigned seq, uint32_t* status, void* stream) {
  if (P < 1 || P > 8) return -2;
  PtrTable8 t{};
  for (int p = 0; p < P; ++p) t.p[p] = reinterpret_cast<uint32_t*>(slots[p]);
  peer_barrier_tab_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(t, rank, P, seq, status);
  return (int)cudaGetLastError();
}

// All-gather -> GEMM in one kernel.  a_full[p]: rank p's full-size A buffer [M,K] bf16 (peer pointers; this rank's own
// rows [rank*M/P, (rank+1)*M/P) must already be in a_full[rank]); ag_flags[p]: rank p's P*(M/P/128) flag words.
//   C[M,N] = A_full * op(B)^T      B: [N,K] (b_mn = 0) or [K,N] (b_mn = 1), local.
// `copier_ctas` CTAs of the launch push this rank's rows to the peers while the others compute. epi 0 (bf16) or 1 (fp32).
// M must be a multiple of P*128. seq: a value unique to this call on this flag array (same on every rank).
extern "C" int otb_tp_ag_gemm(void* const* a_full, void* const* ag_flags, int rank, int P, unsigned seq, const void* B, void* C,
                              int M, int N, int K, long ldb, long ldc, int b_mn, int epi, int copier_ctas, uint32_t* status,
                              void* stream) {
  if (P < 1 || P > 8 || rank < 0 || rank >= P || M % (P * BM) || (K & 7) || (ldb & 7)) return -2;
  if (epi != EPI_BF16 && epi != EPI_F32) return -3;
  const bool bf16_out = epi == EPI_BF16;
  if ((bf16_out && (ldc & 7)) || (!bf16_out && (ldc & 3))) return -2;
  const int sms = otb_sm_count();
  if (copier_ctas < 1) copier_ctas = 1;
  if (P == 1) copier_ctas = 0;
  int gemm_ctas = sms - copier_ctas;
  const int BN = N > 128 ? 256 : 128;
  const long tiles = (long)(M / BM) * ((N + BN - 1) / BN);
  if (gemm_ctas > tiles) gemm_ctas = (int)tiles;
  constexpr int BK = BK_BYTES / 2;
  const void* A = a_full[rank];
  CUtensorMap ta, tb, tc;
  CUresult r = encode_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, BM);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = b_mn ? encode_2d(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK)
           : encode_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, (uint32_t)BN);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = bf16_out ? encode_2d(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 64, 32, 2)
               : encode_2d(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 32, 32, 4);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  TpArgs tp{};
  tp.rank = rank; tp.P = P; tp.seq = seq; tp.gemm_ctas = gemm_ctas;
  tp.tiles_per_shard = M / BM / P;
  tp.flags_in = reinterpret_cast<const uint32_t*>(ag_flags[rank]);
  tp.ag_block_u4 = (long)BM * K * 2 / 16;
  const long shard_u4 = (long)tp.tiles_per_shard * tp.ag_block_u4;
  tp.ag_src = reinterpret_cast<const uint4*>(A) + rank * shard_u4;
  for (int p = 0; p < P; ++p) {
    tp.ag_dst[p] = p == rank ? nullptr : reinterpret_cast<uint4*>(a_full[p]) + rank * shard_u4;
    tp.ag_flags[p] = reinterpret_cast<uint32_t*>(ag_flags[p]);
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = gemm_ctas + copier_ctas;
#define OTB_AG(BN_, ST_, BMN_, EPI_) return launch_tp<BN_, ST_, BMN_, EPI_, 1>(ta, tb, tc, C, nullptr, M, N, K, ldc, 0, status, grid, tp, s);
  if (BN == 256) {
    if (b_mn) { if (bf16_out) { OTB_AG(256, 4, true, EPI_BF16) } OTB_AG(256, 4, true, EPI_F32) }
    if (bf16_out) { OTB_AG(256, 4, false, EPI_BF16) } OTB_AG(256, 4, false, EPI_F32)
  }
  if (b_mn) { if (bf16_out) { OTB_AG(128, 6, true, EPI_BF16) } OTB_AG(128, 6, true, EPI_F32) }
  if (bf16_out) { OTB_AG(128, 6, false, EPI_BF16) } OTB_AG(128, 6, false, EPI_F32)
#undef OTB_AG
}

// Parameter all-gather fused into the consuming GEMM:  C[M,N] = A[M,K] * B[N,K]^T (+ R), where B is a weight (or up to
// three row-concatenated weights, e.g. wq|wk|wv) whose rows are spread over P processes.
//   b_bufs[p]: row 0 of B inside process p's weight buffer (peer pointers; all buffers have the same layout, leading
//   dimension ldb). In b_bufs[rank], the local buffer, only the rows this process owns need to be current: the call pulls
//   every other row from its owner (plain peer loads issued by four extra warps of the GEMM's CTAs, 128-row blocks in ring
//   order starting at this process's own rows) and counts every finished copy unit in `flags` (local, zeroed once:
//   otb_pg_flag_words(N) words, one counter per B tile and one for the weight), and the TMA producer of a tile waits for
//   the counter of its own B rows only. Afterwards the local buffer holds all of B, so later GEMMs of the same step (other
//   micro-batches, the backward pass) are plain GEMMs on b_bufs[rank].
//   seg_begin[0..nseg-1] / rows_per_owner[0..nseg-1]: first row of each concatenated weight and how many of its rows
//   each process holds (process p: rows [p*rpo, (p+1)*rpo), the last one to the end). seq: how many calls this weight's
//   `flags` have seen, this one included (1, 2, 3, ...): the counters only grow. The owners' rows must be final before the launch (the barrier after the
//   optimizer step) and stay so until every process has pulled (the next optimizer step is behind the next reduction).
//   epi: 0 bf16, 1 fp32, 3 bf16 + residual. Same bits as otb_gemm_bf16 on a complete B. Never allocates.
extern "C" int otb_pg_flag_words(int N) { return (N + (N >= 256 ? 256 : 128) - 1) / (N >= 256 ? 256 : 128) + 1; }

extern "C" int otb_pg_gemm(const void* A, void* const* b_bufs, void* flags, int rank, int P, unsigned seq, void* C, const void* R,
                           int M, int N, int K, long lda, long ldb, long ldc, long ldr, const int* seg_begin,
                           const int* rows_per_owner, int nseg, int epi, uint32_t* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (P < 1 || P > 8 || rank < 0 || rank >= P || nseg < 1 || nseg > 3 || seq == 0) return -2;
  if (epi != EPI_BF16 && epi != EPI_F32 && epi != EPI_BF16_RES) return -3;
  const void* B = b_bufs[rank];
  if ((lda & 7) || (ldb & 7) || (K & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(C) & 15)) return -2;
  for (int p = 0; p < P; ++p)
    if (!b_bufs[p] || (reinterpret_cast<uintptr_t>(b_bufs[p]) & 15)) return -2;
  for (int j = 0; j < nseg; ++j)
    if (rows_per_owner[j] < 1 || seg_begin[j] < 0 || seg_begin[j] >= N || (j && seg_begin[j] <= seg_begin[j - 1])) return -2;
  if (seg_begin[0] != 0) return -2;
  const bool bf16_out = epi != EPI_F32;
  if ((bf16_out && (ldc & 7)) || (!bf16_out && (ldc & 3)) || (epi == EPI_BF16_RES && (!R || (ldr & 7)))) return -2;
  const int sms = otb_sm_count();
  const int BN = N >= 256 ? 256 : 128;
  const long tiles = (long)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sms ? (int)tiles : sms;
  constexpr int BK = BK_BYTES / 2;
  CUtensorMap ta, tb, tc;
  CUresult r = encode_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = encode_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, (uint32_t)BN);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = bf16_out ? encode_2d(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 64, 32, 2)
               : encode_2d(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 32, 32, 4);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  TpArgs tp{};
  tp.rank = rank; tp.P = P; tp.seq = seq; tp.gemm_ctas = grid;
  for (int p = 0; p < P; ++p) tp.pg_src[p] = reinterpret_cast<const uint4*>(b_bufs[p]);
  tp.pg_dst = reinterpret_cast<uint4*>(b_bufs[rank]);
  tp.pg_flags = reinterpret_cast<uint32_t*>(flags);
  tp.pg_nseg = nseg;
  for (int j = 0; j < nseg; ++j) { tp.pg_seg_begin[j] = seg_begin[j]; tp.pg_rows_per_owner[j] = rows_per_owner[j]; }
  tp.pg_seg_begin[nseg] = N;
  tp.pg_row_u4 = K / 8;
  tp.pg_ld_u4 = (int)(ldb / 8);
  // copy units: cut small weights finer, so that the copier warps of every CTA pull something (a unit is what one CTA's
  // four copier warps fetch before they count it in); the cut depends on N only, so the counters of a weight advance by
  // the same amounts in every call
  tp.pg_unit_rows = N >= 16384 ? 128 : (N >= 8192 ? 64 : 16);
  // start the tile order at the tile that holds the first of this process's rows of the first weight
  const int tiles_n = (N + BN - 1) / BN;
  const int rot = (int)(((long)rank * rows_per_owner[0]) / BN);
  tp.pg_rot = rot < tiles_n ? rot : 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // Tile order: groups of row tiles whose A rows make about 16 MB (32 row tiles at K = 2048) sweep all column tiles. Wider
  // than the plain GEMM's 8, so that a sweep stays on this process's own columns of B longer while the others arrive;
  // much wider costs more in L2 misses on A than it hides (measured: 128 row tiles 3-9 % slower, 32 within 1 %).
  int group_m = (int)((16L << 20) / ((long)K * 2 * BM));
  if (group_m < 8) group_m = 8;
  if (group_m > (M + BM - 1) / BM) group_m = (M + BM - 1) / BM;
#define OTB_PG(BN_, ST_, EPI_) return launch_tp<BN_, ST_, false, EPI_, 3>(ta, tb, tc, C, R, M, N, K, ldc, ldr, status, grid, tp, s, group_m);
  if (BN == 256) {
    if (epi == EPI_BF16) { OTB_PG(256, 4, EPI_BF16) }
    if (epi == EPI_F32) { OTB_PG(256, 4, EPI_F32) }
    OTB_PG(256, 4, EPI_BF16_RES)
  }
  if (epi == EPI_BF16) { OTB_PG(128, 6, EPI_BF16) }
  if (epi == EPI_F32) { OTB_PG(128, 6, EPI_F32) }
  OTB_PG(128, 6, EPI_BF16_RES)
#undef OTB_PG
}

extern "C" int otb_tp_chain_bn(int N) { return tp_chain_bn(N); }

// One rank's part of the K-split GEMM whose partial sums travel rank 0 -> 1 -> ... -> P-1 INSIDE the accumulation:
//   acc_r = acc_{r-1} (+)= A_r[M,Kr] * op(B_r)^T, continued in tensor memory, ascending k, so the last rank holds
//   exactly the bits of the unsplit GEMM. A_r: [M,Kr] bf16 K-major; B_r: [N,Kr] (b_mn 0) or [Kr,N] (b_mn 1).
// inbox / flags_in: this rank's fp32 [M, ld_acc] buffer and its (M/128)*(N/BN)*4 flag words (unused on rank 0).
// out_bufs / out_flags: rank < P-1: one entry, the next rank's inbox and flags; rank P-1: P entries, the result
// buffer and flags of each row owner (rows [p*M/P, (p+1)*M/P) belong to rank p). All buffers are [M, ld_acc] fp32.
extern "C" int otb_tp_chain_gemm(const void* A, const void* B, int M, int N, int K, long lda, long ldb, int b_mn, const float* inbox,
                                 const void* flags_in, void* const* out_bufs, void* const* out_flags, long ld_acc, int rank, int P,
                                 unsigned seq, uint32_t* status, void* stream) {
  if (P < 1 || P > 8 || rank < 0 || rank >= P || M % (P * BM) || (lda & 7) || (ldb & 7) || (ld_acc & 3)) return -2;
  const int BN = tp_chain_bn(N);
  constexpr int BK = BK_BYTES / 2;
  CUtensorMap ta, tb;
  CUresult r = encode_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = b_mn ? encode_2d(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK)
           : encode_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, (uint32_t)BN);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  TpArgs tp{};
  tp.rank = rank; tp.P = P; tp.seq = seq;
  tp.tiles_per_shard = M / BM / P;
  tp.inbox = inbox; tp.ld_in = ld_acc;
  tp.flags_in = reinterpret_cast<const uint32_t*>(flags_in);
  const int n_out = rank == P - 1 ? P : 1;
  for (int i = 0; i < n_out; ++i) {
    r = encode_2d(&tp.tmOut[i], out_bufs[i], (uint64_t)N, (uint64_t)M, (uint64_t)ld_acc, 32, 32, 4);
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
    tp.flags_out[i] = reinterpret_cast<uint32_t*>(out_flags[i]);
  }
  const long tiles = (long)(M / BM) * ((N + BN - 1) / BN);
  int grid = otb_sm_count();
  if (grid > tiles) grid = (int)tiles;
  tp.gemm_ctas = grid;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const CUtensorMap& tc = tp.tmOut[0];
  if (BN == 256) {
    if (b_mn) return launch_tp<256, 4, true, EPI_F32, 2>(ta, tb, tc, nullptr, nullptr, M, N, K, ld_acc, 0, status, grid, tp, s);
    return launch_tp<256, 4, false, EPI_F32, 2>(ta, tb, tc, nullptr, nullptr, M, N, K, ld_acc, 0, status, grid, tp, s);
  }
  if (b_mn) return launch_tp<128, 6, true, EPI_F32, 2>(ta, tb, tc, nullptr, nullptr, M, N, K, ld_acc, 0, status, grid, tp, s);
  return launch_tp<128, 6, false, EPI_F32, 2>(ta, tb, tc, nullptr, nullptr, M, N, K, ld_acc, 0, status, grid, tp, s);
}

// This rank's rows of the chained GEMM, once they have arrived:  y[M/P, N] (bf16) = bf16( acc (+ R) ).
// acc / flags: this rank's result buffer [M, ld_acc] fp32 and flag words; R, y: shard-local [M/P, *] bf16.
extern "C" int otb_tp_finish(const float* acc, const void* flags, unsigned seq, const void* R, void* y, int M, int N, int rank, int P,
                             long ld_acc, long ldr, long ldy, uint32_t* status, void* stream) {
  if (P < 1 || M % (P * BM) || (N & 7) || (ldy & 7) || (R && (ldr & 7))) return -2;
  const int BN = tp_chain_bn(N);
  const int rows = M / P;
  dim3 grid((N + BN - 1) / BN, rows / 32);
  tp_finish_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      acc, reinterpret_cast<const uint32_t*>(flags), seq, reinterpret_cast<const __nv_bfloat16*>(R),
      reinterpret_cast<__nv_bfloat16*>(y), rows, N, BN, rank, ld_acc, ldr, ldy, status);
  return (int)cudaGetLastError();
}
