// Causal / sliding-window flash attention for sm_100a on tcgen05 tensor cores, GQA-native.
//
// Kernels (all: warp 0 = TMA producer, warp 1 = tcgen05.mma issuer, the rest = element warps working straight out of
// tensor memory; a warp may touch TMEM lanes 32*(w%4)..+31 only):
//
//   attn_fwd2     CTA = (batch, query head, TWO 128-row query tiles); one thread per row; S = Q K^T (TMEM) -> online
//                 softmax -> P written back over S as bf16 (the A operand of P V) -> O accumulates in TMEM.
//   attn_bwd_kv2  CTA = (batch, KV head, 128 keys); scores formed transposed (S^T, dP^T: lanes are keys), P^T / dS^T
//                 written back in place, dV += P^T dO and dK += dS^T Q with the A operand in TMEM; 64-query steps over
//                 the heads of the group and the query blocks that see these keys, both ascending.
//   attn_bwd_q2   CTA = (batch, query head, two query tiles); two threads per row; dS written back over S;
//                 dQ += dS K with dS in TMEM; 64-key steps ascending.
//   attn_fwd      (one tile per CTA, four threads per row, P through shared memory, O in registers) serves the int8 P V
//                 variant; attn_bwd_kv (one score buffer, P / dS through shared memory) serves sequence lengths that
//                 are not a multiple of 64.
//
// No atomics, no split accumulation: every output element has one owner CTA and a fixed
// summation order, so results are identical for any grid, stream or GPU count. The window rule
// is "key in (query - window, query]" (window = 0: full causal). Scores are used in the log2
// domain: y = fma(s, c, -m) with c = scale*log2(e), p = det_exp2_attn(y) (shared with the CPU
// twin), masked scores are -inf. The saved row statistic `lse` is m + log2(l) in that domain.
// Row sums: each 32-key quarter keeps two ascending chains (even / odd keys) that are added per block;
// the four quarter sums are combined ((l0 + l1) + l2) + l3 at the end.
//
// int8-PV variant of the forward (I8PV): V is quantised beforehand to int8 per (KV head, 128-key block) with one
// fp32 step per block (quant_v_kernel), the probabilities are quantised on the fly to q = rint(127 p), P V runs on
// the int8 tensor cores (tcgen05 kind::i8, exact int32 sums over the 128 keys of a block) and is dequantised in
// fp32: O = O*alpha + float(sum) * (step / 127). Softmax statistics stay fp32 on the unquantised probabilities;
// the backward is the straight-through float shadow (the ordinary backward kernels on the bf16 q, k, v).
// Reference role: int8pv_causal_flash_attention (attention_repop.py:52; docs/MODEL_OP_DTYPE_TRACE.md:80,117-119).
//
// Layouts: q/k come from one [B*T, ld] bf16 buffer (post-RoPE; head h at column h*D, KV head g
// at column (H+g)*D); v comes from the packed qkv buffer; O is [B*T, H*D]; lse and delta are
// [B, H, T] fp32. Reference role: repop causal_flash_attention fwd/bwd
// (src/pretrain/model/modules/attention_repop.py:38-53).
#include "tc05.cuh"
#include "common.cuh"
#include "det_math.h"

using namespace tc05;

namespace {

// Launch-order permutation for the race tests: block x works as block (x + g_attn_rotation) mod gridDim.x. A block owns
// its query tile (or key block) and sums in a fixed order, so any rotation must give the same bytes (0 in production).
__device__ int g_attn_rotation = 0;

constexpr int BQ = 128;   // query rows per tile
constexpr int BKV = 128;  // keys per block
constexpr int NSPLIT = 4;                 // threads per row
constexpr int KPT = 128 / NSPLIT;         // keys per thread and block
constexpr int SOFTMAX_THREADS = 128 * NSPLIT;
constexpr int ATT_THREADS = 64 + SOFTMAX_THREADS;
constexpr int SOFTMAX_WARPS = SOFTMAX_THREADS / 32;

__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_THREADS) : "memory"); }

// N (16 or 32) consecutive TMEM columns of this thread's lane
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&v)[N]) {
  if constexpr (N == 32) tmem_ld_32x32b_x32(taddr, v);
  else tmem_ld_32x32b_x16(taddr, v);
}

struct Bars {
  uint64_t b[24];
  uint32_t tmem_slot;
  uint32_t abort_flag;
};
struct BarsX : Bars {
  float xch[2][NSPLIT][128];  // [parity][part][row] exchange between the threads of a row
};

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~uintptr_t(1023));
}
// byte offset of the 16-byte chunk `ch` (0..7) of row r in a [rows][128 B] 128B-swizzled tile
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t ch) { return r * 128u + ((ch ^ (r & 7u)) << 4); }

// K-major operand, tile made of [128 rows][64 elems] sub-tiles 16 KB apart; k-step kk = 16 elems
__device__ __forceinline__ uint64_t desc_k(uint32_t base, int kk) {
  return make_smem_desc(base + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
}
// MN-major operand, tile made of [128 k-rows][64 mn elems] chunks 16 KB apart; k-step kk = 16 rows
__device__ __forceinline__ uint64_t desc_mn(uint32_t base, int kk) {
  return make_smem_desc(base + kk * 2048, 16384, 1024);
}

template <int D>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int col, int row, int b) {
#pragma unroll
  for (int c = 0; c < D / 64; ++c) tma_load_3d(dst + c * 16384, tm, bar, col + c * 64, row, b);
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// key kj is hidden from query qi (causal, and the sliding window when window > 0)
__device__ __forceinline__ bool key_hidden(int kj, int qi, int window) { return kj > qi || (window > 0 && kj <= qi - window); }

// Maximum of a thread's KPT raw scores. MASK = false is the common (fully visible) block: no position tests at all.
template <bool MASK>
__device__ __forceinline__ float scores_max(const uint32_t (&sv)[KPT], int kbase, int qi, int window) {
  float mx = -INFINITY;
  if constexpr (MASK) {
#pragma unroll
    for (int e = 0; e < KPT; ++e) mx = fmaxf(mx, key_hidden(kbase + e, qi, window) ? -INFINITY : __uint_as_float(sv[e]));
  } else {
#pragma unroll
    for (int e = 0; e < KPT; e += 2) mx = max3(mx, __uint_as_float(sv[e]), __uint_as_float(sv[e + 1]));
  }
  return mx;
}

// p = exp2(s * c - m) for the thread's KPT scores, packed for the P V product (bf16 pairs, or int8 quadruples when I8),
// and the two ascending row-sum chains (even keys, odd keys) as one packed value.
template <bool MASK, bool I8>
__device__ __forceinline__ f2 probs_pack(const uint32_t (&sv)[KPT], float c_log2, float m_safe, int kbase, int qi, int window,
                                         uint32_t (&pk)[KPT / 2]) {
  const f2 c2 = pack2(c_log2, c_log2), nm2 = pack2(-m_safe, -m_safe);
  f2 lsum2 = pack2(0.0f, 0.0f);
#pragma unroll
  for (int e = 0; e < KPT; e += 2) {
    f2 p2 = exp2_attn2(fma2(pack2(__uint_as_float(sv[e]), __uint_as_float(sv[e + 1])), c2, nm2));
    float p0, p1;
    unpack2(p2, p0, p1);
    if constexpr (MASK) {
      if (key_hidden(kbase + e, qi, window)) p0 = 0.0f;
      if (key_hidden(kbase + e + 1, qi, window)) p1 = 0.0f;
      p2 = pack2(p0, p1);
    }
    lsum2 = add2(lsum2, p2);
    if constexpr (I8) {
      const uint32_t q0b = (uint32_t)(int)rintf(__fmul_rn(p0, 127.0f)), q1b = (uint32_t)(int)rintf(__fmul_rn(p1, 127.0f));
      if ((e & 3) == 0) pk[e >> 2] = 0;
      pk[e >> 2] |= (q0b | (q1b << 8)) << (8 * (e & 3));
    } else {
      pk[e >> 1] = pack_bf16(p0, p1);
    }
  }
  return lsum2;
}

// ---------------------------------------------------------------------------- forward
template <int D, bool I8PV>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQK, const __grid_constant__ CUtensorMap tmV,
                __nv_bfloat16* __restrict__ O, long ldo, float* __restrict__ lse_out, int T, int H, int Hkv, int window,
                float scale, float c_log2, const float* __restrict__ vstep, uint32_t* __restrict__ status) {
  static_assert(!I8PV || D == 128, "the int8 P V path needs 128-byte value rows");
  constexpr int TILE = BQ * D * 2;
  constexpr int ST = 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sQ = smem;
  uint8_t* sP = sQ + TILE;
  uint8_t* sK = sP + BQ * BKV * 2;
  uint8_t* sV = sK + ST * TILE;
  BarsX* bars = reinterpret_cast<BarsX*>(sV + ST * TILE);
  uint64_t* q_full = &bars->b[0];
  uint64_t* k_full = &bars->b[1];    // [ST]
  uint64_t* k_empty = &bars->b[3];   // [ST]
  uint64_t* v_full = &bars->b[5];    // [ST]
  uint64_t* v_empty = &bars->b[7];   // [ST]
  uint64_t* s_full = &bars->b[9];    // [2]
  uint64_t* s_empty = &bars->b[11];  // [2]
  uint64_t* p_ready = &bars->b[13];
  uint64_t* pv_full = &bars->b[14];
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (T + BQ - 1) / BQ;
  const int qt = nq - 1 - (int)((blockIdx.x + g_attn_rotation) % gridDim.x);  // heavy tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (H / Hkv);
  const int q0 = qt * BQ;
  const int jmax = qt;
  const int jmin = (window > 0 && q0 - window + 1 > 0) ? (q0 - window + 1) / BKV : 0;
  const int n = jmax - jmin + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], SOFTMAX_WARPS); }
    mbar_init(p_ready, SOFTMAX_WARPS);
    mbar_init(pv_full, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  const uint32_t tS = tmem, tPV = tmem + 256;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(q_full, TILE);
      load_tile<D>(sQ, &tmQK, q_full, h * D, q0, b);
      for (int i = 0; i < n; ++i) {
        const int st = i % ST;
        const uint32_t ph = (i / ST) & 1;
        const int k0 = (jmin + i) * BKV;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&k_full[st], TILE);
        load_tile<D>(sK + st * TILE, &tmQK, &k_full[st], (H + g) * D, k0, b);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag)) break;
        if (I8PV) {  // int8 values: [128 keys][D bytes], one swizzle row per key
          mbar_expect_tx(&v_full[st], BKV * D);
          tma_load_3d(sV + st * TILE, &tmV, &v_full[st], g * D, k0, b);
        } else {
          mbar_expect_tx(&v_full[st], TILE);
          load_tile<D>(sV + st * TILE, &tmV, &v_full[st], (H + Hkv + g) * D, k0, b);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idS = make_idesc(128, BKV, 0, 0);
      constexpr uint32_t idPV = I8PV ? make_idesc(128, D, 0, 1, 2, 1) : make_idesc(128, D, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_S = [&](int i) {
        const int st = i % ST;
        if (!mbar_wait(&k_full[st], (i / ST) & 1, abort_flag)) return false;
        if (!mbar_wait(&s_empty[i & 1], ((i >> 1) & 1) ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + st * TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_f16_ss(tS + (i & 1) * 128, desc_k(aQ, kk), desc_k(aK, kk), idS, kk != 0);
        mma_commit(&s_full[i & 1]);
        mma_commit(&k_empty[st]);
        return true;
      };
      if (ok) ok = issue_S(0);
      for (int i = 0; i < n && ok; ++i) {
        if (i + 1 < n) { if (!issue_S(i + 1)) { ok = false; break; } }
        const int st = i % ST;
        if (!mbar_wait(p_ready, i & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&v_full[st], (i / ST) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + st * TILE);
        if (I8PV) {
          // P: [128 rows][128 int8 keys] K-major, 32 keys per instruction; V: [128 keys][128 int8] MN-major, 32 key rows per instruction
#pragma unroll
          for (int kk = 0; kk < BKV / 32; ++kk)
            mma_i8_ss(tPV, make_smem_desc(aP + kk * 32, 16, 1024), make_smem_desc(aV + kk * 4096, 16384, 1024), idPV, kk != 0);
        } else {
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk) mma_f16_ss(tPV, desc_k(aP, kk), desc_mn(aV, kk), idPV, kk != 0);
        }
        mma_commit(pv_full);
        mma_commit(&v_empty[st]);
      }
    }
  } else {
    constexpr int DH = D / NSPLIT;            // output columns per thread
    constexpr int CW = 16;                    // TMEM columns per load of the PV accumulator (short loads keep registers free)
    const int qd = warp & 3;
    const int part = (warp - 2) >> 2;
    const int r = qd * 32 + lane;          // row inside the tile == TMEM lane
    const int qi = q0 + r;                 // query position
    const uint32_t lane_off = uint32_t(qd * 32) << 16;
    float m_run = -INFINITY, l_run = 0.0f, alpha_prev = 0.0f;
    float c_prev = 0.0f;  // int8 P V: dequantisation factor (value step / 127) of the block whose P V is pending
    const int nblk = (T + BKV - 1) / BKV;
    // accumulator word -> fp32 contribution
    auto pv_val = [&](uint32_t w) { return I8PV ? __fmul_rn(__int2float_rn((int)w), c_prev) : __uint_as_float(w); };
    f2 o[DH / 2];
#pragma unroll
    for (int d = 0; d < DH / 2; ++d) o[d] = pack2(0.0f, 0.0f);
    bool ok = true;
    for (int i = 0; i < n; ++i) {
      const int j = jmin + i;
      const int kbase = j * BKV + part * KPT;
      const bool need_mask = (j == jmax) || (window > 0 && j * BKV < q0 + BQ - window);
      ok = ok && mbar_wait(&s_full[i & 1], (i >> 1) & 1, abort_flag);
      tc_fence_after();
      const uint32_t tSb = tS + (i & 1) * 128 + part * KPT + lane_off;
      // the thread's 32 raw scores stay in registers for both passes; once they are there the S buffer is free
      uint32_t sv[KPT];
      if (ok) {
        tmem_ld_32x32b_x32(tSb, sv);
        tmem_ld_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0 && ok) mbar_arrive(&s_empty[i & 1]);
      float mx = -INFINITY;
      if (ok) mx = need_mask ? scores_max<true>(sv, kbase, qi, window) : scores_max<false>(sv, kbase, qi, window);
      bars->xch[i & 1][part][r] = mx;
      softmax_bar();
#pragma unroll
      for (int pp = 0; pp < NSPLIT; ++pp) mx = fmaxf(mx, bars->xch[i & 1][pp][r]);
      const float m_new = fmaxf(m_run, __fmul_rn(mx, c_log2));
      const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;
      const float alpha = det_exp2_attn(__fadd_rn(m_run, -m_safe));
      // probabilities and the quarter-row sum first (independent of O), while the tensor core finishes the previous P V
      f2 lsum2 = pack2(0.0f, 0.0f);
      uint32_t pk[KPT / 2];
      if (ok)
        lsum2 = need_mask ? probs_pack<true, I8PV>(sv, c_log2, m_safe, kbase, qi, window, pk)
                          : probs_pack<false, I8PV>(sv, c_log2, m_safe, kbase, qi, window, pk);
      // deferred accumulation of the previous block's P V (its completion also frees the P buffer)
      if (i > 0) {
        ok = ok && mbar_wait(pv_full, (i - 1) & 1, abort_flag);
        tc_fence_after();
        if (ok) {
          const f2 a2 = pack2(alpha_prev, alpha_prev);
#pragma unroll
          for (int c = 0; c < DH / CW; ++c) {
            uint32_t v[CW];
            tmem_ld_cols<CW>(tPV + lane_off + part * DH + c * CW, v);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < CW; e += 2)
              o[(c * CW + e) >> 1] = fma2(o[(c * CW + e) >> 1], a2, pack2(pv_val(v[e]), pv_val(v[e + 1])));
          }
        }
      }
      if (ok) {
        if (I8PV) {
          // keys part*32 .. +31 are bytes part*32 .. +31 of the 128-byte row: chunks part*2, part*2 + 1
#pragma unroll
          for (int w = 0; w < 2; ++w)
            *reinterpret_cast<uint4*>(sP + swz(r, part * 2 + w)) = make_uint4(pk[4 * w], pk[4 * w + 1], pk[4 * w + 2], pk[4 * w + 3]);
        } else {
          // keys part*32 .. +31 -> 64-key sub-tile (part >> 1), 16-byte chunks (part & 1) * 4 .. +3 of the row
          uint8_t* base = sP + (part >> 1) * 16384;
#pragma unroll
          for (int w = 0; w < 4; ++w)
            *reinterpret_cast<uint4*>(base + swz(r, (part & 1) * 4 + w)) =
                make_uint4(pk[4 * w], pk[4 * w + 1], pk[4 * w + 2], pk[4 * w + 3]);
        }
      }
      float ls0, ls1;
      unpack2(lsum2, ls0, ls1);
      const float lsum = __fadd_rn(ls0, ls1);
      l_run = __fmaf_rn(l_run, alpha, lsum);
      m_run = m_new;
      alpha_prev = alpha;
      if (I8PV) c_prev = __fmul_rn(vstep[((long)b * Hkv + g) * nblk + j], 1.0f / 127.0f);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0 && ok) mbar_arrive(p_ready);
    }
    ok = ok && mbar_wait(pv_full, (n - 1) & 1, abort_flag);
    tc_fence_after();
    bars->xch[n & 1][part][r] = l_run;
    softmax_bar();
    float l_tot = bars->xch[n & 1][0][r];
#pragma unroll
    for (int pp = 1; pp < NSPLIT; ++pp) l_tot = __fadd_rn(l_tot, bars->xch[n & 1][pp][r]);
    if (ok) {
      const bool in_range = qi < T;
      __nv_bfloat16* orow = O + ((long)b * T + qi) * ldo + (long)h * D + part * DH;
#pragma unroll
      for (int c = 0; c < DH / CW; ++c) {
        uint32_t v[CW];
        tmem_ld_cols<CW>(tPV + lane_off + part * DH + c * CW, v);
        tmem_ld_wait();
        uint32_t pk[CW / 2];
#pragma unroll
        for (int e = 0; e < CW; e += 2) {
          float a0, a1;
          unpack2(fma2(o[(c * CW + e) >> 1], pack2(alpha_prev, alpha_prev), pack2(pv_val(v[e]), pv_val(v[e + 1]))), a0, a1);
          pk[e >> 1] = pack_bf16(__fdiv_rn(a0, l_tot), __fdiv_rn(a1, l_tot));
        }
        if (in_range) {
#pragma unroll
          for (int w = 0; w < CW / 8; ++w)
            reinterpret_cast<uint4*>(orow + c * CW)[w] = make_uint4(pk[4 * w], pk[4 * w + 1], pk[4 * w + 2], pk[4 * w + 3]);
        }
      }
      if (in_range && part == 0)
        lse_out[((long)b * H + h) * T + qi] = __fmaf_rn(det_logf(l_tot), 1.44269504088896341f, m_run);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bars->abort_flag && status) atomicExch(status, 2u);
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// ------------------------------------------------- forward, two query tiles per CTA
// The bf16 forward. One CTA owns TWO adjacent 128-row query tiles (A, B) of one (batch, head) and walks the key blocks
// both need; warp 0 loads K and V once for both tiles, warp 1 issues every tensor-core product, warps 2..5 are tile A's
// softmax (ONE THREAD PER ROW, so no value ever crosses threads) and warps 6..9 tile B's. While one tile's softmax
// runs, the tensor core works for the other tile. Tensor memory: S_A | S_B | O_A | O_B, 128 columns each.
//   S = Q K^T lands in S_X; the row's thread reads it twice (maximum, then probabilities) and overwrites its first 64
//   columns with P as bf16 pairs, which is the A operand of P V (tcgen05.mma with A in tensor memory); O_X is the
//   accumulator of P V over all key blocks: before block i > first the thread multiplies its O row by
//   alpha = exp2(m_old - m_new) in place (skipped, with identical bits, when alpha == 1 for the whole warp), then the
//   tensor core adds the block's 8 k-steps to it. The row sum keeps the four 32-key quarter chains of the CPU twin.
constexpr int F2_THREADS = 64 + 256;

struct Bars2 {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_ready[2], o_done[2];
  uint32_t tmem_slot;
  uint32_t abort_flag;
};

template <int D>
__global__ void __launch_bounds__(F2_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQK, const __grid_constant__ CUtensorMap tmV,
                 __nv_bfloat16* __restrict__ O, long ldo, float* __restrict__ lse_out, int T, int H, int Hkv, int window,
                 float c_log2, uint32_t* __restrict__ status) {
  constexpr int TILE = BQ * D * 2;
  constexpr int ST = 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sQ = smem;                  // [2] tiles A, B
  uint8_t* sK = sQ + 2 * TILE;         // [ST]
  uint8_t* sV = sK + ST * TILE;        // [ST]
  Bars2* bars = reinterpret_cast<Bars2*>(sV + ST * TILE);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (T + BQ - 1) / BQ;
  const int pr = (int)gridDim.x - 1 - (int)((blockIdx.x + g_attn_rotation) % gridDim.x);  // heavy pairs first
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (H / Hkv);
  const int tile0 = 2 * pr;
  const bool hasB = tile0 + 1 < nq;
  // key-block range [jlo_X, jhi_X] of tile X; the CTA walks [jlo_A, jhi_B] (jlo_A <= jlo_B, jhi_A < jhi_B)
  auto jlo_of = [&](int t) { const int q0 = t * BQ; return (window > 0 && q0 - window + 1 > 0) ? (q0 - window + 1) / BKV : 0; };
  const int jloA = jlo_of(tile0), jhiA = tile0;
  const int jloB = hasB ? jlo_of(tile0 + 1) : 0, jhiB = tile0 + 1;
  const int jlo = jloA, jhi = hasB ? jhiB : jhiA;
  const int n = jhi - jlo + 1;
  auto act = [&](int X, int j) { return X == 0 ? (j <= jhiA) : (hasB && j >= jloB && j <= jhiB); };

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(&bars->k_full[s], 1); mbar_init(&bars->k_empty[s], 1); mbar_init(&bars->v_full[s], 1); mbar_init(&bars->v_empty[s], 1);
    }
    for (int x = 0; x < 2; ++x) { mbar_init(&bars->s_full[x], 1); mbar_init(&bars->p_ready[x], 4); mbar_init(&bars->o_done[x], 1); }
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&bars->q_full, hasB ? 2 * TILE : TILE);
      load_tile<D>(sQ, &tmQK, &bars->q_full, h * D, tile0 * BQ, b);
      if (hasB) load_tile<D>(sQ + TILE, &tmQK, &bars->q_full, h * D, (tile0 + 1) * BQ, b);
      for (int i = 0; i < n; ++i) {
        const int st = i % ST;
        const uint32_t ph = (i / ST) & 1;
        const int k0 = (jlo + i) * BKV;
        if (!mbar_wait(&bars->k_empty[st], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&bars->k_full[st], TILE);
        load_tile<D>(sK + st * TILE, &tmQK, &bars->k_full[st], (H + g) * D, k0, b);
        if (!mbar_wait(&bars->v_empty[st], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&bars->v_full[st], TILE);
        load_tile<D>(sV + st * TILE, &tmV, &bars->v_full[st], (H + Hkv + g) * D, k0, b);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idS = make_idesc(128, BKV, 0, 0);
      constexpr uint32_t idPV = make_idesc(128, D, 0, 1);
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag);
      int done[2] = {0, 0};  // P V products issued per tile
      // S of block i for every tile that takes part in it; frees the K stage afterwards
      auto issue_S = [&](int i) {
        const int st = i % ST;
        if (!mbar_wait(&bars->k_full[st], (i / ST) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + st * TILE);
        for (int X = 0; X < 2; ++X) {
          if (!act(X, jlo + i)) continue;
          const uint32_t aQ = smem_u32(sQ + X * TILE);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_f16_ss(tmem + X * 128, desc_k(aQ, kk), desc_k(aK, kk), idS, kk != 0);
          mma_commit(&bars->s_full[X]);
        }
        mma_commit(&bars->k_empty[st]);
        return true;
      };
      // S of tile X only (block i), K stage not released
      auto issue_S1 = [&](int X, int i) {
        const uint32_t aK = smem_u32(sK + (i % ST) * TILE), aQ = smem_u32(sQ + X * TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_f16_ss(tmem + X * 128, desc_k(aQ, kk), desc_k(aK, kk), idS, kk != 0);
        mma_commit(&bars->s_full[X]);
      };
      if (ok) ok = issue_S(0);
      for (int i = 0; i < n && ok; ++i) {
        const int st = i % ST, j = jlo + i;
        const bool more = i + 1 < n;
        bool k_next = false;  // K of block i + 1 is in shared memory
        for (int X = 0; X < 2 && ok; ++X) {
          if (act(X, j)) {
            if (!mbar_wait(&bars->p_ready[X], done[X] & 1, abort_flag)) { ok = false; break; }
            if (!mbar_wait(&bars->v_full[st], (i / ST) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t aV = smem_u32(sV + st * TILE);
#pragma unroll
            for (int kk = 0; kk < BKV / 16; ++kk)
              mma_f16_ts(tmem + 256 + X * 128, tmem + X * 128 + kk * 8, desc_mn(aV, kk), idPV, (done[X] | kk) != 0);
            ++done[X];
            if (j == (X == 0 ? jhiA : jhiB)) mma_commit(&bars->o_done[X]);
          }
          // this tile's next S goes right behind its P V (it overwrites the P just consumed)
          if (more && act(X, j + 1)) {
            if (!k_next) {
              if (!mbar_wait(&bars->k_full[(i + 1) % ST], ((i + 1) / ST) & 1, abort_flag)) { ok = false; break; }
              tc_fence_after();
              k_next = true;
            }
            issue_S1(X, i + 1);
          }
        }
        if (!ok) break;
        mma_commit(&bars->v_empty[st]);
        if (more) mma_commit(&bars->k_empty[(i + 1) % ST]);
      }
    }
  } else {
    const int X = (warp - 2) >> 2;           // tile of this warp
    const int quad = warp & 3;               // TMEM lane quadrant this warp may touch
    const int r = quad * 32 + lane;          // row inside the tile == TMEM lane
    const int q0 = (tile0 + X) * BQ;
    const int qi = q0 + r;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    const uint32_t tS = tmem + X * 128 + lane_off, tO = tmem + 256 + X * 128 + lane_off;
    const int jhiX = X == 0 ? jhiA : jhiB;
    float m_run = -INFINITY, l_run[NSPLIT] = {0.0f, 0.0f, 0.0f, 0.0f};
    int cnt = 0;
    bool ok = true;
    if (X == 0 || hasB) {
      for (int i = 0; i < n && ok; ++i) {
        const int j = jlo + i;
        if (!act(X, j)) continue;
        const bool need_mask = (j == jhiX) || (window > 0 && j * BKV < q0 + BQ - window);
        if (!mbar_wait(&bars->s_full[X], cnt & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // pass 1: row maximum. Fully visible blocks take the unrolled path with the next 32 columns already in flight
        // while the current ones are reduced; blocks on the diagonal or the window edge take a compact loop.
        float mx = -INFINITY;
        if (!need_mask) {
          uint32_t sa[KPT], sb[KPT];
          tmem_ld_32x32b_x32(tS, sa);
          tmem_ld_wait();
          tmem_ld_32x32b_x32(tS + KPT, sb);
          mx = scores_max<false>(sa, 0, 0, 0);
          tmem_ld_wait();
          tmem_ld_32x32b_x32(tS + 2 * KPT, sa);
          mx = fmaxf(mx, scores_max<false>(sb, 0, 0, 0));
          tmem_ld_wait();
          tmem_ld_32x32b_x32(tS + 3 * KPT, sb);
          mx = fmaxf(mx, scores_max<false>(sa, 0, 0, 0));
          tmem_ld_wait();
          mx = fmaxf(mx, scores_max<false>(sb, 0, 0, 0));
        } else {
#pragma unroll 1
          for (int c = 0; c < NSPLIT; ++c) {
            uint32_t sv[KPT];
            tmem_ld_32x32b_x32(tS + c * KPT, sv);
            tmem_ld_wait();
            mx = fmaxf(mx, scores_max<true>(sv, j * BKV + c * KPT, qi, window));
          }
        }
        const float m_new = fmaxf(m_run, __fmul_rn(mx, c_log2));
        const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;
        const float alpha = det_exp2_attn(__fadd_rn(m_run, -m_safe));
        // O row *= alpha (the previous P V is complete: its S product was issued behind it)
        if (cnt > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
          const f2 a2 = pack2(alpha, alpha);
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(tO + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              float a0, a1;
              unpack2(mul2(pack2(__uint_as_float(v[e]), __uint_as_float(v[e + 1])), a2), a0, a1);
              v[e] = __float_as_uint(a0);
              v[e + 1] = __float_as_uint(a1);
            }
            tmem_st_32x32b_x32(tO + c * 32, v);
          }
        }
        // pass 2: probabilities, quarter sums, P (bf16 pairs) over the first 64 columns of S (a P store only ever
        // covers columns whose scores have been read already)
        if (!need_mask) {
          uint32_t sa[KPT], sb[KPT], pk[KPT / 2];
          float ls0, ls1;
          tmem_ld_32x32b_x32(tS, sa);
          tmem_ld_wait();
          tmem_ld_32x32b_x32(tS + KPT, sb);
          unpack2(probs_pack<false, false>(sa, c_log2, m_safe, 0, 0, 0, pk), ls0, ls1);
          l_run[0] = __fmaf_rn(l_run[0], alpha, __fadd_rn(ls0, ls1));
          tmem_ld_wait();
          tmem_st_32x32b_x16(tS, pk);
          tmem_ld_32x32b_x32(tS + 2 * KPT, sa);
          unpack2(probs_pack<false, false>(sb, c_log2, m_safe, 0, 0, 0, pk), ls0, ls1);
          l_run[1] = __fmaf_rn(l_run[1], alpha, __fadd_rn(ls0, ls1));
          tmem_ld_wait();
          tmem_st_32x32b_x16(tS + KPT / 2, pk);
          tmem_ld_32x32b_x32(tS + 3 * KPT, sb);
          unpack2(probs_pack<false, false>(sa, c_log2, m_safe, 0, 0, 0, pk), ls0, ls1);
          l_run[2] = __fmaf_rn(l_run[2], alpha, __fadd_rn(ls0, ls1));
          tmem_ld_wait();
          tmem_st_32x32b_x16(tS + KPT, pk);
          unpack2(probs_pack<false, false>(sb, c_log2, m_safe, 0, 0, 0, pk), ls0, ls1);
          l_run[3] = __fmaf_rn(l_run[3], alpha, __fadd_rn(ls0, ls1));
          tmem_st_32x32b_x16(tS + 3 * (KPT / 2), pk);
        } else {
          float lq[NSPLIT];
#pragma unroll 1
          for (int c = 0; c < NSPLIT; ++c) {
            uint32_t sv[KPT], pk[KPT / 2];
            tmem_ld_32x32b_x32(tS + c * KPT, sv);
            tmem_ld_wait();
            float ls0, ls1;
            unpack2(probs_pack<true, false>(sv, c_log2, m_safe, j * BKV + c * KPT, qi, window, pk), ls0, ls1);
            const float lq_c = __fadd_rn(ls0, ls1);
            lq[0] = c == 0 ? lq_c : lq[0]; lq[1] = c == 1 ? lq_c : lq[1]; lq[2] = c == 2 ? lq_c : lq[2]; lq[3] = c == 3 ? lq_c : lq[3];
            tmem_st_32x32b_x16(tS + c * (KPT / 2), pk);
          }
#pragma unroll
          for (int c = 0; c < NSPLIT; ++c) l_run[c] = __fmaf_rn(l_run[c], alpha, lq[c]);
        }
        tmem_st_wait();
        m_run = m_new;
        ++cnt;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_ready[X]);
      }
      ok = ok && mbar_wait(&bars->o_done[X], 0, abort_flag);
      tc_fence_after();
      if (ok) {
        const float l_tot = __fadd_rn(__fadd_rn(__fadd_rn(l_run[0], l_run[1]), l_run[2]), l_run[3]);
        const bool in_range = qi < T;
        __nv_bfloat16* orow = O + ((long)b * T + qi) * ldo + (long)h * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tO + c * 32, v);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2)
            pk[e >> 1] = pack_bf16(__fdiv_rn(__uint_as_float(v[e]), l_tot), __fdiv_rn(__uint_as_float(v[e + 1]), l_tot));
          if (in_range) {
#pragma unroll
            for (int w = 0; w < 4; ++w)
              reinterpret_cast<uint4*>(orow + c * 32)[w] = make_uint4(pk[4 * w], pk[4 * w + 1], pk[4 * w + 2], pk[4 * w + 3]);
          }
        }
        if (in_range) lse_out[((long)b * H + h) * T + qi] = __fmaf_rn(det_logf(l_tot), 1.44269504088896341f, m_run);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bars->abort_flag && status) atomicExch(status, 2u);
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// Backward element math for a thread's KPT (score, dP) pairs: p = exp2(s * c - lse) (0 where hidden or the row is out of
// range), ds = (p * (dp - delta)) * scale; both packed to bf16 pairs.
template <bool MASK, bool WANT_P, int N = KPT>
__device__ __forceinline__ void bwd_probs(const uint32_t (&vs)[N], const uint32_t (&vd)[N], float c_log2, float lse_r, float dl_r,
                                          float scale, bool row_ok, int kbase, int qi, int window, uint32_t (&pk)[N / 2],
                                          uint32_t (&dsr)[N / 2]) {
  const f2 c2 = pack2(c_log2, c_log2), nl2 = pack2(-lse_r, -lse_r), nd2 = pack2(-dl_r, -dl_r), sc2 = pack2(scale, scale);
#pragma unroll
  for (int e = 0; e < N; e += 2) {
    f2 p2 = exp2_attn2(fma2(pack2(__uint_as_float(vs[e]), __uint_as_float(vs[e + 1])), c2, nl2));
    if constexpr (MASK) {
      float p0, p1;
      unpack2(p2, p0, p1);
      if (!row_ok || key_hidden(kbase + e, qi, window)) p0 = 0.0f;
      if (!row_ok || key_hidden(kbase + e + 1, qi, window)) p1 = 0.0f;
      p2 = pack2(p0, p1);
    }
    const f2 d2 = mul2(mul2(p2, add2(pack2(__uint_as_float(vd[e]), __uint_as_float(vd[e + 1])), nd2)), sc2);
    float d0, d1;
    unpack2(d2, d0, d1);
    dsr[e >> 1] = pack_bf16(d0, d1);
    if constexpr (WANT_P) {
      float p0, p1;
      unpack2(p2, p0, p1);
      pk[e >> 1] = pack_bf16(p0, p1);
    }
  }
}

// -------------------------------------------------------- backward: dK and dV
template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_kv_kernel(const __grid_constant__ CUtensorMap tmQK, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmDO, const float* __restrict__ lse,
                   const float* __restrict__ delta, __nv_bfloat16* __restrict__ dK, long lddk,
                   __nv_bfloat16* __restrict__ dV, long lddv, int T, int H, int Hkv, int window, float scale,
                   float c_log2, uint32_t* __restrict__ status) {
  constexpr int TILE = BQ * D * 2;
  constexpr int ST = 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE;
  uint8_t* sPdS = sV + TILE;
  uint8_t* sQ = sPdS + BQ * BKV * 2;  // [ST]
  uint8_t* sDO = sQ + ST * TILE;      // [ST]
  Bars* bars = reinterpret_cast<Bars*>(sDO + ST * TILE);
  uint64_t* kv_full = &bars->b[0];
  uint64_t* qdo_full = &bars->b[1];   // [ST]
  uint64_t* qdo_empty = &bars->b[3];  // [ST]
  uint64_t* sdp_full = &bars->b[5];
  uint64_t* sdp_empty = &bars->b[6];
  uint64_t* p_ready = &bars->b[7];
  uint64_t* dv_done = &bars->b[8];
  uint64_t* ds_ready = &bars->b[9];
  uint64_t* dk_done = &bars->b[10];
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (T + BQ - 1) / BQ;
  const int kb = (int)((blockIdx.x + g_attn_rotation) % gridDim.x), g = blockIdx.y, b = blockIdx.z;
  const int G = H / Hkv;
  const int k0 = kb * BKV;
  int qlast = nq - 1;
  if (window > 0) qlast = min(qlast, (k0 + BKV - 1 + window - 1) / BQ);
  const int nqi = qlast - kb + 1;  // query blocks per head
  const int n = G * nqi;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < ST; ++s) { mbar_init(&qdo_full[s], 1); mbar_init(&qdo_empty[s], 1); }
    mbar_init(sdp_full, 1); mbar_init(sdp_empty, SOFTMAX_WARPS); mbar_init(p_ready, SOFTMAX_WARPS); mbar_init(dv_done, 1);
    mbar_init(ds_ready, SOFTMAX_WARPS); mbar_init(dk_done, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 128, tDV = tmem + 256, tDK = tmem + 384;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(kv_full, 2 * TILE);
      load_tile<D>(sK, &tmQK, kv_full, (H + g) * D, k0, b);
      load_tile<D>(sV, &tmV, kv_full, (H + Hkv + g) * D, k0, b);
      for (int i = 0; i < n; ++i) {
        const int st = i % ST;
        const int h = g * G + i / nqi;
        const int q0 = (kb + i % nqi) * BQ;
        if (!mbar_wait(&qdo_empty[st], ((i / ST) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(&qdo_full[st], 2 * TILE);
        load_tile<D>(sQ + st * TILE, &tmQK, &qdo_full[st], h * D, q0, b);
        load_tile<D>(sDO + st * TILE, &tmDO, &qdo_full[st], h * D, q0, b);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idS = make_idesc(128, BKV, 0, 0);   // S = Q K^T, dP = dO V^T
      constexpr uint32_t idG = make_idesc(128, D, 1, 1);     // dV = P^T dO, dK = dS^T Q
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sPdS);
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      auto issue_sdp = [&](int i) {
        const int st = i % ST;
        if (!mbar_wait(&qdo_full[st], (i / ST) & 1, abort_flag)) return false;
        if (!mbar_wait(sdp_empty, (i & 1) ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ + st * TILE), aDO = smem_u32(sDO + st * TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_f16_ss(tS, desc_k(aQ, kk), desc_k(aK, kk), idS, kk != 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_f16_ss(tDP, desc_k(aDO, kk), desc_k(aV, kk), idS, kk != 0);
        mma_commit(sdp_full);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int i = 0; i < n && ok; ++i) {
        const int st = i % ST;
        const uint32_t aQ = smem_u32(sQ + st * TILE), aDO = smem_u32(sDO + st * TILE);
        // S and dP of the next block run while the softmax warps work on this one (they released the buffers
        // as soon as the values were in registers)
        if (i + 1 < n) { if (!issue_sdp(i + 1)) { ok = false; break; } }
        if (!mbar_wait(p_ready, i & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) mma_f16_ss(tDV, desc_mn(aP, kk), desc_mn(aDO, kk), idG, (i | kk) != 0);
        mma_commit(dv_done);
        if (!mbar_wait(ds_ready, i & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) mma_f16_ss(tDK, desc_mn(aP, kk), desc_mn(aQ, kk), idG, (i | kk) != 0);
        mma_commit(dk_done);
        mma_commit(&qdo_empty[st]);
      }
    }
  } else {
    constexpr int DH = D / NSPLIT;
    constexpr int CW = DH >= 32 ? 32 : 16;
    const int qd = warp & 3;
    const int part = (warp - 2) >> 2;
    const int r = qd * 32 + lane;
    const uint32_t lane_off = uint32_t(qd * 32) << 16;
    bool ok = true;
    for (int i = 0; i < n && ok; ++i) {
      const int h = g * G + i / nqi;
      const int qb = kb + i % nqi;
      const int qi = qb * BQ + r;
      const bool row_ok = qi < T;
      const bool need_mask = (qb == kb) || (window > 0 && k0 < qb * BQ + BQ - window) || (qb * BQ + BQ > T);
      const float lse_r = row_ok ? lse[((long)b * H + h) * T + qi] : 0.0f;
      const float dl_r = row_ok ? delta[((long)b * H + h) * T + qi] : 0.0f;
      if (!mbar_wait(sdp_full, i & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t dsr[KPT / 2], pk[KPT / 2];
      {
        uint32_t vs[KPT], vd[KPT];
        tmem_ld_32x32b_x32(tS + lane_off + part * KPT, vs);
        tmem_ld_32x32b_x32(tDP + lane_off + part * KPT, vd);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sdp_empty);  // S and dP are in registers: the next block's products may overwrite them
        if (need_mask) bwd_probs<true, true>(vs, vd, c_log2, lse_r, dl_r, scale, row_ok, k0 + part * KPT, qi, window, pk, dsr);
        else bwd_probs<false, true>(vs, vd, c_log2, lse_r, dl_r, scale, row_ok, k0 + part * KPT, qi, window, pk, dsr);
      }
      // the shared P / dS buffer is free once the previous block's dK product has read it
      if (i > 0) { if (!mbar_wait(dk_done, (i - 1) & 1, abort_flag)) { ok = false; break; } }
      uint8_t* base = sPdS + (part >> 1) * 16384;
#pragma unroll
      for (int w = 0; w < 4; ++w)
        *reinterpret_cast<uint4*>(base + swz(r, (part & 1) * 4 + w)) = make_uint4(pk[4 * w], pk[4 * w + 1], pk[4 * w + 2], pk[4 * w + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
      if (!mbar_wait(dv_done, i & 1, abort_flag)) { ok = false; break; }
#pragma unroll
      for (int w = 0; w < 4; ++w)
        *reinterpret_cast<uint4*>(base + swz(r, (part & 1) * 4 + w)) = make_uint4(dsr[4 * w], dsr[4 * w + 1], dsr[4 * w + 2], dsr[4 * w + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    if (ok && mbar_wait(dk_done, (n - 1) & 1, abort_flag)) {
      tc_fence_after();
      const int kj = k0 + r;  // TMEM lane == key row
      const bool in_range = kj < T;
      __nv_bfloat16* dkrow = dK + ((long)b * T + kj) * lddk + (long)g * D + part * DH;
      __nv_bfloat16* dvrow = dV + ((long)b * T + kj) * lddv + (long)g * D + part * DH;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
#pragma unroll
        for (int c = 0; c < DH / CW; ++c) {
          uint32_t v[CW];
          tmem_ld_cols<CW>((which ? tDK : tDV) + lane_off + part * DH + c * CW, v);
          tmem_ld_wait();
          if (in_range) {
            uint4* dst = reinterpret_cast<uint4*>((which ? dkrow : dvrow) + c * CW);
#pragma unroll
            for (int w = 0; w < CW / 8; ++w)
              dst[w] = make_uint4(pack_bf16(__uint_as_float(v[8 * w]), __uint_as_float(v[8 * w + 1])),
                                  pack_bf16(__uint_as_float(v[8 * w + 2]), __uint_as_float(v[8 * w + 3])),
                                  pack_bf16(__uint_as_float(v[8 * w + 4]), __uint_as_float(v[8 * w + 5])),
                                  pack_bf16(__uint_as_float(v[8 * w + 6]), __uint_as_float(v[8 * w + 7])));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bars->abort_flag && status) atomicExch(status, 3u);
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// ------------------------------------------------ backward: dQ, two query tiles per CTA
// Same organisation as the forward: one CTA owns two adjacent 128-row query tiles, one thread per query row, and the
// tensor core serves one tile while the other tile's threads do the element math (two threads per row, each with half
// of the step's keys; nothing crosses threads in the backward). Keys advance in steps of 64: S = Q K^T and
// dP = dO V^T (128 x 64 each) land in tensor memory, the row's threads turn them into dS = p (dP - delta) scale, store
// it as bf16 pairs over their own score columns, and dQ += dS K runs with dS as the tensor-memory A operand. dQ accumulates over ascending keys in 16-key tensor-core steps, exactly as before.
// Tensor memory per tile: S 64 | dP 64 | dQ 128 columns.
constexpr int HK = 64;  // keys per step

template <int D, int ROWS>
__device__ __forceinline__ void load_tile_r(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int col, int row, int b) {
#pragma unroll
  for (int c = 0; c < D / 64; ++c) tma_load_3d(dst + c * (ROWS * 128), tm, bar, col + c * 64, row, b);
}
// K-major / MN-major operand descriptors for tiles of ROWS rows ([ROWS][64 elems] sub-tiles ROWS * 128 bytes apart)
template <int ROWS>
__device__ __forceinline__ uint64_t desc_k_r(uint32_t base, int kk) {
  return make_smem_desc(base + (kk >> 2) * (ROWS * 128) + (kk & 3) * 32, 16, 1024);
}
template <int ROWS>
__device__ __forceinline__ uint64_t desc_mn_r(uint32_t base, int kk) {
  return make_smem_desc(base + kk * 2048, ROWS * 128, 1024);
}

struct BarsQ2 {
  uint64_t qdo_full, kv_full[3], kv_empty[3], sdp_full[2], ds_ready[2], dq_done[2];
  uint32_t tmem_slot;
  uint32_t abort_flag;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_q2_kernel(const __grid_constant__ CUtensorMap tmQK, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmK64, const __grid_constant__ CUtensorMap tmV64,
                   const float* __restrict__ lse, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dQ, long lddq, int T,
                   int H, int Hkv, int window, float scale, float c_log2, uint32_t* __restrict__ status) {
  constexpr int TILE = BQ * D * 2;    // a [128][D] query-side tile
  constexpr int KT = HK * D * 2;      // a [64][D] key-side tile
  constexpr int ST = 3;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sQ = smem;                 // [2]
  uint8_t* sDO = sQ + 2 * TILE;       // [2]
  uint8_t* sK = sDO + 2 * TILE;       // [ST]
  uint8_t* sV = sK + ST * KT;         // [ST]
  BarsQ2* bars = reinterpret_cast<BarsQ2*>(sV + ST * KT);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (T + BQ - 1) / BQ;
  const int pr = (int)gridDim.x - 1 - (int)((blockIdx.x + g_attn_rotation) % gridDim.x);
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (H / Hkv);
  const int tile0 = 2 * pr;
  const bool hasB = tile0 + 1 < nq;
  // 64-key steps [ulo_X, uhi_X] of tile X: every step that holds a key some row of the tile can see
  auto ulo_of = [&](int t) { const int q0 = t * BQ; return (window > 0 && q0 - window + 1 > 0) ? (q0 - window + 1) / HK : 0; };
  const int uloA = ulo_of(tile0), uhiA = 2 * tile0 + 1;
  const int uloB = hasB ? ulo_of(tile0 + 1) : 0, uhiB = 2 * tile0 + 3;
  const int ulo = uloA, uhi = hasB ? uhiB : uhiA;
  const int n = uhi - ulo + 1;
  auto act = [&](int X, int u) { return X == 0 ? (u <= uhiA) : (hasB && u >= uloB && u <= uhiB); };

  if (threadIdx.x == 0) {
    mbar_init(&bars->qdo_full, 1);
    for (int s = 0; s < ST; ++s) { mbar_init(&bars->kv_full[s], 1); mbar_init(&bars->kv_empty[s], 1); }
    for (int x = 0; x < 2; ++x) { mbar_init(&bars->sdp_full[x], 1); mbar_init(&bars->ds_ready[x], 8); mbar_init(&bars->dq_done[x], 1); }
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&bars->qdo_full, (hasB ? 4 : 2) * TILE);
      for (int X = 0; X < (hasB ? 2 : 1); ++X) {
        load_tile<D>(sQ + X * TILE, &tmQK, &bars->qdo_full, h * D, (tile0 + X) * BQ, b);
        load_tile<D>(sDO + X * TILE, &tmDO, &bars->qdo_full, h * D, (tile0 + X) * BQ, b);
      }
      for (int i = 0; i < n; ++i) {
        const int st = i % ST;
        const int k0 = (ulo + i) * HK;
        if (!mbar_wait(&bars->kv_empty[st], ((i / ST) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(&bars->kv_full[st], 2 * KT);
        load_tile_r<D, HK>(sK + st * KT, &tmK64, &bars->kv_full[st], (H + g) * D, k0, b);
        load_tile_r<D, HK>(sV + st * KT, &tmV64, &bars->kv_full[st], (H + Hkv + g) * D, k0, b);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idS = make_idesc(128, HK, 0, 0);  // S = Q K^T, dP = dO V^T: 128 x 64
      constexpr uint32_t idQ = make_idesc(128, D, 0, 1);   // dQ = dS K: A in tensor memory, B MN-major
      bool ok = mbar_wait(&bars->qdo_full, 0, abort_flag);
      int done[2] = {0, 0};
      auto issue_sdp = [&](int X, int i) {
        const uint32_t aK = smem_u32(sK + (i % ST) * KT), aV = smem_u32(sV + (i % ST) * KT);
        const uint32_t aQ = smem_u32(sQ + X * TILE), aDO = smem_u32(sDO + X * TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_f16_ss(tmem + X * 256, desc_k(aQ, kk), desc_k_r<HK>(aK, kk), idS, kk != 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_f16_ss(tmem + X * 256 + 64, desc_k(aDO, kk), desc_k_r<HK>(aV, kk), idS, kk != 0);
        mma_commit(&bars->sdp_full[X]);
      };
      if (ok) ok = mbar_wait(&bars->kv_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        for (int X = 0; X < 2; ++X)
          if (act(X, ulo)) issue_sdp(X, 0);
      }
      for (int i = 0; i < n && ok; ++i) {
        const int st = i % ST, u = ulo + i;
        const bool more = i + 1 < n;
        bool kv_next = false;
        for (int X = 0; X < 2 && ok; ++X) {
          if (act(X, u)) {
            if (!mbar_wait(&bars->ds_ready[X], done[X] & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t aK = smem_u32(sK + st * KT);
#pragma unroll
            for (int kk = 0; kk < HK / 16; ++kk)
              mma_f16_ts(tmem + X * 256 + 128, tmem + X * 256 + (kk >> 1) * 32 + (kk & 1) * 8, desc_mn_r<HK>(aK, kk), idQ, (done[X] | kk) != 0);
            ++done[X];
            if (u == (X == 0 ? uhiA : uhiB)) mma_commit(&bars->dq_done[X]);
          }
          if (more && act(X, u + 1)) {
            if (!kv_next) {
              if (!mbar_wait(&bars->kv_full[(i + 1) % ST], ((i + 1) / ST) & 1, abort_flag)) { ok = false; break; }
              tc_fence_after();
              kv_next = true;
            }
            issue_sdp(X, i + 1);
          }
        }
        if (!ok) break;
        mma_commit(&bars->kv_empty[st]);
      }
    }
  } else {
    // sixteen element warps: two threads per query row (32 of the step's 64 keys each), 8 warps per tile
    const int X = (warp - 2) >> 3;
    const int quad = warp & 3;
    const int hf = ((warp - 2) & 7) >> 2;    // which half of the step's keys
    const int r = quad * 32 + lane;
    const int q0 = (tile0 + X) * BQ;
    const int qi = q0 + r;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    const uint32_t tS = tmem + X * 256 + lane_off + hf * 32, tDP = tS + 64, tDQ = tmem + X * 256 + 128 + lane_off;
    const bool row_ok = qi < T;
    bool ok = true;
    if (X == 0 || hasB) {
      const float lse_r = row_ok ? lse[((long)b * H + h) * T + qi] : 0.0f;
      const float dl_r = row_ok ? delta[((long)b * H + h) * T + qi] : 0.0f;
      int cnt = 0;
      for (int i = 0; i < n && ok; ++i) {
        const int u = ulo + i;
        if (!act(X, u)) continue;
        const int k0 = u * HK;
        // some (row, key) pair of this step is hidden, or the tile has rows past the end of the sequence
        const bool need_mask = (k0 + HK - 1 > q0) || (window > 0 && k0 <= q0 + BQ - 1 - window) || (q0 + BQ > T);
        if (!mbar_wait(&bars->sdp_full[X], cnt & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // dS (bf16 pairs, 8 columns per 16 keys) goes over the thread's own score columns, which it has read by then
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t sa[16], da[16], pk[8], unused[8];
          tmem_ld_32x32b_x16(tS + c * 16, sa);
          tmem_ld_32x32b_x16(tDP + c * 16, da);
          tmem_ld_wait();
          if (need_mask) bwd_probs<true, false, 16>(sa, da, c_log2, lse_r, dl_r, scale, row_ok, k0 + hf * 32 + c * 16, qi, window, unused, pk);
          else bwd_probs<false, false, 16>(sa, da, c_log2, lse_r, dl_r, scale, true, 0, 0, 0, unused, pk);
          tmem_st_32x32b_x8(tS + c * 8, pk);
        }
        tmem_st_wait();
        ++cnt;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->ds_ready[X]);
      }
      ok = ok && mbar_wait(&bars->dq_done[X], 0, abort_flag);
      tc_fence_after();
      if (ok) {
        constexpr int DHALF = D / 2;
        __nv_bfloat16* dqrow = dQ + ((long)b * T + qi) * lddq + (long)h * D + hf * DHALF;
#pragma unroll
        for (int c = 0; c < DHALF / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tDQ + hf * DHALF + c * 32, v);
          tmem_ld_wait();
          if (row_ok) {
            uint4* dst = reinterpret_cast<uint4*>(dqrow + c * 32);
#pragma unroll
            for (int w = 0; w < 4; ++w)
              dst[w] = make_uint4(pack_bf16(__uint_as_float(v[8 * w]), __uint_as_float(v[8 * w + 1])),
                                  pack_bf16(__uint_as_float(v[8 * w + 2]), __uint_as_float(v[8 * w + 3])),
                                  pack_bf16(__uint_as_float(v[8 * w + 4]), __uint_as_float(v[8 * w + 5])),
                                  pack_bf16(__uint_as_float(v[8 * w + 6]), __uint_as_float(v[8 * w + 7])));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bars->abort_flag && status) atomicExch(status, 4u);
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// ------------------------------------------- backward: dK and dV, transposed scores
// One CTA owns 128 keys of one KV head and walks, head by head of the group and in ascending query order, the 64-row
// query steps that see those keys. The products are formed TRANSPOSED, S^T = K Q^T and dP^T = V dO^T (128 keys x 64
// queries), so a tensor-memory lane is a key: the threads of a key row write P^T and dS^T back over their own columns
// as bf16 pairs and both accumulations, dV += P^T dO and dK += dS^T Q, take their A operand straight from tensor memory.
// Two score buffers alternate, so the tensor core forms the next step's scores while the 16 element warps (four threads
// per key row, 16 queries each, no value crosses threads) work on the current one. Per-query statistics (-lse, -delta)
// arrive through a small bulk copy beside each Q / dO tile. dV and dK accumulate over (head, query) in 16-query
// tensor-core steps in the same order as the one-buffer kernel above, so the bits are the same.
// Tensor memory: dV 128 | dK 128 | buffer 0: S^T 64, dP^T 64 | buffer 1: S^T 64, dP^T 64. Needs T % 64 == 0.
constexpr int KV2_ST = 4;

struct BarsKV2 {
  uint64_t kv_full, qdo_full[KV2_ST], qdo_empty[KV2_ST], sdp_full[2], pds_ready[2], acc_done;
  uint32_t tmem_slot;
  uint32_t abort_flag;
};

template <bool MASK>
__device__ __forceinline__ void bwd_probs_t(const uint32_t (&vs)[16], const uint32_t (&vd)[16], const float* __restrict__ nl,
                                            const float* __restrict__ nd, float c_log2, float scale, int kj, int qbase, int window,
                                            uint32_t (&pk)[8], uint32_t (&dsr)[8]) {
  const f2 c2 = pack2(c_log2, c_log2), sc2 = pack2(scale, scale);
#pragma unroll
  for (int e = 0; e < 16; e += 4) {
    const float4 l4 = *reinterpret_cast<const float4*>(nl + e), d4 = *reinterpret_cast<const float4*>(nd + e);
#pragma unroll
    for (int w = 0; w < 4; w += 2) {
      const f2 nl2 = w ? pack2(l4.z, l4.w) : pack2(l4.x, l4.y), nd2 = w ? pack2(d4.z, d4.w) : pack2(d4.x, d4.y);
      f2 p2 = exp2_attn2(fma2(pack2(__uint_as_float(vs[e + w]), __uint_as_float(vs[e + w + 1])), c2, nl2));
      float p0, p1;
      unpack2(p2, p0, p1);
      if constexpr (MASK) {
        if (key_hidden(kj, qbase + e + w, window)) p0 = 0.0f;
        if (key_hidden(kj, qbase + e + w + 1, window)) p1 = 0.0f;
        p2 = pack2(p0, p1);
      }
      const f2 d2 = mul2(mul2(p2, add2(pack2(__uint_as_float(vd[e + w]), __uint_as_float(vd[e + w + 1])), nd2)), sc2);
      float d0, d1;
      unpack2(d2, d0, d1);
      pk[(e + w) >> 1] = pack_bf16(p0, p1);
      dsr[(e + w) >> 1] = pack_bf16(d0, d1);
    }
  }
}

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_kv2_kernel(const __grid_constant__ CUtensorMap tmQK, const __grid_constant__ CUtensorMap tmV,
                    const __grid_constant__ CUtensorMap tmQ64, const __grid_constant__ CUtensorMap tmDO64,
                    const float* __restrict__ nlse, const float* __restrict__ ndelta, __nv_bfloat16* __restrict__ dK, long lddk,
                    __nv_bfloat16* __restrict__ dV, long lddv, int T, int H, int Hkv, int window, float scale, float c_log2,
                    uint32_t* __restrict__ status) {
  constexpr int TILE = BKV * D * 2;  // [128 keys][D]
  constexpr int QT = HK * D * 2;     // [64 queries][D]
  constexpr int ST = KV2_ST;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE;
  uint8_t* sQ = sV + TILE;           // [ST]
  uint8_t* sDO = sQ + ST * QT;       // [ST]
  float* sStat = reinterpret_cast<float*>(sDO + ST * QT);  // [ST][2][64]: -lse, -delta of the step's queries
  BarsKV2* bars = reinterpret_cast<BarsKV2*>(sStat + ST * 2 * HK);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb = (int)((blockIdx.x + g_attn_rotation) % gridDim.x), g = blockIdx.y, b = blockIdx.z;
  const int G = H / Hkv;
  const int k0 = kb * BKV;
  const int nu = T / HK;  // query steps in the sequence
  const int ulo = k0 / HK;
  int uhi = nu - 1;
  if (window > 0) uhi = min(uhi, (k0 + BKV - 1 + window - 1) / HK);
  const int nqi = uhi - ulo + 1;  // query steps per head
  const int n = G * nqi;

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < ST; ++s) { mbar_init(&bars->qdo_full[s], 1); mbar_init(&bars->qdo_empty[s], 1); }
    for (int z = 0; z < 2; ++z) { mbar_init(&bars->sdp_full[z], 1); mbar_init(&bars->pds_ready[z], SOFTMAX_WARPS); }
    mbar_init(&bars->acc_done, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  const uint32_t tDV = tmem, tDK = tmem + 128, tBuf = tmem + 256;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&bars->kv_full, 2 * TILE);
      load_tile<D>(sK, &tmQK, &bars->kv_full, (H + g) * D, k0, b);
      load_tile<D>(sV, &tmV, &bars->kv_full, (H + Hkv + g) * D, k0, b);
      for (int i = 0; i < n; ++i) {
        const int st = i % ST;
        const int h = g * G + i / nqi;
        const int q0 = (ulo + i % nqi) * HK;
        if (!mbar_wait(&bars->qdo_empty[st], ((i / ST) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(&bars->qdo_full[st], 2 * QT + 2 * HK * 4);
        load_tile_r<D, HK>(sQ + st * QT, &tmQ64, &bars->qdo_full[st], h * D, q0, b);
        load_tile_r<D, HK>(sDO + st * QT, &tmDO64, &bars->qdo_full[st], h * D, q0, b);
        bulk_load(sStat + st * 2 * HK, nlse + ((long)b * H + h) * T + q0, HK * 4, &bars->qdo_full[st]);
        bulk_load(sStat + st * 2 * HK + HK, ndelta + ((long)b * H + h) * T + q0, HK * 4, &bars->qdo_full[st]);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idS = make_idesc(128, HK, 0, 0);  // S^T = K Q^T, dP^T = V dO^T: 128 keys x 64 queries
      constexpr uint32_t idG = make_idesc(128, D, 0, 1);   // dV = P^T dO, dK = dS^T Q: A in tensor memory, B MN-major
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV);
      bool ok = mbar_wait(&bars->kv_full, 0, abort_flag);
      auto issue_sdp = [&](int i) {
        const int st = i % ST, z = i & 1;
        if (!mbar_wait(&bars->qdo_full[st], (i / ST) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ + st * QT), aDO = smem_u32(sDO + st * QT);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_f16_ss(tBuf + z * 128, desc_k(aK, kk), desc_k_r<HK>(aQ, kk), idS, kk != 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_f16_ss(tBuf + z * 128 + 64, desc_k(aV, kk), desc_k_r<HK>(aDO, kk), idS, kk != 0);
        mma_commit(&bars->sdp_full[z]);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      if (ok && n > 1) ok = issue_sdp(1);
      for (int i = 0; i < n && ok; ++i) {
        const int st = i % ST, z = i & 1;
        if (!mbar_wait(&bars->pds_ready[z], (i >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ + st * QT), aDO = smem_u32(sDO + st * QT);
#pragma unroll
        for (int kk = 0; kk < HK / 16; ++kk)
          mma_f16_ts(tDV, tBuf + z * 128 + kk * 16, desc_mn_r<HK>(aDO, kk), idG, (i | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < HK / 16; ++kk)
          mma_f16_ts(tDK, tBuf + z * 128 + 64 + kk * 16, desc_mn_r<HK>(aQ, kk), idG, (i | kk) != 0);
        mma_commit(&bars->qdo_empty[st]);
        if (i + 1 == n) mma_commit(&bars->acc_done);
        if (i + 2 < n) { if (!issue_sdp(i + 2)) { ok = false; break; } }  // into the buffer just consumed
      }
    }
  } else {
    constexpr int DH = D / NSPLIT;
    const int quad = warp & 3;
    const int cq = (warp - 2) >> 2;          // which 16 of the step's 64 queries
    const int r = quad * 32 + lane;          // key row == TMEM lane
    const int kj = k0 + r;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    bool ok = true;
    for (int i = 0; i < n && ok; ++i) {
      const int st = i % ST, z = i & 1;
      const int q0 = (ulo + i % nqi) * HK;
      const int qbase = q0 + cq * 16;
      // some (key, query) pair of the step is hidden
      const bool need_mask = (k0 + BKV - 1 > q0) || (window > 0 && k0 <= q0 + HK - 1 - window);
      if (!mbar_wait(&bars->qdo_full[st], (i / ST) & 1, abort_flag)) { ok = false; break; }  // the statistics are in shared memory
      if (!mbar_wait(&bars->sdp_full[z], (i >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tSt = tBuf + z * 128 + cq * 16 + lane_off, tDPt = tSt + 64;
      const float* nl = sStat + st * 2 * HK + cq * 16;
      const float* nd = nl + HK;
      uint32_t vs[16], vd[16], pk[8], dsr[8];
      tmem_ld_32x32b_x16(tSt, vs);
      tmem_ld_32x32b_x16(tDPt, vd);
      tmem_ld_wait();
      if (need_mask) bwd_probs_t<true>(vs, vd, nl, nd, c_log2, scale, kj, qbase, window, pk, dsr);
      else bwd_probs_t<false>(vs, vd, nl, nd, c_log2, scale, kj, qbase, window, pk, dsr);
      tmem_st_32x32b_x8(tSt, pk);
      tmem_st_32x32b_x8(tDPt, dsr);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->pds_ready[z]);
    }
    if (ok && mbar_wait(&bars->acc_done, 0, abort_flag)) {
      tc_fence_after();
      const bool in_range = kj < T;
      __nv_bfloat16* dkrow = dK + ((long)b * T + kj) * lddk + (long)g * D + cq * DH;
      __nv_bfloat16* dvrow = dV + ((long)b * T + kj) * lddv + (long)g * D + cq * DH;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
#pragma unroll
        for (int c = 0; c < DH / 16; ++c) {
          uint32_t v[16];
          tmem_ld_32x32b_x16((which ? tDK : tDV) + lane_off + cq * DH + c * 16, v);
          tmem_ld_wait();
          if (in_range) {
            uint4* dst = reinterpret_cast<uint4*>((which ? dkrow : dvrow) + c * 16);
#pragma unroll
            for (int w = 0; w < 2; ++w)
              dst[w] = make_uint4(pack_bf16(__uint_as_float(v[8 * w]), __uint_as_float(v[8 * w + 1])),
                                  pack_bf16(__uint_as_float(v[8 * w + 2]), __uint_as_float(v[8 * w + 3])),
                                  pack_bf16(__uint_as_float(v[8 * w + 4]), __uint_as_float(v[8 * w + 5])),
                                  pack_bf16(__uint_as_float(v[8 * w + 6]), __uint_as_float(v[8 * w + 7])));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bars->abort_flag && status) atomicExch(status, 3u);
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// delta[b,h,t] = sum_d dO[t,h,d] * O[t,h,d]; one warp per (row, head), lane_tree with VW = 4. The scratch has three
// [B, H, T] planes: delta, -lse and -delta (the negated copies feed the transposed dK/dV kernel's packed arithmetic).
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, long lddo, const __nv_bfloat16* __restrict__ O,
                                  long ldo, const float* __restrict__ lse, float* __restrict__ delta, int B, int T, int H, int D) {
  const long wid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const long rows = (long)B * T;
  if (wid >= rows * H) return;
  const long row = wid / H;
  const int h = (int)(wid - row * H);
  float acc = 0.0f;
  if (lane * 4 < D) {
    const __nv_bfloat16* a = dO + row * lddo + (long)h * D + lane * 4;
    const __nv_bfloat16* o = O + row * ldo + (long)h * D + lane * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc = __fmaf_rn(__bfloat162float(a[e]), __bfloat162float(o[e]), acc);
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
  if (lane == 0) {
    const long bb = row / T, t = row - bb * T;
    const long idx = (bb * H + h) * T + t, plane = (long)B * H * T;
    delta[idx] = acc;
    delta[plane + idx] = -lse[idx];
    delta[2 * plane + idx] = -acc;
  }
}

// One CTA per (128-key block, KV head, batch): step = max(max|V| / 127, FLT_MIN) over the block, V_q = clamp(rint(V / step)).
template <int D>
__global__ void quant_v_kernel(const __nv_bfloat16* __restrict__ qkv, long ldqkv, int vcol0, int8_t* __restrict__ vq, long ldvq,
                               float* __restrict__ vstep, int T, int Hkv) {
  __shared__ float sh[32];
  const int blk = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int nblk = gridDim.x;
  const int k0 = blk * BKV;
  constexpr int VPR = D / 8;  // 16-byte vectors per row
  float m = 0.0f;
  for (int i = threadIdx.x; i < BKV * VPR; i += blockDim.x) {
    const int r = i / VPR, c = (i % VPR) * 8;
    if (k0 + r >= T) continue;
    const uint4 v = *reinterpret_cast<const uint4*>(qkv + ((long)b * T + k0 + r) * ldqkv + vcol0 + g * D + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      m = fmaxf(m, fabsf(__uint_as_float(w[e] << 16)));
      m = fmaxf(m, fabsf(__uint_as_float(w[e] & 0xFFFF0000u)));
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = m;
  __syncthreads();
  m = 0.0f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, sh[w]);
  const float step = fmaxf(__fmul_rn(m, 1.0f / 127.0f), 1.17549435e-38f);
  if (threadIdx.x == 0) vstep[((long)b * Hkv + g) * nblk + blk] = step;
  for (int i = threadIdx.x; i < BKV * VPR; i += blockDim.x) {
    const int r = i / VPR, c = (i % VPR) * 8;
    if (k0 + r >= T) continue;
    const uint4 v = *reinterpret_cast<const uint4*>(qkv + ((long)b * T + k0 + r) * ldqkv + vcol0 + g * D + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[2] = {0, 0};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float f = (e & 1) ? __uint_as_float(w[e >> 1] & 0xFFFF0000u) : __uint_as_float(w[e >> 1] << 16);
      const int qv = (int)fminf(fmaxf(rintf(__fdiv_rn(f, step)), -127.0f), 127.0f);
      o[e >> 2] |= (uint32_t)(qv & 0xFF) << (8 * (e & 3));
    }
    *reinterpret_cast<uint2*>(vq + ((long)b * T + k0 + r) * ldvq + g * D + c) = make_uint2(o[0], o[1]);
  }
}

CUresult encode_3d_u8(CUtensorMap* out, const void* ptr, uint64_t cols, uint64_t T, uint64_t B, uint64_t ld_bytes) {
  static PFN_encodeTiled fn = get_encode_tiled();
  if (!fn) return CUDA_ERROR_NOT_SUPPORTED;
  cuuint64_t dims[3] = {cols, T, B};
  cuuint64_t strides[2] = {ld_bytes, T * ld_bytes};
  cuuint32_t box[3] = {128, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

CUresult encode_3d(CUtensorMap* out, const void* ptr, uint64_t cols, uint64_t T, uint64_t B, uint64_t ld_elems, uint32_t box_rows = 128) {
  static PFN_encodeTiled fn = get_encode_tiled();
  if (!fn) return CUDA_ERROR_NOT_SUPPORTED;
  cuuint64_t dims[3] = {cols, T, B};
  cuuint64_t strides[2] = {ld_elems * 2, T * ld_elems * 2};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

template <int D> constexpr int attn_smem_bytes() { return (1 + 2 * 2) * (BQ * D * 2) + BQ * BKV * 2 + 1024 + 512 + 4096; }
template <int D> constexpr int attn_bwd_smem_bytes() { return (2 + 2 * 2) * (BQ * D * 2) + BQ * BKV * 2 + 1024 + 256; }

template <int D> constexpr int attn_bwd_q2_smem_bytes() { return 4 * (BQ * D * 2) + 2 * 3 * (HK * D * 2) + 1024 + 256; }
template <int D> constexpr int attn_bwd_kv2_smem_bytes() { return 2 * (BKV * D * 2) + 2 * KV2_ST * (HK * D * 2) + KV2_ST * 2 * HK * 4 + 1024 + 256; }
template <int D> constexpr int attn_fwd2_smem_bytes() { return (2 + 2 * 2) * (BQ * D * 2) + 1024 + 256; }

template <typename K>
int set_smem(K kern, int bytes) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

}  // namespace

// qk: [B*T, ldqk] bf16 holding H query heads then Hkv key heads (width D each); qkv: [B*T, ldqkv] bf16 whose
// value heads start at column (H + Hkv) * D; O: [B*T, ldo]; lse: [B, H, T] fp32. D in {64, 128}.
extern "C" int otb_set_attn_rotation(int rotation) {
  if (rotation < 0) return -2;
  return (int)cudaMemcpyToSymbol(g_attn_rotation, &rotation, sizeof(rotation));
}
extern "C" int otb_attn_fwd(const void* qk, long ldqk, const void* qkv, long ldqkv, void* O, long ldo, float* lse, int B,
                            int T, int H, int Hkv, int D, int window, float scale, uint32_t* status, void* stream) {
  if ((D != 64 && D != 128) || H % Hkv || (ldqk & 7) || (ldqkv & 7) || (ldo & 7)) return -2;
  CUtensorMap tq, tv;
  CUresult r = encode_3d(&tq, qk, (uint64_t)ldqk, (uint64_t)T, (uint64_t)B, (uint64_t)ldqk);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = encode_3d(&tv, qkv, (uint64_t)ldqkv, (uint64_t)T, (uint64_t)B, (uint64_t)ldqkv);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  const float c_log2 = (float)((double)scale * 1.4426950408889634);
  const int nq = (T + BQ - 1) / BQ;
  dim3 grid((nq + 1) / 2, H, B);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) {
    static int once = set_smem(attn_fwd2_kernel<128>, attn_fwd2_smem_bytes<128>());
    if (once) return once;
    attn_fwd2_kernel<128><<<grid, F2_THREADS, attn_fwd2_smem_bytes<128>(), s>>>(tq, tv, (__nv_bfloat16*)O, ldo, lse, T, H, Hkv, window,
                                                                              c_log2, status);
  } else {
    static int once = set_smem(attn_fwd2_kernel<64>, attn_fwd2_smem_bytes<64>());
    if (once) return once;
    attn_fwd2_kernel<64><<<grid, F2_THREADS, attn_fwd2_smem_bytes<64>(), s>>>(tq, tv, (__nv_bfloat16*)O, ldo, lse, T, H, Hkv, window,
                                                                            c_log2, status);
  }
  return (int)cudaGetLastError();
}

// Forward with P V on the int8 tensor cores (head_dim 128 only). vq: int8 scratch [B*T, Hkv*D]; vstep: fp32 scratch
// [B, Hkv, ceil(T/128)]; both are written here (the per-block value quantisation) and read by the attention kernel.
extern "C" int otb_attn_fwd_i8pv(const void* qk, long ldqk, const void* qkv, long ldqkv, void* O, long ldo, float* lse, void* vq,
                                 float* vstep, int B, int T, int H, int Hkv, int D, int window, float scale, uint32_t* status,
                                 void* stream) {
  if (D != 128 || H % Hkv || (ldqk & 7) || (ldqkv & 7) || (ldo & 7)) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int nblk = (T + BKV - 1) / BKV;
  const long ldvq = (long)Hkv * D;
  quant_v_kernel<128><<<dim3(nblk, Hkv, B), 256, 0, s>>>((const __nv_bfloat16*)qkv, ldqkv, (H + Hkv) * D, (int8_t*)vq, ldvq, vstep, T, Hkv);
  CUtensorMap tq, tv;
  CUresult r = encode_3d(&tq, qk, (uint64_t)ldqk, (uint64_t)T, (uint64_t)B, (uint64_t)ldqk);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = encode_3d_u8(&tv, vq, (uint64_t)ldvq, (uint64_t)T, (uint64_t)B, (uint64_t)ldvq);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  const float c_log2 = (float)((double)scale * 1.4426950408889634);
  dim3 grid((T + BQ - 1) / BQ, H, B);
  static int once = set_smem(attn_fwd_kernel<128, true>, attn_smem_bytes<128>());
  if (once) return once;
  attn_fwd_kernel<128, true><<<grid, ATT_THREADS, attn_smem_bytes<128>(), s>>>(tq, tv, (__nv_bfloat16*)O, ldo, lse, T, H, Hkv, window,
                                                                               scale, c_log2, vstep, status);
  return (int)cudaGetLastError();
}

// dO, O: [B*T, ld] bf16 (head h at column h*D). Outputs: dqk [B*T, lddqk] (dQ heads then dK heads),
// dV written at column (H + Hkv) * D of dqkv [B*T, lddqkv]; delta: [3, B, H, T] fp32 scratch (delta, -lse, -delta).
extern "C" int otb_attn_bwd(const void* qk, long ldqk, const void* qkv, long ldqkv, const void* O, long ldo,
                            const void* dO, long lddo, const float* lse, float* delta, void* dqk, long lddqk, void* dqkv,
                            long lddqkv, int B, int T, int H, int Hkv, int D, int window, float scale, uint32_t* status,
                            void* stream) {
  if ((D != 64 && D != 128) || H % Hkv || (ldqk & 7) || (ldqkv & 7) || (ldo & 7) || (lddo & 7) || (lddqk & 7) ||
      (lddqkv & 7))
    return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const float c_log2 = (float)((double)scale * 1.4426950408889634);
  CUtensorMap tq, tv, tdo;
  CUresult r = encode_3d(&tq, qk, (uint64_t)ldqk, (uint64_t)T, (uint64_t)B, (uint64_t)ldqk);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = encode_3d(&tv, qkv, (uint64_t)ldqkv, (uint64_t)T, (uint64_t)B, (uint64_t)ldqkv);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = encode_3d(&tdo, dO, (uint64_t)lddo, (uint64_t)T, (uint64_t)B, (uint64_t)lddo);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  const long warps = (long)B * T * H;
  attn_delta_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>((const __nv_bfloat16*)dO, lddo, (const __nv_bfloat16*)O,
                                                               ldo, lse, delta, B, T, H, D);
  __nv_bfloat16* dQp = (__nv_bfloat16*)dqk;
  __nv_bfloat16* dKp = dQp + (long)H * D;
  __nv_bfloat16* dVp = (__nv_bfloat16*)dqkv + (long)(H + Hkv) * D;
  CUtensorMap tk64, tv64;
  r = encode_3d(&tk64, qk, (uint64_t)ldqk, (uint64_t)T, (uint64_t)B, (uint64_t)ldqk, HK);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  r = encode_3d(&tv64, qkv, (uint64_t)ldqkv, (uint64_t)T, (uint64_t)B, (uint64_t)ldqkv, HK);
  if (r != CUDA_SUCCESS) return 1000 + (int)r;
  const int nq = (T + BQ - 1) / BQ;
  dim3 gkv((T + BKV - 1) / BKV, Hkv, B), gq((nq + 1) / 2, H, B);
  const bool kv2 = T % HK == 0;  // the transposed dK/dV kernel walks whole 64-query steps
  const long plane = (long)B * H * T;
  CUtensorMap tq64, tdo64;
  if (kv2) {
    r = encode_3d(&tq64, qk, (uint64_t)ldqk, (uint64_t)T, (uint64_t)B, (uint64_t)ldqk, HK);
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
    r = encode_3d(&tdo64, dO, (uint64_t)lddo, (uint64_t)T, (uint64_t)B, (uint64_t)lddo, HK);
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
  }
  if (D == 128) {
    static int once = set_smem(attn_bwd_kv_kernel<128>, attn_bwd_smem_bytes<128>()) |
                      set_smem(attn_bwd_kv2_kernel<128>, attn_bwd_kv2_smem_bytes<128>()) |
                      set_smem(attn_bwd_q2_kernel<128>, attn_bwd_q2_smem_bytes<128>());
    if (once) return once;
    if (kv2)
      attn_bwd_kv2_kernel<128><<<gkv, ATT_THREADS, attn_bwd_kv2_smem_bytes<128>(), s>>>(
          tq, tv, tq64, tdo64, delta + plane, delta + 2 * plane, dKp, lddqk, dVp, lddqkv, T, H, Hkv, window, scale, c_log2, status);
    else
      attn_bwd_kv_kernel<128><<<gkv, ATT_THREADS, attn_bwd_smem_bytes<128>(), s>>>(tq, tv, tdo, lse, delta, dKp, lddqk, dVp,
                                                                                   lddqkv, T, H, Hkv, window, scale, c_log2, status);
    attn_bwd_q2_kernel<128><<<gq, ATT_THREADS, attn_bwd_q2_smem_bytes<128>(), s>>>(tq, tdo, tk64, tv64, lse, delta, dQp, lddqk, T, H,
                                                                                  Hkv, window, scale, c_log2, status);
  } else {
    static int once = set_smem(attn_bwd_kv_kernel<64>, attn_bwd_smem_bytes<64>()) |
                      set_smem(attn_bwd_kv2_kernel<64>, attn_bwd_kv2_smem_bytes<64>()) |
                      set_smem(attn_bwd_q2_kernel<64>, attn_bwd_q2_smem_bytes<64>());
    if (once) return once;
    if (kv2)
      attn_bwd_kv2_kernel<64><<<gkv, ATT_THREADS, attn_bwd_kv2_smem_bytes<64>(), s>>>(
          tq, tv, tq64, tdo64, delta + plane, delta + 2 * plane, dKp, lddqk, dVp, lddqkv, T, H, Hkv, window, scale, c_log2, status);
    else
      attn_bwd_kv_kernel<64><<<gkv, ATT_THREADS, attn_bwd_smem_bytes<64>(), s>>>(tq, tv, tdo, lse, delta, dKp, lddqk, dVp,
                                                                                 lddqkv, T, H, Hkv, window, scale, c_log2, status);
    attn_bwd_q2_kernel<64><<<gq, ATT_THREADS, attn_bwd_q2_smem_bytes<64>(), s>>>(tq, tdo, tk64, tv64, lse, delta, dQp, lddqk, T, H, Hkv,
                                                                                window, scale, c_log2, status);
  }
  return (int)cudaGetLastError();
}
