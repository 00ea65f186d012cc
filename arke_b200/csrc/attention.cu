// Grouped-query flash-attention forward on tcgen05 / TMEM / TMA for sm_100a.
//
// Semantics: ref_grouped_query_attention (arke/ir/ops/reference_impls.py:236-244) =
// F.scaled_dot_product_attention on KV heads repeated Hq/Hkv times; `is_causal` masks keys
// j > i (top-left aligned).  Additionally returns the natural-log logsumexp of the scaled,
// masked scores per query row.
//
// One CTA owns two consecutive 128-row query tiles of one (batch, query head) and walks the
// key/value sequence in 128-key tiles:
//   warps 0-3   softmax + O correction + epilogue for query tile 0 (one thread per row)
//   warps 4-7   the same for query tile 1
//   warp 8      TMA producer: Q tiles once, then a 2-stage ring of K and V tiles (3-D tensor
//               maps {D, S, B*H} so that rows past the sequence end are zero-filled)
//   warp 9      MMA issuer: S_t = Q_t K^T (SS form) and O_t += P_t V (P read from tensor memory,
//               V as MN-major shared-memory operand); the two query tiles are interleaved so
//               the tensor core works on one tile while the other tile's softmax runs
//   (warps 10-11 idle: roles are aligned to warpgroups so that setmaxnreg can move registers
//    from the producer/MMA warpgroup to the two softmax warpgroups)
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each; P_t (16-bit) overwrites
// the first 64 columns of S_t in place.  The running maximum is only moved when it grows by more
// than 2^8 (the accumulator and row sum are then rescaled), which keeps the O read-modify-write
// off the critical path for almost every tile.
#include "common.cuh"
#include "capi_internal.h"
#include <math.h>
#include <stdio.h>

namespace arke {

constexpr int kAttThreads = 384;  // 3 warpgroups: softmax tile 0, softmax tile 1, {producer, MMA, 2 idle}
constexpr int kAttBM = 128;   // query rows per tile
constexpr int kAttBN = 128;   // keys per tile
constexpr float kRescaleThreshold = 8.f;  // log2 units
#ifndef ARKE_ATT_EMU_MASK
#define ARKE_ATT_EMU_MASK 3
#endif
constexpr int kEmuMask = ARKE_ATT_EMU_MASK;  // pairs with (i & mask) == mask use the FMA-pipe exp2: 1 -> half, 3 -> quarter

struct AttParams {
  void* o;
  float* lse;
  int B, Hq, Hkv, S, Skv;
  int causal;
  float scale_log2;  // softmax_scale * log2(e)
  int is_bf16;
  int* status;
};

template <int D>
struct AttSmem {
  static constexpr int kChunks = D / 64;                     // 64-element (128-byte) chunks per row
  static constexpr int kTileBytes = kAttBM * D * 2;          // one 128 x D tile of 16-bit values
  static constexpr int kChunkBytes = kAttBM * 128;           // one 128-row x 128-byte box
  static constexpr int kQOff = 0;                            // Q0, Q1
  static constexpr int kKOff = 2 * kTileBytes;               // K stage 0, 1
  static constexpr int kVOff = 4 * kTileBytes;               // V stage 0, 1
  static constexpr int kBarOff = 6 * kTileBytes;
  // barriers: q_full[2] k_full[2] k_empty[2] v_full[2] v_empty[2] s_full[2] p_ready[2] pv_done[2]
  static constexpr int kNumBars = 18;  // + p_half[2]
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16 + 1024;       // + alignment slack
};

__device__ __forceinline__ bool att_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) return false;
  }
  return true;
}
__device__ __forceinline__ void att_abort(int* status, volatile int* abort_flag, int code) {
  atomicCAS(status, 0, code);
  *abort_flag = 1;
  __threadfence_block();
}

// number of 128-key tiles a query tile starting at row r0 has to visit
__device__ __forceinline__ int kv_tiles_for(int r0, int S, int Skv, int causal) {
  const int all = (Skv + kAttBN - 1) / kAttBN;
  if (!causal) return all;
  int r_last = r0 + kAttBM - 1;
  if (r_last > S - 1) r_last = S - 1;
  if (r_last < 0) r_last = 0;
  int k_last = r_last < Skv - 1 ? r_last : Skv - 1;
  return k_last / kAttBN + 1;
}

// 2^t for a packed pair, t <= 0, on the FMA pipe: n = round(t) by the 1.5*2^23 adder trick,
// f = t - n in [-0.5, 0.5], 2^f by a cubic (minimax fit, max relative error 7.6e-5), then n is
// added into the exponent field.  Inputs below -125 (including -inf of masked keys) give 0.
__device__ __forceinline__ void exp2_poly2(uint64_t t2, float& p0, float& p1) {
  float t0, t1;
  f2_unpack(t2, t0, t1);
  t0 = fmaxf(t0, -125.f);
  t1 = fmaxf(t1, -125.f);
  const uint64_t tc = f2_pack(t0, t1);
  const uint64_t magic = f2_pack(12582912.f, 12582912.f);
  const uint64_t r2 = f2_add(tc, magic);                                       // low bits = n
  const uint64_t n2 = f2_add(r2, f2_pack(-12582912.f, -12582912.f));           // n as float
  const uint64_t f2 = f2_fma(n2, f2_pack(-1.f, -1.f), tc);                     // f = t - n
  uint64_t q = f2_fma(f2, f2_pack(0.05520550534129143f, 0.05520550534129143f), f2_pack(0.24261397123336792f, 0.24261397123336792f));
  q = f2_fma(q, f2, f2_pack(0.6932547688484192f, 0.6932547688484192f));
  q = f2_fma(q, f2, f2_pack(0.9999276995658875f, 0.9999276995658875f));
  float q0, q1, r0, r1;
  f2_unpack(q, q0, q1);
  f2_unpack(r2, r0, r1);
  p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(r0) << 23));
  p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(r1) << 23));
}

template <int D, bool IS_BF16>
__global__ void __launch_bounds__(kAttThreads, 1)
gqa_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const AttParams p) {
  using SM = AttSmem<D>;
  constexpr int KSTEPS_QK = D / 16;
  constexpr int KSTEPS_PV = kAttBN / 16;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL0 = 0, S_COL1 = 128, O_COL0 = 256, O_COL1 = 256 + D;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::kBarOff);
  uint64_t* q_full = bars;          // [2]
  uint64_t* k_full = bars + 2;      // [2]
  uint64_t* k_empty = bars + 4;     // [2]
  uint64_t* v_full = bars + 6;      // [2]
  uint64_t* v_empty = bars + 8;     // [2]
  uint64_t* s_full = bars + 10;     // [2] per query tile
  uint64_t* p_ready = bars + 12;    // [2] per query tile
  uint64_t* pv_done = bars + 14;    // [2] per query tile
  uint64_t* p_half = bars + 16;     // [2] per query tile: first 64 keys of P are in tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kMiscOff + 4);

  const int warp = threadIdx.x >> 5;
  // heaviest (latest) query tiles first: causal work grows with the row index
  const int pair = gridDim.x - 1 - blockIdx.x;
  const int bh = blockIdx.y;                 // b * Hq + hq
  const int b = bh / p.Hq, hq = bh % p.Hq;
  const int kvh = b * p.Hkv + hq / (p.Hq / p.Hkv);
  const int row0 = pair * 2 * kAttBM;        // first row of query tile 0
  const int n_kv0 = kv_tiles_for(row0, p.S, p.Skv, p.causal);
  int n_kv1 = (row0 + kAttBM < p.S) ? kv_tiles_for(row0 + kAttBM, p.S, p.Skv, p.causal) : n_kv0;
  if (n_kv1 < n_kv0) n_kv1 = n_kv0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 10; ++i) mbar_init(&bars[i], 1);
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(&p_ready[0], 4);   // one arrival per softmax warp (lane 0 after __syncwarp)
    mbar_init(&p_ready[1], 4);
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
    mbar_init(&p_half[0], 4);
    mbar_init(&p_half[1], 4);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Register re-balancing between warpgroups: the producer/MMA warpgroup gives registers up, the
  // two softmax warpgroups take them (every warp of a warpgroup executes the same setmaxnreg).
  if (warp >= 8) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
   if (warp == 8) {
    // =============================== TMA producer ===============================
    if (elect_one()) {
      for (int t = 0; t < 2; ++t) {
        mbar_arrive_expect_tx(&q_full[t], SM::kTileBytes);
#pragma unroll
        for (int c = 0; c < SM::kChunks; ++c)
          tma_load_3d(smem + SM::kQOff + t * SM::kTileBytes + c * SM::kChunkBytes, &tmap_q, &q_full[t],
                      c * 64, row0 + t * kAttBM, bh);
      }
      for (int j = 0; j < n_kv1; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!att_wait(&k_empty[s], ph ^ 1, abort_flag)) { att_abort(p.status, abort_flag, KSTAT_TIMEOUT_PRODUCER); break; }
        mbar_arrive_expect_tx(&k_full[s], SM::kTileBytes);
#pragma unroll
        for (int c = 0; c < SM::kChunks; ++c)
          tma_load_3d(smem + SM::kKOff + s * SM::kTileBytes + c * SM::kChunkBytes, &tmap_k, &k_full[s],
                      c * 64, j * kAttBN, kvh);
        if (!att_wait(&v_empty[s], ph ^ 1, abort_flag)) { att_abort(p.status, abort_flag, KSTAT_TIMEOUT_PRODUCER); break; }
        mbar_arrive_expect_tx(&v_full[s], SM::kTileBytes);
#pragma unroll
        for (int c = 0; c < SM::kChunks; ++c)
          tma_load_3d(smem + SM::kVOff + s * SM::kTileBytes + c * SM::kChunkBytes, &tmap_v, &v_full[s],
                      c * 64, j * kAttBN, kvh);
      }
    }
   } else if (warp == 9) {
    // =============================== MMA issuer ===============================
    if (elect_one()) {
      const uint32_t fmt = IS_BF16 ? UMMA_BF16 : UMMA_F16;
      const uint32_t idesc_qk = make_idesc(UMMA_C_F32, fmt, fmt, 0, 0, kAttBM, kAttBN);
      const uint32_t idesc_pv = make_idesc(UMMA_C_F32, fmt, fmt, 0, 1, kAttBM, D);
      const uint32_t q_s = smem_u32(smem + SM::kQOff);
      const uint32_t k_s = smem_u32(smem + SM::kKOff);
      const uint32_t v_s = smem_u32(smem + SM::kVOff);
      bool ok = true;

      // Descriptor words: the high words are constants of the layouts; the low words advance by
      // compile-time offsets inside the unrolled loops (one 32-bit add per operand per MMA).
      const uint32_t hi_k = smem_desc_hi_sw128(1024);
      const uint32_t q_lo0 = smem_desc_lo(q_s, 16), k_lo0 = smem_desc_lo(k_s, 16);
      const uint32_t v_lo0 = smem_desc_lo(v_s, SM::kChunkBytes);
      constexpr uint32_t kTileLo = SM::kTileBytes >> 4;

      auto issue_qk = [&](int t, int j) {  // S_t = Q_t * K_j^T
        const uint32_t qa = q_lo0 + t * kTileLo;
        const uint32_t ka = k_lo0 + (j & 1) * kTileLo;
        const uint32_t d = tmem_base + (t == 0 ? S_COL0 : S_COL1);
#pragma unroll
        for (int k = 0; k < KSTEPS_QK; ++k) {
          const uint32_t off = ((k >> 2) * SM::kChunkBytes + (k & 3) * 32) >> 4;
          if (k == 0) umma_ss_f16_lohi<false>(d, qa + off, hi_k, ka + off, hi_k, idesc_qk);
          else umma_ss_f16_lohi<true>(d, qa + off, hi_k, ka + off, hi_k, idesc_qk);
        }
        tc_commit(&s_full[t]);
      };
      // O_t (+)= P_t * V_j, issued in two halves of 64 keys: the first half starts as soon as the
      // softmax warps have written the first 64 columns of P, while they still work on the rest
      auto issue_pv_half = [&](int t, int j, int half) {
        const uint32_t va = v_lo0 + (j & 1) * kTileLo + half * ((KSTEPS_PV / 2) * 2048 >> 4);
        const uint32_t d = tmem_base + (t == 0 ? O_COL0 : O_COL1);
        const uint32_t pa = tmem_base + (t == 0 ? S_COL0 : S_COL1) + half * ((KSTEPS_PV / 2) * 8);
        // V is MN-major: 16 key rows per step (2048 B); 64-wide head-dim chunks kChunkBytes apart
        if (j == 0 && half == 0) umma_ts_f16_lohi<false>(d, pa, va, hi_k, idesc_pv);
        else umma_ts_f16_lohi<true>(d, pa, va, hi_k, idesc_pv);
#pragma unroll
        for (int kk = 1; kk < KSTEPS_PV / 2; ++kk)
          umma_ts_f16_lohi<true>(d, pa + kk * 8, va + kk * (2048 >> 4), hi_k, idesc_pv);
        if (half == 1) tc_commit(&pv_done[t]);
      };
      auto issue_pv = [&](int t, int j) -> bool {
        const uint32_t jp = j & 1;
        if (!att_wait(&p_half[t], jp, abort_flag) || !att_wait(&v_full[j & 1], (j >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        issue_pv_half(t, j, 0);
        if (!att_wait(&p_ready[t], jp, abort_flag)) return false;
        tc_fence_after();
        issue_pv_half(t, j, 1);
        return true;
      };

      // prologue: S_0(0), S_1(0)
      if (!att_wait(&q_full[0], 0, abort_flag) || !att_wait(&q_full[1], 0, abort_flag) ||
          !att_wait(&k_full[0], 0, abort_flag)) {
        att_abort(p.status, abort_flag, KSTAT_TIMEOUT_MMA);
        ok = false;
      }
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
        issue_qk(1, 0);
        tc_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_kv1 && ok; ++j) {
        const int s = j & 1;
        if (j < n_kv0) {
          if (!issue_pv(0, j)) { ok = false; break; }
          if (j + 1 < n_kv0) {
            if (!att_wait(&k_full[s ^ 1], ((j + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            issue_qk(0, j + 1);
          }
        }
        if (!issue_pv(1, j)) { ok = false; break; }
        tc_commit(&v_empty[s]);
        if (j + 1 < n_kv1) {
          if (!att_wait(&k_full[s ^ 1], ((j + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_qk(1, j + 1);
          tc_commit(&k_empty[s ^ 1]);
        }
      }
      if (!ok) att_abort(p.status, abort_flag, KSTAT_TIMEOUT_MMA);
    }
   }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ===================== softmax / correction / epilogue warps =====================
    const int t = warp >> 2;                     // query tile handled by this warpgroup
    const int quarter = warp & 3;                // TMEM lane quarter this warp may touch
    const int lane = threadIdx.x & 31;
    const int row_in_tile = quarter * 32 + lane;
    const int row = row0 + t * kAttBM + row_in_tile;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + (t == 0 ? S_COL0 : S_COL1);
    const uint32_t o_addr = tmem_base + lane_off + (t == 0 ? O_COL0 : O_COL1);
    const int n_t = t ? n_kv1 : n_kv0;
    const float c = p.scale_log2;
    float m_used = -INFINITY;   // running max (log2 domain, scale included) the sums are based on
    float l = 0.f;              // running sum of 2^(s - m_used)
    bool ok = true;

    for (int j = 0; j < n_t; ++j) {
      const uint32_t jp = j & 1;
      bool got = att_wait(&s_full[t], jp, abort_flag);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * kAttBN;
      // masking is needed only on tiles that cross the causal diagonal or the sequence end
      const int tile_r0 = row0 + t * kAttBM;
      const bool need_mask = (p.causal && (k0 + kAttBN - 1 > tile_r0)) || (k0 + kAttBN > p.Skv);
      int limit = p.Skv - 1;                       // last visible key for this row
      if (p.causal && row < limit) limit = row;
      // ---- the whole 128-key score row goes to registers with one wait ----
      uint32_t v[4][32];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) tmem_ld32(s_addr + ch * 32, v[ch]);
      tmem_ld_wait();
      if (need_mask) {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (k0 + ch * 32 + i > limit) v[ch][i] = 0xff800000u;  // -inf
      }
      // row maximum: 16 independent three-input-max chains of depth 4, then a short tree
      float mc[16];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch)
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int b0 = q4 * 8;
          float a = max3(__uint_as_float(v[ch][b0]), __uint_as_float(v[ch][b0 + 1]), __uint_as_float(v[ch][b0 + 2]));
          a = max3(a, __uint_as_float(v[ch][b0 + 3]), __uint_as_float(v[ch][b0 + 4]));
          a = max3(a, __uint_as_float(v[ch][b0 + 5]), __uint_as_float(v[ch][b0 + 6]));
          mc[ch * 4 + q4] = fmaxf(a, __uint_as_float(v[ch][b0 + 7]));
        }
#pragma unroll
      for (int i = 0; i < 5; ++i) mc[i] = max3(mc[i], mc[5 + 2 * i], mc[6 + 2 * i]);
      mc[0] = max3(mc[0], mc[1], mc[2]);
      const float mx = max3(mc[0], mc[3], fmaxf(mc[4], mc[15]));
      const float m_new = fmaxf(m_used, mx * c);
      // ---- lazy rescale of O and l (warp-uniform decision: TMEM access is warp-collective) ----
      const bool want = (j > 0) && (m_new > m_used + kRescaleThreshold);
      if (j == 0) {
        m_used = m_new;
      } else if (__any_sync(0xffffffffu, want)) {
        got = att_wait(&pv_done[t], (j - 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        tc_fence_after();
        const float alpha = ex2_approx(m_used - m_new);
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t o[32];
          tmem_ld32(o_addr + ch * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(o_addr + ch * 32, o);
        }
        tmem_st_wait();
        l *= alpha;
        m_used = m_new;
      }
      // ---- P = 2^(s*c - m_used), row sum, 16-bit P written over S in place ----
      // The scale-and-subtract and the row sum use packed two-wide fp32 instructions.  Three pairs
      // out of four take the MUFU ex2; the fourth is evaluated on the FMA pipe (round-to-nearest
      // range reduction + cubic polynomial, relative error < 8e-5, below the 16-bit rounding of P)
      // because the special-function unit (16 ex2 per clock per SM) is otherwise as busy as the
      // tensor core.  (Half-precision paired ex2 was measured slower than this mix.)
      const uint64_t c2 = f2_pack(c, c);
      const uint64_t nm2 = f2_pack(-m_used, -m_used);
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint64_t tt = f2_fma(f2_pack(__uint_as_float(v[ch][2 * i]), __uint_as_float(v[ch][2 * i + 1])), c2, nm2);
          float p0, p1;
          if ((i & kEmuMask) == kEmuMask) {
            exp2_poly2(tt, p0, p1);
          } else {
            float t0, t1;
            f2_unpack(tt, t0, t1);
            p0 = ex2_approx(t0);
            p1 = ex2_approx(t1);
          }
          sum2[i & 3] = f2_add(sum2[i & 3], f2_pack(p0, p1));
          pk[i] = IS_BF16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
        }
        tmem_st16(s_addr + ch * 16, pk);
        if (ch == 1) {
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_half[t]);
        }
      }
      {
        float a0, a1;
        f2_unpack(f2_add(f2_add(sum2[0], sum2[1]), f2_add(sum2[2], sum2[3])), a0, a1);
        l += a0 + a1;
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
    }

    // ---- epilogue: O / l -> 16-bit, logsumexp ----
    if (ok) {
      bool got = att_wait(&pv_done[t], (n_t - 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, got)) ok = false;
    }
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      const bool row_ok = row < p.S;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + ((int64_t)bh * p.S + (row_ok ? row : 0)) * D;
      uint32_t ov[D / 32][32];
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) tmem_ld32(o_addr + ch * 32, ov[ch]);
      tmem_ld_wait();
      const int64_t o_first = ((int64_t)bh * p.S + row) * D;
      if (row_ok && ARKE_CHK(o_first, o_first + D - 1, (int64_t)p.B * p.Hq * p.S * D)) {
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float a0 = __uint_as_float(ov[ch][2 * i]) * inv_l, a1 = __uint_as_float(ov[ch][2 * i + 1]) * inv_l;
            w[i] = IS_BF16 ? pack_bf16x2(a0, a1) : pack_f16x2(a0, a1);
          }
          uint4* dst = reinterpret_cast<uint4*>(orow + ch * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
      }
      if (row_ok && p.lse != nullptr && ARKE_CHK((int64_t)bh * p.S + row, (int64_t)bh * p.S + row, (int64_t)p.B * p.Hq * p.S))
        p.lse[(int64_t)bh * p.S + row] = (m_used + log2f(l)) * 0.6931471805599453f;
    } else if (lane == 0) {
      att_abort(p.status, abort_flag, KSTAT_TIMEOUT_SOFTMAX);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    if (*abort_flag) {
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) { __nanosleep(1000); }
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D, bool IS_BF16>
static int launch_gqa(const void* q, const void* k, const void* v, const AttParams& prm, cudaStream_t st) {
  using SM = AttSmem<D>;
  const char* op = "gqa_fwd";
  auto kern = gqa_fwd_kernel<D, IS_BF16>;
  cudaError_t e = ensure_dynamic_smem(kern, SM::kTotal);
  if (e != cudaSuccess) return set_cuda_error("cudaFuncSetAttribute(gqa smem)", e);
  CUtensorMap tq, tk, tv;
  uint32_t box[3] = {64, (uint32_t)kAttBM, 1};
  {
    uint64_t dims[3] = {(uint64_t)D, (uint64_t)prm.S, (uint64_t)prm.B * prm.Hq};
    uint64_t str[2] = {(uint64_t)D * 2, (uint64_t)prm.S * D * 2};
    int rc = make_tensor_map(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, q, dims, str, box, 1, op);
    if (rc != ARKE_OK) return rc;
  }
  {
    uint64_t dims[3] = {(uint64_t)D, (uint64_t)prm.Skv, (uint64_t)prm.B * prm.Hkv};
    uint64_t str[2] = {(uint64_t)D * 2, (uint64_t)prm.Skv * D * 2};
    int rc = make_tensor_map(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, k, dims, str, box, 1, op);
    if (rc != ARKE_OK) return rc;
    rc = make_tensor_map(&tv, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, v, dims, str, box, 1, op);
    if (rc != ARKE_OK) return rc;
  }
  dim3 grid((prm.S + 2 * kAttBM - 1) / (2 * kAttBM), prm.B * prm.Hq);
  kern<<<grid, kAttThreads, SM::kTotal, st>>>(tq, tk, tv, prm);
  e = cudaGetLastError();
  return e == cudaSuccess ? ARKE_OK : set_cuda_error("gqa_fwd launch", e);
}

}  // namespace arke

using namespace arke;

extern "C" int arke_b200_gqa_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                                 int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t S,
                                 int64_t Skv, int64_t D, int causal, float softmax_scale,
                                 void* stream) {
  ARKE_API_ENTER("arke_b200_gqa_fwd");
  const char* op = "gqa_fwd";
  if (dtype != ARKE_BF16 && dtype != ARKE_F16) return set_error(ARKE_ERR_DTYPE, "gqa_fwd: q, k, v must be bf16 or f16");
  if (B < 0 || Hq <= 0 || Hkv <= 0 || S < 0 || Skv < 0 || Hq % Hkv != 0) return set_error(ARKE_ERR_SHAPE, "gqa_fwd: bad shape (need Hq % Hkv == 0)");
  if (D != 64 && D != 128) return set_error(ARKE_ERR_SHAPE, "gqa_fwd: head_dim must be 64 or 128");
  if (B * Hq > 65535 || S > (1 << 30) || Skv > (1 << 30)) return set_error(ARKE_ERR_SHAPE, "gqa_fwd: B*Hq must be <= 65535 and S, Skv <= 2^30");
  if (B == 0 || S == 0) return ARKE_OK;
  if (Skv == 0) return set_error(ARKE_ERR_SHAPE, "gqa_fwd: empty key sequence");
  if (!q || !k || !v || !o) return set_error(ARKE_ERR_ARG, "gqa_fwd: null pointer");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return set_error(ARKE_ERR_ALIGN, "gqa_fwd: q, k, v, o must be 16-byte aligned");
  int rc = require_sm100(op);
  if (rc != ARKE_OK) return rc;
  int* status = kernel_status_ptr();
  if (!status) return ARKE_ERR_CUDA;
  const float scale = softmax_scale > 0.f ? softmax_scale : 1.f / sqrtf((float)D);
  AttParams prm{o, lse, (int)B, (int)Hq, (int)Hkv, (int)S, (int)Skv, causal ? 1 : 0,
                scale * 1.4426950408889634f, dtype == ARKE_BF16 ? 1 : 0, status};
  cudaStream_t st = (cudaStream_t)stream;
  if (D == 128) return dtype == ARKE_BF16 ? launch_gqa<128, true>(q, k, v, prm, st) : launch_gqa<128, false>(q, k, v, prm, st);
  return dtype == ARKE_BF16 ? launch_gqa<64, true>(q, k, v, prm, st) : launch_gqa<64, false>(q, k, v, prm, st);
}
