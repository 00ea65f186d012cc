// Two-CTA (cta_group::2) variant of the persistent tcgen05 GEMM main loop.
//
//   C_tile[256 x 256] (+)= A[256 x K] * B[K x 256]   per CTA pair (cluster of 2 along M)
//
// Each CTA of the pair stages its own 128 rows of A and its own 128 columns of B (never with
// cluster multicast), and one tcgen05.mma.cta_group::2 issued by the even ("leader") CTA drives
// the tensor cores of both SMs with M = 256, N = 256: per 128 x 256 accumulator each CTA reads
// 16 KB of A and only 16 KB of B from L2 per pipeline stage instead of 16 + 32 KB, which is what
// the one-CTA kernel is limited by at high clocks (L2 -> SM bandwidth).
//
//   warp 0      TMA producer of this CTA (loads signal the leader's "full" barrier)
//   warp 1      leader CTA: MMA issuer; both CTAs: tensor-memory allocation
//   warps 2..5  epilogue of this CTA's 128 rows (same policy classes as the one-CTA kernel)
//
// Barriers: full[s] lives in the leader (expects the bytes of both CTAs); empty[s] and
// acc_full[a] exist in both CTAs and are signalled by one multicast tcgen05.commit; acc_empty[a]
// lives in the leader and counts the eight epilogue warps of the pair.  Every wait is bounded;
// an expired wait records a status code, raises the CTA's abort flag and both CTAs drain to the
// common exit (cluster barrier, then TMEM release).
#pragma once
#include "gemm_core.cuh"

namespace arke {

constexpr int kPairBN = 256;

template <int STAGES>
struct PairSmem {
  static constexpr int kABytes = kGemmBM * kStageKBytes;       // 16 KB: this CTA's 128 rows of A
  static constexpr int kBBytes = (kPairBN / 2) * kStageKBytes; // 16 KB: this CTA's 128 columns of B
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  static constexpr int kNumBars = 2 * STAGES + 4;
  static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
  static constexpr int kEpiOffset = ((kMiscOffset + 16 + 127) / 128) * 128;
};

template <int KIND, bool B_MN, int STAGES, class Epi, bool A_MN = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_pair_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b, const typename Epi::Params ep,
                         int M, int N, int K, int band_m, int* status,
                         unsigned* epoch_ctr = nullptr, int epoch_kb = 0) {
  using KT = KindTraits<KIND>;
  using SM = PairSmem<STAGES>;
  constexpr int BN = kPairBN;
  constexpr int BK = kStageKBytes / KT::kElemBytes;
  constexpr int KSTEPS = BK / KT::kUmmaK;
  constexpr int B_CHUNK_COLS = kStageKBytes / KT::kElemBytes;   // N elements per 128 B (MN-major)
  constexpr int B_CHUNKS = (BN / 2) / B_CHUNK_COLS;             // boxes per stage per CTA (MN-major)
  constexpr int B_CHUNK_BYTES = BK * kStageKBytes;
  constexpr int A_CHUNKS = kGemmBM / B_CHUNK_COLS;              // boxes per stage per CTA when A is MN-major
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SM::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kMiscOffset);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kMiscOffset + 4);
  uint8_t* epi_smem = smem + SM::kEpiOffset;

  const int warp = threadIdx.x >> 5;
  const uint32_t rank = cluster_ctarank();      // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * kGemmBM - 1) / (2 * kGemmBM);   // 256-row tile pairs
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);    // leader producer's arrive.expect_tx (bytes of both CTAs)
      mbar_init(&empty_bar[i], 1);   // one multicast commit
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);    // one multicast commit
      mbar_init(&acc_empty[i], 8);   // four epilogue warps of each CTA (leader's copy is the one used)
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // barriers of both CTAs are initialised before any remote signal
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // set-up above may overlap the previous kernel of the stream; its results are read below

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    // With `epoch_ctr` the producers of all CTAs meet every `epoch_kb` k-blocks (and at every tile
    // start) at an ADVISORY grid barrier: CTAs that share operand tiles through the L2 then stay at
    // the same k offset instead of drifting apart over many tiles or a very long K, which is what
    // turns L2 hits into HBM re-reads.  The barrier is a device counter that every producer
    // increments once per epoch; a producer waits (bounded, ~20 us) until all have arrived and
    // then goes on regardless, so a CTA that is not co-resident only costs the others that wait.
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const int waves = (num_tiles + num_pairs - 1) / num_pairs;
      const int ep_per_tile = (epoch_ctr != nullptr && epoch_kb > 0) ? (num_kb + epoch_kb - 1) / epoch_kb : 0;
      for (int it = 0; it < waves && ok; ++it) {
        const int t = pair_id + it * num_pairs;
        const bool has_tile = t < num_tiles;
        const TileCoord tc = tile_coord(has_tile ? t : 0, tiles_m, tiles_n, band_m);
        const int row0 = tc.m * 2 * kGemmBM + (int)rank * kGemmBM;   // this CTA's rows of A
        const int col0 = tc.n * BN + (int)rank * (BN / 2);           // this CTA's columns of B
        for (int kb = 0; kb < num_kb; ++kb) {
          if (ep_per_tile > 0 && kb % epoch_kb == 0) {
            const unsigned target = (unsigned)(it * ep_per_tile + kb / epoch_kb + 1) * gridDim.x;
            atomicAdd(epoch_ctr, 1u);
            if (has_tile) {
              const long long t0 = clock64();
              while (*reinterpret_cast<volatile unsigned*>(epoch_ctr) < target && clock64() - t0 < 40000LL) __nanosleep(200);
            }
          }
          if (!has_tile) continue;
          if (!mbar_wait_abortable(&empty_bar[s], ph ^ 1, abort_flag)) {
            raise_abort(status, abort_flag, KSTAT_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * SM::kStageBytes;
          uint8_t* sb = sa + SM::kABytes;
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * SM::kStageBytes);
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &tmap_a, &full_bar[s], kb * BK, row0);
          } else {
#pragma unroll
            for (int c = 0; c < A_CHUNKS; ++c)
              tma_load_2d_pair(sa + c * B_CHUNK_BYTES, &tmap_a, &full_bar[s], row0 + c * B_CHUNK_COLS, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tmap_b, &full_bar[s], kb * BK, col0);
          } else {
#pragma unroll
            for (int c = 0; c < B_CHUNKS; ++c)
              tma_load_2d_pair(sb + c * B_CHUNK_BYTES, &tmap_b, &full_bar[s], col0 + c * B_CHUNK_COLS, kb * BK);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (ep_per_tile > 0) {
        // the last producer to leave resets the counters for the next launch that uses this slot
        if (atomicAdd(epoch_ctr + 1, 1u) == gridDim.x - 1) {
          epoch_ctr[0] = 0u;
          epoch_ctr[1] = 0u;
          __threadfence();
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc =
          make_idesc(KIND == KIND_I8 ? UMMA_C_S32 : UMMA_C_F32,
                     KIND == KIND_I8 ? UMMA_S8 : (KIND == KIND_F8 ? UMMA_E4M3 : (KIND == KIND_TF32 ? UMMA_TF32 : 0u)),
                     KIND == KIND_I8 ? UMMA_S8 : (KIND == KIND_F8 ? UMMA_E4M3 : (KIND == KIND_TF32 ? UMMA_TF32 : 0u)), A_MN ? 1u : 0u,
                     B_MN ? 1u : 0u, 2 * kGemmBM, BN);
      const uint32_t idesc_rt = idesc | (KIND == KIND_F16 ? ((ep.ab_format << 7) | (ep.ab_format << 10)) : 0u);
      int s = 0;
      uint32_t ph = 0;
      int a = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait_abortable(&acc_empty[a], aph ^ 1, abort_flag)) {
          raise_abort(status, abort_flag, KSTAT_TIMEOUT_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_abortable(&full_bar[s], ph, abort_flag)) {
            raise_abort(status, abort_flag, KSTAT_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * SM::kStageBytes);
          const uint32_t sb = sa + SM::kABytes;
#pragma unroll
          for (int k = 0; k < KSTEPS; ++k) {
            uint64_t adesc;
            if constexpr (!A_MN) adesc = make_smem_desc_sw128(sa + k * (KT::kUmmaK * KT::kElemBytes), 16, 1024);
            else adesc = make_smem_desc_sw128(sa + k * (KT::kUmmaK * kStageKBytes), B_CHUNK_BYTES, 1024);
            uint64_t bdesc;
            if constexpr (!B_MN) bdesc = make_smem_desc_sw128(sb + k * (KT::kUmmaK * KT::kElemBytes), 16, 1024);
            else bdesc = make_smem_desc_sw128(sb + k * (KT::kUmmaK * kStageKBytes), B_CHUNK_BYTES, 1024);
            umma_ss_pair<KIND>(d_tmem, adesc, bdesc, idesc_rt, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit_pair(&empty_bar[s], 3);   // frees the stage in both CTAs
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) tc_commit_pair(&acc_full[a], 3);
        a ^= 1;
        if (a == 0) aph ^= 1;
      }
    }
  } else {
    // ------------------------------ epilogue warps (both CTAs) ------------------------------
    const int epi_tid = threadIdx.x - 64;
    const uint32_t leader_acc_empty0 = mapa_cluster(smem_u32(&acc_empty[0]), 0);
    int a = 0;
    uint32_t aph = 0;
    for (int t = pair_id; t < num_tiles; t += num_pairs) {
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n, band_m);
      const bool got = mbar_wait_abortable(&acc_full[a], aph, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if ((threadIdx.x & 31) == 0) raise_abort(status, abort_flag, KSTAT_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      Epi::tile(ep, epi_smem, tmem_base + a * BN, tc.m * 2 + (int)rank, tc.n, M, N, epi_tid);
      tc_fence_before();
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive_cluster(leader_acc_empty0 + a * 8);
      a ^= 1;
      if (a == 0) aph ^= 1;
    }
  }

  // common exit: both CTAs meet before either releases tensor memory or leaves (the peer may still
  // signal barriers in this CTA's shared memory until then)
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    if (*abort_flag) {
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) { __nanosleep(1000); }
    }
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace arke
