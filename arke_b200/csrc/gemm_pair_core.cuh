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
//   warp 6      leader CTA: tile scheduler of the pair (dynamic assignment only)
//
// Barriers: full[s] lives in the leader (expects the bytes of both CTAs); empty[s] and
// acc_full[a] exist in both CTAs and are signalled by one multicast tcgen05.commit; acc_empty[a]
// lives in the leader and counts the eight epilogue warps of the pair.  Every wait is bounded;
// an expired wait records a status code, raises the CTA's abort flag and both CTAs drain to the
// common exit (cluster barrier, then TMEM release).
//
// Tile assignment.  With a device counter (`sched`) the pairs take tiles dynamically: a thread of
// its own in the leader CTA is the pair's scheduler (atomicAdd on the counter; the last pair to
// finish zeroes it) and hands the ids to the other roles through a small ring in the shared
// memory of both CTAs — so the tiles in flight on the GPU are always a contiguous window of the
// tile order, whatever the pairs' relative speed, and pairs that share an operand tile through
// the L2 work on it at the same time.  The scheduler has a warp to itself because its global
// atomic and the cluster-scope release of its remote stores each take a fraction of a
// microsecond: on the producer thread that was measured to cost 5 % of a W8A8 GEMM.  Without a
// counter (`sched == nullptr`) tiles are assigned round robin.
//
// Narrow units for the last wave.  With T tiles on P pairs the last T mod P tiles would run as
// one thin wave while most pairs idle.  When the epilogue policy allows it (`Epi::kSplitN`: every
// output column is finished on its own) each of those tiles is cut into 2 or 4 units along N: a
// unit's MMA has N = 128 or 64 and reads, from the B tile each CTA has staged as usual, only the
// unit's 64 or 32 columns (a start-address offset in the operand descriptor), so the work of the
// last tiles spreads over 2 or 4 times as many pairs.  Every output element is still produced by
// the same sequence of MMAs over K: results do not change.
#pragma once
#include "gemm_core.cuh"

namespace arke {

constexpr int kPairBN = 256;
constexpr int kPairThreads = kGemmThreads + 32;   // + the scheduler warp
constexpr int kSchedRing = 4;   // tile ids in flight between the scheduler thread and the other roles

template <int STAGES>
struct PairSmem {
  static constexpr int kABytes = kGemmBM * kStageKBytes;       // 16 KB: this CTA's 128 rows of A
  static constexpr int kBBytes = (kPairBN / 2) * kStageKBytes; // 16 KB: this CTA's 128 columns of B
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  // full[STAGES] empty[STAGES] acc_full[2] acc_empty[2] sched_full[kSchedRing] sched_empty[kSchedRing]
  static constexpr int kNumBars = 2 * STAGES + 4 + 2 * kSchedRing;
  static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
  // tmem slot (4) + abort flag (4) + pad (8) + ring of tile ids (4 * kSchedRing)
  static constexpr int kEpiOffset = ((kMiscOffset + 16 + 4 * kSchedRing + 127) / 128) * 128;
};

// wait / store forms with cluster scope: the scheduler thread of the leader CTA writes tile ids
// into the peer CTA's shared memory and signals the peer's barrier
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(kTryWaitSuspendNs)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster_abortable(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait_cluster(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) return false;
  }
  return true;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

// The last `tail` tiles of the tile order are cut into `parts` units along N (all zero: none).
struct SplitTail {
  int tail = 0;
  int parts = 1;   // 2 or 4
};
// A unit of work: a whole tile (part = -1) or one N range of a split tile.
struct WorkUnit {
  int tile, part;
};

// One role's view of the tile sequence of its CTA pair.
//   static  (sched == nullptr): tiles pair_id, pair_id + num_pairs, ... (round robin)
//   dynamic (sched != nullptr): the ids the leader's producer thread took from the device counter,
//           read from this CTA's ring after the slot's "full" barrier; the reader then arrives on
//           the leader's "empty" barrier of the slot (eleven readers per slot: each CTA's producer
//           thread and four epilogue warps, and the leader's MMA thread).
struct TileSeq {
  int it = 0;
  int slot = 0;
  uint32_t ph = 0;
};

template <int KIND, bool B_MN, int STAGES, class Epi, bool A_MN = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_pair_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b, const typename Epi::Params ep,
                         int M, int N, int K, int band_m, int* status, unsigned* sched, const SplitTail sp) {
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
  uint64_t* sched_full = acc_empty + 2;          // [kSchedRing] in each CTA: one arrival (the scheduler thread)
  uint64_t* sched_empty = sched_full + kSchedRing;  // [kSchedRing] the leader's copy is used: eleven readers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kMiscOffset);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kMiscOffset + 4);
  volatile int* ring = reinterpret_cast<volatile int*>(smem + SM::kMiscOffset + 16);
  uint8_t* epi_smem = smem + SM::kEpiOffset;

  const int warp = threadIdx.x >> 5;
  const uint32_t rank = cluster_ctarank();      // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * kGemmBM - 1) / (2 * kGemmBM);   // 256-row tile pairs
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const bool dynamic = sched != nullptr;
  // work units: the whole tiles in tile order, then the N ranges of the split tiles
  const int full_tiles = num_tiles - sp.tail;
  const int num_units = full_tiles + sp.tail * sp.parts;
  auto unit_of = [&](int u) -> WorkUnit {
    if (u < full_tiles) return WorkUnit{u, -1};
    const int v = u - full_tiles;
    const int ti = v / sp.parts;
    return WorkUnit{full_tiles + ti, v - ti * sp.parts};
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);    // leader producer's arrive.expect_tx (bytes of both CTAs)
      mbar_init(&empty_bar[i], 1);   // one multicast commit
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);    // one multicast commit
      mbar_init(&acc_empty[i], 8);   // four epilogue warps of each CTA (leader's copy is the one used)
    }
    for (int i = 0; i < kSchedRing; ++i) {
      mbar_init(&sched_full[i], 1);
      mbar_init(&sched_empty[i], 11);
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

  const uint32_t leader_sched_empty0 = mapa_cluster(smem_u32(&sched_empty[0]), 0);

  // Next tile id of this pair for a reading role, or -1 at the end (or after a failed wait, with
  // the abort raised).  `lane0` = this thread signals the slot free (one thread per reading role).
  auto next_tile = [&](TileSeq& q, bool lane0, int fail_code) -> int {
    if (!dynamic) {
      const int t = pair_id + q.it * num_pairs;
      ++q.it;
      return t < num_units ? t : -1;
    }
    // the peer's copy of the ring is written from the leader CTA: cluster-scope acquire there
    const bool got = rank == 0 ? mbar_wait_abortable(&sched_full[q.slot], q.ph, abort_flag)
                               : mbar_wait_cluster_abortable(&sched_full[q.slot], q.ph, abort_flag);
    if (!got) {
      if (lane0) raise_abort(status, abort_flag, fail_code);
      return -1;
    }
    const int t = ring[q.slot];
    if (lane0) {
      if (rank == 0) mbar_arrive(&sched_empty[q.slot]);
      else mbar_arrive_cluster(leader_sched_empty0 + q.slot * 8);
    }
    if (++q.slot == kSchedRing) { q.slot = 0; q.ph ^= 1; }
    return t;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      // One stage of loads for tile coordinates `tc`, k-block `kb` (this CTA's half of the pair's tile).
      auto load_stage = [&](const TileCoord& tc, int kb) -> bool {
        if (!mbar_wait_abortable(&empty_bar[s], ph ^ 1, abort_flag)) {
          raise_abort(status, abort_flag, KSTAT_TIMEOUT_PRODUCER);
          return false;
        }
        const int row0 = tc.m * 2 * kGemmBM + (int)rank * kGemmBM;   // this CTA's rows of A
        const int col0 = tc.n * BN + (int)rank * (BN / 2);           // this CTA's columns of B
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
        return true;
      };

      {
        TileSeq q;
        for (int t = next_tile(q, true, KSTAT_TIMEOUT_PRODUCER); t >= 0 && ok; t = next_tile(q, true, KSTAT_TIMEOUT_PRODUCER)) {
          // (a narrow unit stages the whole B tile like any other: only its MMA is narrower)
          const TileCoord tc = tile_coord(unit_of(t).tile, tiles_m, tiles_n, band_m);
          for (int kb = 0; kb < num_kb && ok; ++kb) ok = load_stage(tc, kb);
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
      TileSeq q;
      for (int t = next_tile(q, true, KSTAT_TIMEOUT_MMA); t >= 0 && ok; t = next_tile(q, true, KSTAT_TIMEOUT_MMA)) {
        if (!mbar_wait_abortable(&acc_empty[a], aph ^ 1, abort_flag)) {
          raise_abort(status, abort_flag, KSTAT_TIMEOUT_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        // a narrow unit: N = BN / parts, and B read from the unit's columns of each CTA's half
        uint32_t idesc_u = idesc_rt, b_off = 0;
        if constexpr (Epi::kSplitN) {
          const WorkUnit un = unit_of(t);
          if (un.part >= 0) {
            idesc_u = (idesc_rt & ~(0x3Fu << 17)) | (static_cast<uint32_t>((BN / sp.parts) >> 3) << 17);
            const int col_off = (BN / 2 / sp.parts) * un.part;   // first of the unit's columns inside a CTA's 128
            if constexpr (B_MN) b_off = (col_off / B_CHUNK_COLS) * B_CHUNK_BYTES + (col_off % B_CHUNK_COLS) * KT::kElemBytes;
            else b_off = col_off * kStageKBytes;                  // K-major: one 128-byte row per column
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_abortable(&full_bar[s], ph, abort_flag)) {
            raise_abort(status, abort_flag, KSTAT_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * SM::kStageBytes);
          const uint32_t sb = sa + SM::kABytes + b_off;
#pragma unroll
          for (int k = 0; k < KSTEPS; ++k) {
            uint64_t adesc;
            if constexpr (!A_MN) adesc = make_smem_desc_sw128(sa + k * (KT::kUmmaK * KT::kElemBytes), 16, 1024);
            else adesc = make_smem_desc_sw128(sa + k * (KT::kUmmaK * kStageKBytes), B_CHUNK_BYTES, 1024);
            uint64_t bdesc;
            if constexpr (!B_MN) bdesc = make_smem_desc_sw128(sb + k * (KT::kUmmaK * KT::kElemBytes), 16, 1024);
            else bdesc = make_smem_desc_sw128(sb + k * (KT::kUmmaK * kStageKBytes), B_CHUNK_BYTES, 1024);
            umma_ss_pair<KIND>(d_tmem, adesc, bdesc, idesc_u, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit_pair(&empty_bar[s], 3);   // frees the stage in both CTAs
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) tc_commit_pair(&acc_full[a], 3);
        a ^= 1;
        if (a == 0) aph ^= 1;
      }
    }
  } else if (warp == 6) {
    // ------------------------------ tile scheduler (leader CTA, dynamic assignment) ------------------------------
    if (dynamic && rank == 0 && elect_one()) {
      const uint32_t peer_ring = mapa_cluster(smem_u32(const_cast<int*>(ring)), 1);
      const uint32_t peer_full0 = mapa_cluster(smem_u32(&sched_full[0]), 1);
      int pslot = 0;
      uint32_t pph = 0;
      bool ok = true;
      // blocks while the ring is full: the scheduler runs at most kSchedRing tiles ahead of the
      // pair's slowest reader, i.e. one or two tiles ahead of the producers
      auto publish = [&](int t) -> bool {
        if (!mbar_wait_cluster_abortable(&sched_empty[pslot], pph ^ 1, abort_flag)) {
          raise_abort(status, abort_flag, KSTAT_TIMEOUT_PRODUCER);
          return false;
        }
        ring[pslot] = t;
        st_cluster_u32(peer_ring + pslot * 4, (uint32_t)t);
        mbar_arrive(&sched_full[pslot]);                 // leader's readers (release, CTA scope)
        mbar_arrive_cluster(peer_full0 + pslot * 8);     // peer's readers (release, cluster scope)
        if (++pslot == kSchedRing) { pslot = 0; pph ^= 1; }
        return true;
      };
      // every pair's first tile is fixed, so nobody waits for the counter at kernel start; the
      // counter hands out the tiles after the first num_pairs
      int t = pair_id < num_units ? pair_id : -1;
      ok = publish(t);
      while (ok && t >= 0) {
        const unsigned nt = atomicAdd(sched, 1u) + (unsigned)num_pairs;
        t = nt < (unsigned)num_units ? (int)nt : -1;
        ok = publish(t);
      }
      // the last scheduler to leave zeroes the counters for the next launch that uses this slot
      if (atomicAdd(sched + 1, 1u) == (unsigned)num_pairs - 1) {
        sched[0] = 0u;
        sched[1] = 0u;
        __threadfence();
      }
    }
  } else {
    // ------------------------------ epilogue warps (both CTAs) ------------------------------
    const int epi_tid = threadIdx.x - 64;
    const bool lane0 = (threadIdx.x & 31) == 0;
    const uint32_t leader_acc_empty0 = mapa_cluster(smem_u32(&acc_empty[0]), 0);
    int a = 0;
    uint32_t aph = 0;
    TileSeq q;
    for (;;) {
      int t = next_tile(q, lane0, KSTAT_TIMEOUT_EPILOGUE);
      t = __shfl_sync(0xffffffffu, t, 0);      // one decision per warp (a lane's wait may have failed)
      if (t < 0) break;
      const WorkUnit un = unit_of(t);
      const TileCoord tc = tile_coord(un.tile, tiles_m, tiles_n, band_m);
      const bool got = mbar_wait_abortable(&acc_full[a], aph, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane0) raise_abort(status, abort_flag, KSTAT_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      bool whole = true;
      if constexpr (Epi::kSplitN) {
        if (un.part >= 0) {
          Epi::tile_part(ep, epi_smem, tmem_base + a * BN, tc.m * 2 + (int)rank, tc.n, M, N, epi_tid, un.part, sp.parts);
          whole = false;
        }
      }
      if (whole) Epi::tile(ep, epi_smem, tmem_base + a * BN, tc.m * 2 + (int)rank, tc.n, M, N, epi_tid);
      tc_fence_before();
      __syncwarp();
      if (lane0) mbar_arrive_cluster(leader_acc_empty0 + a * 8);
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
