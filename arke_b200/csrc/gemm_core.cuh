// Persistent, warp-specialised tcgen05 GEMM main loop for sm_100a.
//
//   C_tile[128 x BN] (+)= A[128 x K] * B[K x BN]
//
//   warp 0      : TMA producer  (one elected lane issues cp.async.bulk.tensor loads, no multicast)
//   warp 1      : TMEM allocator + MMA issuer (one elected lane issues tcgen05.mma / commit)
//   warps 2..5  : epilogue (each warp owns the 32 TMEM lanes of its quarter, warp_id % 4)
//
// Operands are staged in a STAGES-deep ring of 128-byte-swizzled shared-memory tiles
// (K extent of a stage = 128 bytes), accumulators are double-buffered in tensor memory
// (2 x BN columns) so the epilogue of tile i overlaps the main loop of tile i+1.
// Every mbarrier wait is bounded; on expiry the waiting role records a code in the status
// word, raises the CTA's abort flag and all roles drain to the common exit where TMEM is freed.
//
// The epilogue is a policy class:
//   struct Epi { struct Params; static constexpr int kSmemBytes;
//     static __device__ void tile(const Params&, uint8_t* smem, uint32_t tmem_acc,
//                                 int tile_m, int tile_n, int M, int N, int epi_tid); };
// `tmem_acc` is the TMEM address (lane 0) of the finished accumulator; epi_tid is 0..127 and
// the calling thread may read TMEM lanes 32*(warp_id%4) .. +31 only.
#pragma once
#include "common.cuh"

namespace arke {

template <int KIND> struct KindTraits;
template <> struct KindTraits<KIND_I8> { static constexpr int kElemBytes = 1; static constexpr int kUmmaK = 32; };
template <> struct KindTraits<KIND_F8> { static constexpr int kElemBytes = 1; static constexpr int kUmmaK = 32; };
template <> struct KindTraits<KIND_F16> { static constexpr int kElemBytes = 2; static constexpr int kUmmaK = 16; };
template <> struct KindTraits<KIND_TF32> { static constexpr int kElemBytes = 4; static constexpr int kUmmaK = 8; };

constexpr int kGemmBM = 128;
constexpr int kGemmThreads = 192;
constexpr int kStageKBytes = 128;  // K extent of one pipeline stage, in bytes (= swizzle span)

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int kABytes = kGemmBM * kStageKBytes;  // 16 KB
  static constexpr int kBBytes = BN * kStageKBytes;       // 16/32 KB
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], then tmem ptr + abort flag
  static constexpr int kNumBars = 2 * STAGES + 4;
  static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
  static constexpr int kEpiOffset = ((kMiscOffset + 16 + 127) / 128) * 128;
};

__device__ __forceinline__ bool mbar_wait_abortable(uint64_t* bar, uint32_t parity,
                                                    volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) return false;
  }
  return true;
}

__device__ __forceinline__ void raise_abort(int* status, volatile int* abort_flag, int code) {
  atomicCAS(status, 0, code);
  *abort_flag = 1;
  __threadfence_block();
}

// tile index -> (tile_m, tile_n).  band_m > 0: M is the fast index inside a band of `band_m`
// M-tiles and N sweeps once per band: the CTAs running at the same time share a few B (weight)
// tiles, and the band's A tiles (band_m x 128 rows x K) stay resident in L2 while B streams
// through, so B is read from HBM ceil(tiles_m / band_m) times and A once.  band_m >= tiles_m gives
// plain M-fastest order (everything L2-resident).  band_m < 0 is the mirrored order for a B that
// is the smaller operand: bands of -band_m N-tiles whose B columns stay resident, N fastest inside
// a band, M sweeping once per band (A is then read ceil(tiles_n / -band_m) times).
struct TileCoord { int m, n; };
__device__ __forceinline__ TileCoord tile_coord(int t, int tiles_m, int tiles_n, int band_m) {
  if (band_m < 0) {
    const int band_n = -band_m;
    const int band_tiles = band_n * tiles_m;
    const int g = t / band_tiles;
    const int r = t - g * band_tiles;
    const int n0 = g * band_n;
    const int bn = min(band_n, tiles_n - n0);  // the last band may be narrower
    return {r / bn, n0 + r % bn};
  }
  const int band_tiles = band_m * tiles_n;
  const int g = t / band_tiles;
  const int r = t - g * band_tiles;
  const int m0 = g * band_m;
  const int bm = min(band_m, tiles_m - m0);  // the last band may be narrower
  return {m0 + r % bm, r / bm};
}

template <int KIND, bool B_MN, int BN, int STAGES, class Epi, bool A_MN = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b, const typename Epi::Params ep,
                    int M, int N, int K, int band_m, int* status) {
  using KT = KindTraits<KIND>;
  using SM = GemmSmem<BN, STAGES>;
  constexpr int BK = kStageKBytes / KT::kElemBytes;          // K elements per stage
  constexpr int KSTEPS = BK / KT::kUmmaK;                     // MMAs per stage (= 4)
  constexpr int B_CHUNK_COLS = kStageKBytes / KT::kElemBytes; // N elements per 128 B (MN-major)
  constexpr int B_CHUNKS = BN / B_CHUNK_COLS;                 // TMA boxes per stage (MN-major)
  constexpr int B_CHUNK_BYTES = BK * kStageKBytes;            // bytes of one MN-major box
  constexpr int A_CHUNKS = kGemmBM / B_CHUNK_COLS;            // boxes per stage when A is MN-major
  constexpr uint32_t TMEM_COLS = 2 * BN;
  static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM columns: power of 2 <= 512");

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: round up to the swizzle atom
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SM::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kMiscOffset);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kMiscOffset + 4);
  uint8_t* epi_smem = smem + SM::kEpiOffset;

  const int warp = threadIdx.x >> 5;
  const int tiles_m = (M + kGemmBM - 1) / kGemmBM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // set-up above may overlap the previous kernel of the stream; its results are read below

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n, band_m);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_abortable(&empty_bar[s], ph ^ 1, abort_flag)) {
            raise_abort(status, abort_flag, KSTAT_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * SM::kStageBytes;
          uint8_t* sb = sa + SM::kABytes;
          mbar_arrive_expect_tx(&full_bar[s], SM::kStageBytes);
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmap_a, &full_bar[s], kb * BK, tc.m * kGemmBM);
          } else {
#pragma unroll
            for (int c = 0; c < A_CHUNKS; ++c)
              tma_load_2d(sa + c * B_CHUNK_BYTES, &tmap_a, &full_bar[s],
                          tc.m * kGemmBM + c * B_CHUNK_COLS, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tmap_b, &full_bar[s], kb * BK, tc.n * BN);
          } else {
#pragma unroll
            for (int c = 0; c < B_CHUNKS; ++c)
              tma_load_2d(sb + c * B_CHUNK_BYTES, &tmap_b, &full_bar[s],
                          tc.n * BN + c * B_CHUNK_COLS, kb * BK);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc =
          make_idesc(KIND == KIND_I8 ? UMMA_C_S32 : UMMA_C_F32,
                     KIND == KIND_I8 ? UMMA_S8 : (KIND == KIND_F8 ? UMMA_E4M3 : (KIND == KIND_TF32 ? UMMA_TF32 : 0u)),
                     KIND == KIND_I8 ? UMMA_S8 : (KIND == KIND_F8 ? UMMA_E4M3 : (KIND == KIND_TF32 ? UMMA_TF32 : 0u)), A_MN ? 1u : 0u,
                     B_MN ? 1u : 0u, kGemmBM, BN);
      // for KIND_F16 the a/b format (f16 = 0 / bf16 = 1) is a run-time property of the call
      const uint32_t idesc_rt = idesc | (KIND == KIND_F16 ? ((ep.ab_format << 7) | (ep.ab_format << 10)) : 0u);
      int s = 0;
      uint32_t ph = 0;
      int a = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
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
            // A K-major: step 32 bytes along the swizzled 128-byte row; A MN-major ([K,M] in
            // memory): same layout as an MN-major B (below)
            uint64_t adesc;
            if constexpr (!A_MN) adesc = make_smem_desc_sw128(sa + k * (KT::kUmmaK * KT::kElemBytes), 16, 1024);
            else adesc = make_smem_desc_sw128(sa + k * (KT::kUmmaK * kStageKBytes), B_CHUNK_BYTES, 1024);
            uint64_t bdesc;
            if constexpr (!B_MN) {
              bdesc = make_smem_desc_sw128(sb + k * (KT::kUmmaK * KT::kElemBytes), 16, 1024);
            } else {
              // B is MN-major: one K row = 128 B of N; step kUmmaK rows; 128 B-wide N chunks
              // are B_CHUNK_BYTES apart (LBO), groups of 8 K rows 1024 B apart (SBO)
              bdesc = make_smem_desc_sw128(sb + k * (KT::kUmmaK * kStageKBytes), B_CHUNK_BYTES, 1024);
            }
            umma_ss<KIND>(d_tmem, adesc, bdesc, idesc_rt, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) tc_commit(&acc_full[a]);
        a ^= 1;
        if (a == 0) aph ^= 1;
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const int epi_tid = threadIdx.x - 64;
    int a = 0;
    uint32_t aph = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n, band_m);
      // the outcome is made warp-uniform: a warp either runs the whole tile epilogue (which
      // contains warp-collective tcgen05.ld) or leaves as one; warps never wait on each other
      const bool got = mbar_wait_abortable(&acc_full[a], aph, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if ((threadIdx.x & 31) == 0) raise_abort(status, abort_flag, KSTAT_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      Epi::tile(ep, epi_smem, tmem_base + a * BN, tc.m, tc.n, M, N, epi_tid);
      tc_fence_before();
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(&acc_empty[a]);
      a ^= 1;
      if (a == 0) aph ^= 1;
    }
  }

  // common exit: every role ends up here (normally or after an expired wait)
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // give copies / MMAs still in flight time to land before the memory is released
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) { __nanosleep(1000); }
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace arke
