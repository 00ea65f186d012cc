// Quantised GEMM (INT8 x INT8 -> int32, e4m3 x e4m3 -> fp32) with a fused per-row x per-channel
// dequantising epilogue, and the dense 16-bit GEMM, on the tcgen05 main loop of gemm_core.cuh.
//
// Semantics: composition of quantize_per_token, matmul and dequantize_per_channel of the
// reference (arke/ir/ops/reference_impls.py:118-119, 215-224):
//   acc = A @ W (exact int32, or fp32);  Y = out_dtype((float(acc) * sa[i]) * sw[j]).
#include "gemm_core.cuh"
#include "gemm_pair_core.cuh"
#include "capi_internal.h"
#include <stdio.h>
#include <stdlib.h>

namespace arke {

template <int KIND, int BN>
struct EpiStore {
  struct Params {
    const float* sa;    // per-row scale or nullptr
    const float* sw;    // per-column scale or nullptr
    void* y;            // scaled output or nullptr
    void* acc;          // raw accumulators (int32 / fp32) or nullptr
    int64_t ldy, ldacc;
    int y_dtype;        // ARKE_BF16 / ARKE_F16 / ARKE_F32
    int vec_y, vec_acc; // rows are 16-byte aligned: 128-bit stores allowed
    uint32_t ab_format; // KIND_F16 only: 0 = f16, 1 = bf16
    const float* alpha = nullptr;  // device scalar multiplied into every row scale, or nullptr
  };
  static constexpr int kSmemBytes = 4 * BN * 4;  // one copy of the tile's column scales per warp

  static __device__ __forceinline__ float to_f(uint32_t v) {
    if constexpr (KIND == KIND_I8) return (float)(int)v;
    else return __uint_as_float(v);
  }

  // every output column is finished on its own: a tile may be cut into narrower units along N
  static constexpr bool kSplitN = true;

  // the tile's column scales, one copy per epilogue warp
  static __device__ __forceinline__ const float* stage_col_scales(const Params& p, uint8_t* smem, int tile_n, int N, int epi_tid) {
    const int lane = threadIdx.x & 31;
    float* sw_s = reinterpret_cast<float*>(smem) + (epi_tid >> 5) * BN;
    const int col_base = tile_n * BN;
    __syncwarp();
    for (int j = lane; j < BN; j += 32) {
      const int col = col_base + j;
      sw_s[j] = (p.sw != nullptr && col < N) ? __ldg(p.sw + col) : 1.f;
    }
    __syncwarp();
    return sw_s;
  }

  // 32 accumulator columns of one row -> output columns [col0, col0 + 32) of the requested outputs
  static __device__ __forceinline__ void emit_chunk(const Params& p, const uint32_t (&v)[32], const float* sws, float sa,
                                                    int row, bool row_ok, int col0, int M, int N) {
    const bool full = col0 + 32 <= N;
    // checked build: this thread's 32 (or fewer) columns of row `row` lie inside the outputs
    const int last_col = (col0 + 31 < N ? col0 + 31 : N - 1);
    if (p.acc != nullptr && row_ok && ARKE_CHK((int64_t)row * p.ldacc + col0, (int64_t)row * p.ldacc + last_col, span_elems(M, N, p.ldacc))) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(p.acc) + (int64_t)row * p.ldacc + col0;
      if (full && p.vec_acc) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (col0 + i < N) dst[i] = v[i];
      }
    }
    if (p.y != nullptr && row_ok && ARKE_CHK((int64_t)row * p.ldy + col0, (int64_t)row * p.ldy + last_col, span_elems(M, N, p.ldy))) {
      float f[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = (to_f(v[i]) * sa) * sws[i];
      if (p.y_dtype == ARKE_F32) {
        float* dst = reinterpret_cast<float*>(p.y) + (int64_t)row * p.ldy + col0;
        if (full && p.vec_y) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            reinterpret_cast<float4*>(dst)[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < N) dst[i] = f[i];
        }
      } else {
        const bool bf = p.y_dtype == ARKE_BF16;
        uint16_t* dst = reinterpret_cast<uint16_t*>(p.y) + (int64_t)row * p.ldy + col0;
        if (full && p.vec_y) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            w[i] = bf ? pack_bf16x2(f[2 * i], f[2 * i + 1]) : pack_f16x2(f[2 * i], f[2 * i + 1]);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (col0 + i < N) {
              dst[i] = bf ? __bfloat16_as_ushort(__float2bfloat16_rn(f[i]))
                          : __half_as_ushort(__float2half_rn(f[i]));
            }
          }
        }
      }
    }
  }

  static __device__ void tile(const Params& p, uint8_t* smem, uint32_t tmem_acc, int tile_m,
                              int tile_n, int M, int N, int epi_tid) {
    const int q = (threadIdx.x >> 5) & 3;  // TMEM lane quarter this warp may read
    const int lane = threadIdx.x & 31;
    const float* sw_s = stage_col_scales(p, smem, tile_n, N, epi_tid);
    const int col_base = tile_n * BN;
    const int row = tile_m * kGemmBM + q * 32 + lane;
    const bool row_ok = row < M;
    float sa = (p.sa != nullptr && row_ok) ? __ldg(p.sa + row) : 1.f;
    if (p.alpha != nullptr) sa *= __ldg(p.alpha);   // (left alone when absent: quantised outputs keep their bits)
    const uint32_t taddr = tmem_acc + (static_cast<uint32_t>(q * 32) << 16);

#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      const int col0 = col_base + c * 32;
      if (col0 >= N) break;  // uniform over the CTA
      uint32_t v[32];
      tmem_ld32(taddr + c * 32, v);
      tmem_ld_wait();
      emit_chunk(p, v, sw_s + c * 32, sa, row, row_ok, col0, M, N);
    }
  }

  // Unit `part` of `parts` (2 or 4) of a tile cut along N in the CTA-pair kernel.  The pair's
  // MMA had N = BN / parts: accumulator columns [0, n_half) come from the leader CTA's half of
  // the B tile and [n_half, 2 n_half) from the peer's, each starting at column n_half * part of
  // that half (n_half = BN / 2 / parts = 64 or 32).
  static __device__ void tile_part(const Params& p, uint8_t* smem, uint32_t tmem_acc, int tile_m,
                                   int tile_n, int M, int N, int epi_tid, int part, int parts) {
    const int q = (threadIdx.x >> 5) & 3;
    const int lane = threadIdx.x & 31;
    const float* sw_s = stage_col_scales(p, smem, tile_n, N, epi_tid);
    const int col_base = tile_n * BN;
    const int row = tile_m * kGemmBM + q * 32 + lane;
    const bool row_ok = row < M;
    float sa = (p.sa != nullptr && row_ok) ? __ldg(p.sa + row) : 1.f;
    if (p.alpha != nullptr) sa *= __ldg(p.alpha);
    const uint32_t taddr = tmem_acc + (static_cast<uint32_t>(q * 32) << 16);
    const int n_half = BN / 2 / parts;
#pragma unroll 1
    for (int c = 0; c < (BN / parts) / 32; ++c) {
      const int j0 = c * 32;                                   // first accumulator column of the chunk
      const int in_tile = (j0 / n_half) * (BN / 2) + n_half * part + (j0 % n_half);
      const int col0 = col_base + in_tile;
      if (col0 >= N) continue;  // uniform over the CTA
      uint32_t v[32];
      tmem_ld32(taddr + j0, v);
      tmem_ld_wait();
      emit_chunk(p, v, sw_s + in_tile, sa, row, row_ok, col0, M, N);
    }
  }
};

// --------------------------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------------------------
unsigned* pair_sched_counter(int tiles, int pairs);

struct GemmOperands {
  const void* a; int64_t lda;      // per layout
  const void* b; int64_t ldb;      // per layout
  int b_mn;                        // 1: B is [K,N] with N contiguous; 0: B is [N,K] with K contiguous
  int M, N, K;
  int elem_bytes;
  int a_mn = 0;                    // 1: A is [K,M] with M contiguous (C = A^T B); 0: A is [M,K]
};

static int build_maps(const GemmOperands& g, int BN, CUtensorMap* ta, CUtensorMap* tb, const char* op) {
  const CUtensorMapDataType dt = g.elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : (g.elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32);
  const uint32_t bk = 128 / g.elem_bytes;
  if (!g.a_mn) {
    uint64_t dims[2] = {(uint64_t)g.K, (uint64_t)g.M};
    uint64_t str[1] = {(uint64_t)g.lda * g.elem_bytes};
    uint32_t box[2] = {bk, (uint32_t)kGemmBM};
    int rc = make_tensor_map(ta, dt, 2, g.a, dims, str, box, 1, op);
    if (rc != ARKE_OK) return rc;
  } else {
    uint64_t dims[2] = {(uint64_t)g.M, (uint64_t)g.K};
    uint64_t str[1] = {(uint64_t)g.lda * g.elem_bytes};
    uint32_t box[2] = {bk /* 128 bytes of M */, bk /* K rows of one stage */};
    int rc = make_tensor_map(ta, dt, 2, g.a, dims, str, box, 1, op);
    if (rc != ARKE_OK) return rc;
  }
  if (!g.b_mn) {
    uint64_t dims[2] = {(uint64_t)g.K, (uint64_t)g.N};
    uint64_t str[1] = {(uint64_t)g.ldb * g.elem_bytes};
    uint32_t box[2] = {bk, (uint32_t)BN};
    return make_tensor_map(tb, dt, 2, g.b, dims, str, box, 1, op);
  }
  uint64_t dims[2] = {(uint64_t)g.N, (uint64_t)g.K};
  uint64_t str[1] = {(uint64_t)g.ldb * g.elem_bytes};
  uint32_t box[2] = {bk /* 128 bytes of N */, bk /* K rows of one stage */};
  return make_tensor_map(tb, dt, 2, g.b, dims, str, box, 1, op);
}

static int check_gemm_operands(const GemmOperands& g, const char* op) {
  char buf[256];
  if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.b) & 15)) {
    snprintf(buf, sizeof(buf), "%s: operand pointers must be 16-byte aligned", op);
    return set_error(ARKE_ERR_ALIGN, buf);
  }
  if ((g.lda * g.elem_bytes) % 16 != 0 || (g.ldb * g.elem_bytes) % 16 != 0) {
    snprintf(buf, sizeof(buf), "%s: operand row strides must be multiples of 16 bytes (lda=%lld, ldb=%lld elements)",
             op, (long long)g.lda, (long long)g.ldb);
    return set_error(ARKE_ERR_ALIGN, buf);
  }
  if (g.lda < (g.a_mn ? g.M : g.K) || g.ldb < (g.b_mn ? g.N : g.K)) {
    snprintf(buf, sizeof(buf), "%s: row stride smaller than the row length", op);
    return set_error(ARKE_ERR_SHAPE, buf);
  }
  return ARKE_OK;
}

// Launch with programmatic stream serialization: the kernel's set-up (barrier init, tensor-memory
// allocation, descriptor prefetch) may overlap the tail of the previous kernel in the stream; the
// kernel itself waits (griddepcontrol.wait) before it reads any input.
template <class Kern, class... Args>
static cudaError_t launch_pdl(Kern kern, int grid, int threads, int smem_bytes, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3((unsigned)threads, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// M-tiles per band.  When A and B together fit comfortably in L2 everything stays resident and
// plain M-fastest order is used; otherwise one band of A (band_m x 128 rows x K) is limited to a
// budget (default 32 MB) that leaves room for the streaming B tiles.
int gemm_band_m(int M, int N, int K, int elem_bytes) {
  const int tiles_m = (M + kGemmBM - 1) / kGemmBM;
  const long long a_bytes = (long long)M * K * elem_bytes, b_bytes = (long long)N * K * elem_bytes;
  if (a_bytes + b_bytes <= (100ll << 20)) return tiles_m;
  long long budget = 32ll << 20;
  if (const int mb = tuning_options().gemm_band_mb) budget = (long long)mb << 20;        // caller's choice
  const long long tile_bytes = (long long)kGemmBM * K * elem_bytes;
  long long band = budget / (tile_bytes > 0 ? tile_bytes : 1);
  if (band < 1) band = 1;
  if (band > tiles_m) band = tiles_m;
  const int nbands = (int)((tiles_m + band - 1) / band);  // spread the tiles evenly over the bands
  return (tiles_m + nbands - 1) / nbands;
}

// Signed band for the plain GEMM launchers: > 0 = M-tiles per band (see gemm_band_m), < 0 = minus
// the number of N-tiles (of `bn` columns) per band, chosen when B is the smaller operand and at
// least two of its tile columns fit the budget: B's band stays in L2 and A streams.
static int gemm_band(int M, int N, int K, int elem_bytes, int bn) {
  const long long a_bytes = (long long)M * K * elem_bytes, b_bytes = (long long)N * K * elem_bytes;
  if (a_bytes + b_bytes <= (100ll << 20) || b_bytes >= a_bytes) return gemm_band_m(M, N, K, elem_bytes);
  long long budget = 32ll << 20;
  if (const int mb = tuning_options().gemm_band_mb) budget = (long long)mb << 20;        // caller's choice
  const long long col_bytes = (long long)bn * K * elem_bytes;
  if (2 * col_bytes > budget) return gemm_band_m(M, N, K, elem_bytes);
  const int tiles_n = (N + bn - 1) / bn;
  const int nbands = (int)((b_bytes + budget - 1) / budget);
  int band = (tiles_n + nbands - 1) / nbands;
  if (band < 1) band = 1;
  return -band;
}

template <int KIND, bool B_MN, int BN, int STAGES, bool A_MN = false>
static int launch_gemm(const GemmOperands& g, const typename EpiStore<KIND, BN>::Params& ep,
                       cudaStream_t st, const char* op) {
  using Epi = EpiStore<KIND, BN>;
  using SM = GemmSmem<BN, STAGES>;
  constexpr int smem_bytes = SM::kEpiOffset + Epi::kSmemBytes + 1024;
  static_assert(smem_bytes <= 227 * 1024, "shared memory budget");
  auto kern = gemm_tcgen05_kernel<KIND, B_MN, BN, STAGES, Epi, A_MN>;
  cudaError_t e = ensure_dynamic_smem(kern, smem_bytes);
  if (e != cudaSuccess) return set_cuda_error("cudaFuncSetAttribute(gemm smem)", e);
  CUtensorMap ta, tb;
  int rc = build_maps(g, BN, &ta, &tb, op);
  if (rc != ARKE_OK) return rc;
  int* status = kernel_status_ptr();
  if (!status) return ARKE_ERR_CUDA;
  const int tiles = ((g.M + kGemmBM - 1) / kGemmBM) * ((g.N + BN - 1) / BN);
  int grid = sm_count();
  if (grid <= 0) return ARKE_ERR_CUDA;
  if (tiles < grid) grid = tiles;
  e = launch_pdl(kern, grid, kGemmThreads, smem_bytes, st, ta, tb, ep, g.M, g.N, g.K, gemm_band(g.M, g.N, g.K, g.elem_bytes, BN), status);
  return e == cudaSuccess ? ARKE_OK : set_cuda_error(op, e);
}

// How the last `tiles mod pairs` tiles of a CTA-pair GEMM are cut along N (into 4 or 2 units each)
// so that the thin last wave spreads over more pairs: only while the units of that wave still fit
// the pairs once.  All zero: no narrow units.
static SplitTail plan_split_tail(int tiles, int pairs) {
  SplitTail sp{};
  if (pairs <= 0 || tuning_options().gemm_no_split) return sp;
  const int tail = tiles % pairs;
  if (tail == 0) return sp;
  if (4 * tail <= pairs) sp.parts = 4;
  else if (2 * tail <= pairs) sp.parts = 2;
  else return sp;
  sp.tail = tail;
  return sp;
}

// Two-CTA (cta_group::2) launch: 256 x 256 tile per CTA pair, 6 stages of 32 KB per CTA.
template <int KIND, bool B_MN, bool A_MN = false>
static int launch_gemm_pair(const GemmOperands& g, const typename EpiStore<KIND, 256>::Params& ep,
                            cudaStream_t st, const char* op) {
  using Epi = EpiStore<KIND, 256>;
  constexpr int STAGES = 6;
  using SM = PairSmem<STAGES>;
  constexpr int smem_bytes = SM::kEpiOffset + Epi::kSmemBytes + 1024;
  static_assert(smem_bytes <= 227 * 1024, "shared memory budget");
  auto kern = gemm_pair_tcgen05_kernel<KIND, B_MN, STAGES, Epi, A_MN>;
  cudaError_t e = ensure_dynamic_smem(kern, smem_bytes);
  if (e != cudaSuccess) return set_cuda_error("cudaFuncSetAttribute(gemm pair smem)", e);
  CUtensorMap ta, tb;
  int rc = build_maps(g, 128 /* each CTA stages half of the 256 B columns */, &ta, &tb, op);
  if (rc != ARKE_OK) return rc;
  int* status = kernel_status_ptr();
  if (!status) return ARKE_ERR_CUDA;
  const int tiles = ((g.M + 2 * kGemmBM - 1) / (2 * kGemmBM)) * ((g.N + 255) / 256);
  int grid = sm_count() & ~1;
  if (grid <= 0) return ARKE_ERR_CUDA;
  const SplitTail sp = plan_split_tail(tiles, grid / 2);
  const int units = tiles - sp.tail + sp.tail * sp.parts;
  if (2 * units < grid) grid = 2 * units;
  int band = gemm_band(g.M, g.N, g.K, g.elem_bytes, 256);
  if (band > 0) band = (band + 1) / 2;   // M bands are counted in 256-row pairs here
  e = launch_pdl(kern, grid, kPairThreads, smem_bytes, st, ta, tb, ep, g.M, g.N, g.K, band, status, pair_sched_counter(units, grid / 2), sp);
  return e == cudaSuccess ? ARKE_OK : set_cuda_error(op, e);
}

// Device counter for the pair kernel's dynamic tile assignment, or nullptr for round robin: one
// wave of tiles (or the caller's option) needs no scheduler.
unsigned* pair_sched_counter(int tiles, int pairs) {
  if (tuning_options().gemm_static_sched || tiles <= pairs) return nullptr;
  return sched_counter_slot();
}

// The CTA-pair kernel pays off on large problems; small ones keep the one-CTA kernel (finer tiles).
static bool use_pair_kernel(const GemmOperands& g) {
  if (const int tm = tuning_options().gemm_tile_m) return tm == 256;              // caller's choice
  return g.M >= 1024 && g.N >= 1024;
}

template <int KIND>
static int dispatch_gemm(const GemmOperands& g, const void* sa, const void* sw, void* y, int y_dtype,
                         int64_t ldy, void* acc, int64_t ldacc, uint32_t ab_format,
                         cudaStream_t st, const char* op, const float* alpha = nullptr) {
  const int y_es = y_dtype == ARKE_F32 ? 4 : 2;
  const int vec_y = y && (reinterpret_cast<uintptr_t>(y) % 16 == 0) && ((ldy * y_es) % 16 == 0);
  const int vec_acc = acc && (reinterpret_cast<uintptr_t>(acc) % 16 == 0) && ((ldacc * 4) % 16 == 0);
#define ARKE_G(BMN, BN_, ST_)                                                                  \
  do {                                                                                         \
    typename EpiStore<KIND, BN_>::Params ep{(const float*)sa, (const float*)sw, y, acc, ldy,   \
                                            ldacc, y_dtype, vec_y, vec_acc, ab_format, alpha}; \
    return launch_gemm<KIND, BMN, BN_, ST_>(g, ep, st, op);                                    \
  } while (0)
  if constexpr (KIND == KIND_F16) {
    if (g.a_mn) {   // C = A^T B (16-bit operands only): 256-column tiles, both kernel forms
      typename EpiStore<KIND, 256>::Params ep{(const float*)sa, (const float*)sw, y, acc, ldy,
                                              ldacc, y_dtype, vec_y, vec_acc, ab_format, alpha};
      if (use_pair_kernel(g)) {
        if (g.b_mn) return launch_gemm_pair<KIND, true, true>(g, ep, st, op);
        return launch_gemm_pair<KIND, false, true>(g, ep, st, op);
      }
      if (g.b_mn) return launch_gemm<KIND, true, 256, 4, true>(g, ep, st, op);
      return launch_gemm<KIND, false, 256, 4, true>(g, ep, st, op);
    }
  }
  if (use_pair_kernel(g)) {
    typename EpiStore<KIND, 256>::Params ep{(const float*)sa, (const float*)sw, y, acc, ldy,
                                            ldacc, y_dtype, vec_y, vec_acc, ab_format, alpha};
    if (g.b_mn) return launch_gemm_pair<KIND, true>(g, ep, st, op);
    return launch_gemm_pair<KIND, false>(g, ep, st, op);
  }
  if (g.N <= 128) {
    if (g.b_mn) ARKE_G(true, 128, 6);
    ARKE_G(false, 128, 6);
  }
  if (g.b_mn) ARKE_G(true, 256, 4);
  ARKE_G(false, 256, 4);
#undef ARKE_G
}

int gemm_16bit(const void* a, int64_t lda, int a_mn, const void* b, int64_t ldb, int b_mn, int dtype,
               int M, int N, int K, void* c, int c_dtype, int64_t ldc, cudaStream_t st, const char* op,
               const float* alpha) {
  GemmOperands g{a, lda, b, ldb, b_mn, M, N, K, 2, a_mn};
  int rc = check_gemm_operands(g, op);
  if (rc != ARKE_OK) return rc;
  return dispatch_gemm<KIND_F16>(g, nullptr, nullptr, c, c_dtype, ldc, nullptr, 0, dtype == ARKE_BF16 ? 1u : 0u, st, op, alpha);
}

}  // namespace arke

using namespace arke;

extern "C" int arke_b200_quant_gemm(const void* a, int64_t lda, const void* w, int64_t ldw,
                                    int w_layout, int ab_dtype, const float* sa, const float* sw,
                                    int64_t M, int64_t N, int64_t K, void* y, int y_dtype,
                                    int64_t ldy, void* acc_out, int64_t ldacc, void* stream) {
  ARKE_API_ENTER("arke_b200_quant_gemm");
  const char* op = "quant_gemm";
  if (M < 0 || N < 0 || K < 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return set_error(ARKE_ERR_SHAPE, "quant_gemm: bad shape");
  if (ab_dtype != ARKE_I8 && ab_dtype != ARKE_E4M3) return set_error(ARKE_ERR_DTYPE, "quant_gemm: operands must be int8 or e4m3");
  if (w_layout != ARKE_W_KN && w_layout != ARKE_W_NK) return set_error(ARKE_ERR_ARG, "quant_gemm: bad w_layout");
  if (y && y_dtype != ARKE_BF16 && y_dtype != ARKE_F16 && y_dtype != ARKE_F32) return set_error(ARKE_ERR_DTYPE, "quant_gemm: y must be bf16, f16 or f32");
  if (M == 0 || N == 0) return ARKE_OK;
  if (!y && !acc_out) return set_error(ARKE_ERR_ARG, "quant_gemm: no output requested");
  if (K == 0) return set_error(ARKE_ERR_SHAPE, "quant_gemm: K must be positive");
  if (!a || !w) return set_error(ARKE_ERR_ARG, "quant_gemm: null operand");
  if ((y && ldy < N) || (acc_out && ldacc < N)) return set_error(ARKE_ERR_SHAPE, "quant_gemm: output row stride smaller than N");
  int rc = require_sm100(op);
  if (rc != ARKE_OK) return rc;
  GemmOperands g{a, lda, w, ldw, w_layout == ARKE_W_KN ? 1 : 0, (int)M, (int)N, (int)K, 1};
  rc = check_gemm_operands(g, op);
  if (rc != ARKE_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (ab_dtype == ARKE_I8) return dispatch_gemm<KIND_I8>(g, sa, sw, y, y_dtype, ldy, acc_out, ldacc, 0, st, op);
  return dispatch_gemm<KIND_F8>(g, sa, sw, y, y_dtype, ldy, acc_out, ldacc, 0, st, op);
}

extern "C" int arke_b200_matmul(const void* a, int64_t lda, const void* b, int64_t ldb,
                                int w_layout, int dtype, int64_t M, int64_t N, int64_t K, void* c,
                                int64_t ldc, void* stream) {
  ARKE_API_ENTER("arke_b200_matmul");
  const char* op = "matmul";
  if (M < 0 || N < 0 || K < 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return set_error(ARKE_ERR_SHAPE, "matmul: bad shape");
  if (dtype != ARKE_BF16 && dtype != ARKE_F16 && dtype != ARKE_F32) return set_error(ARKE_ERR_DTYPE, "matmul: dtype must be bf16, f16 or f32");
  if (w_layout != ARKE_W_KN && w_layout != ARKE_W_NK) return set_error(ARKE_ERR_ARG, "matmul: bad layout");
  if (M == 0 || N == 0) return ARKE_OK;
  if (K == 0) return set_error(ARKE_ERR_SHAPE, "matmul: K must be positive");
  if (!a || !b || !c) return set_error(ARKE_ERR_ARG, "matmul: null pointer");
  if (ldc < N) return set_error(ARKE_ERR_SHAPE, "matmul: output row stride smaller than N");
  int rc = require_sm100(op);
  if (rc != ARKE_OK) return rc;
  GemmOperands g{a, lda, b, ldb, w_layout == ARKE_W_KN ? 1 : 0, (int)M, (int)N, (int)K, dtype == ARKE_F32 ? 4 : 2};
  rc = check_gemm_operands(g, op);
  if (rc != ARKE_OK) return rc;
  // fp32 operands run on the tensor cores as TF32 (10-bit significand), fp32 accumulate.  Only the
  // K-contiguous B layout is served: an N-contiguous 32-bit operand needs the 32-byte-atom swizzle
  // variant, which this library does not stage.
  if (dtype == ARKE_F32 && w_layout == ARKE_W_KN)
    return set_error(ARKE_ERR_SHAPE, "matmul: fp32 B must be given as [N,K] (K contiguous); transpose it first");
  if (dtype == ARKE_F32)
    return dispatch_gemm<KIND_TF32>(g, nullptr, nullptr, c, ARKE_F32, ldc, nullptr, 0, 0u, (cudaStream_t)stream, op);
  return dispatch_gemm<KIND_F16>(g, nullptr, nullptr, c, dtype, ldc, nullptr, 0,
                                 dtype == ARKE_BF16 ? 1u : 0u, (cudaStream_t)stream, op);
}

extern "C" int arke_b200_matmul_tn(const void* a, int64_t lda, const void* b, int64_t ldb, int w_layout,
                                   int dtype, int64_t M, int64_t N, int64_t K, void* c, int c_dtype,
                                   int64_t ldc, void* stream) {
  ARKE_API_ENTER("arke_b200_matmul_tn");
  const char* op = "matmul_tn";
  if (M < 0 || N < 0 || K < 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return set_error(ARKE_ERR_SHAPE, "matmul_tn: bad shape");
  if (dtype != ARKE_BF16 && dtype != ARKE_F16) return set_error(ARKE_ERR_DTYPE, "matmul_tn: operands must be bf16 or f16");
  if (c_dtype != ARKE_BF16 && c_dtype != ARKE_F16 && c_dtype != ARKE_F32) return set_error(ARKE_ERR_DTYPE, "matmul_tn: c must be bf16, f16 or f32");
  if (w_layout != ARKE_W_KN && w_layout != ARKE_W_NK) return set_error(ARKE_ERR_ARG, "matmul_tn: bad layout");
  if (M == 0 || N == 0) return ARKE_OK;
  if (K == 0) return set_error(ARKE_ERR_SHAPE, "matmul_tn: K must be positive");
  if (!a || !b || !c) return set_error(ARKE_ERR_ARG, "matmul_tn: null pointer");
  if (ldc < N) return set_error(ARKE_ERR_SHAPE, "matmul_tn: output row stride smaller than N");
  int rc = require_sm100(op);
  if (rc != ARKE_OK) return rc;
  return gemm_16bit(a, lda, 1, b, ldb, w_layout == ARKE_W_KN ? 1 : 0, dtype, (int)M, (int)N, (int)K, c, c_dtype, ldc,
                    (cudaStream_t)stream, op);
}
