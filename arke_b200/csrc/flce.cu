// Fused linear + cross-entropy: logits = X * W^T are produced tile by tile on the tcgen05 main
// loop of gemm_core.cuh and consumed in the epilogue by an online softmax, so the [M,V] logits
// never exist in memory.
//
// Semantics: ref_fused_linear_cross_entropy (arke/ir/ops/reference_impls.py:211-213):
//   logits = X.float() @ W.float().T ; loss = F.cross_entropy(logits, labels)
// (mean over rows whose label != ignore_index), plus the per-token vector (reduction="none").
//
// Kernel 1 (GEMM + epilogue): for every 128 x 256 logit tile each epilogue thread owns one row and
//   reduces its 256 columns to (max, sum exp(l - max)); the pair goes to scratch[tile_n][row];
//   the thread whose tile contains the row's label also stores the target logit.
// Kernel 2 (row combine): merges the per-tile pairs of a row, writes (max, sumexp, target) and/or
//   the per-token loss.
// Kernel 3 (mean): deterministic single-block reduction of the per-token losses.
#include "gemm_core.cuh"
#include "gemm_pair_core.cuh"
#include <stdlib.h>
#include "capi_internal.h"
#include <stdio.h>
#include <mutex>

namespace arke {

int gemm_band_m(int M, int N, int K, int elem_bytes);  // gemm.cu

constexpr int kCeBN = 256;
constexpr int kCeStages = 4;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct EpiCE {
  static constexpr bool kSplitN = false;   // a row's reduction runs over all columns of the tile
  struct Params {
    const int64_t* labels;   // [M] global vocabulary indices
    int64_t vocab_offset;    // global index of this W slice's first row
    int64_t ignore_index;
    float2* ms;              // scratch [tiles_n][m_pad] of (max, sumexp)
    float* tgt;              // scratch [m_pad] target logit (zero-initialised by the host)
    int m_pad;
    uint32_t ab_format;      // 0 = f16, 1 = bf16
  };
  static constexpr int kSmemBytes = 16;

  static __device__ void tile(const Params& p, uint8_t*, uint32_t tmem_acc, int tile_m, int tile_n,
                              int M, int N, int) {
    const int q = (threadIdx.x >> 5) & 3;
    const int lane = threadIdx.x & 31;
    const int row = tile_m * kGemmBM + q * 32 + lane;
    const bool row_ok = row < M;
    const int col_base = tile_n * kCeBN;
    const uint32_t taddr = tmem_acc + (static_cast<uint32_t>(q * 32) << 16);
    // label column relative to this W slice; -1 when ignored / outside
    int64_t lab = row_ok ? p.labels[row] : p.ignore_index;
    int lcol = -1;
    if (lab != p.ignore_index) {
      const int64_t l = lab - p.vocab_offset;
      if (l >= 0 && l < N) lcol = (int)l;
    }
    float m = -INFINITY, s = 0.f;
#pragma unroll 1
    for (int c = 0; c < kCeBN / 32; ++c) {
      const int col0 = col_base + c * 32;
      if (col0 >= N) break;  // uniform
      uint32_t v[32];
      tmem_ld32(taddr + c * 32, v);
      tmem_ld_wait();
      float f[32];
      const int nvalid = N - col0;  // >= 1
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = (i < nvalid) ? __uint_as_float(v[i]) : -INFINITY;
      if (static_cast<unsigned>(lcol - col0) < 32u) {
        float tv = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) tv = (lcol - col0 == i) ? f[i] : tv;
        if (ARKE_CHK(row, row, p.m_pad)) p.tgt[row] = tv;
      }
      float cm = f[0];
#pragma unroll
      for (int i = 1; i < 32; ++i) cm = fmaxf(cm, f[i]);
      const float nm = fmaxf(m, cm);
      const float nm2 = nm * kLog2e;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) acc += ex2_approx(fmaf(f[i], kLog2e, -nm2));
      s = s * ex2_approx(m * kLog2e - nm2) + acc;  // m = -inf on the first chunk: factor 0, s = 0
      m = nm;
    }
    if (row_ok && ARKE_CHK((int64_t)tile_n * p.m_pad + row, (int64_t)tile_n * p.m_pad + row, (int64_t)((N + kCeBN - 1) / kCeBN) * p.m_pad))
      p.ms[(int64_t)tile_n * p.m_pad + row] = make_float2(m, s);
  }
};

// Merge the per-tile (max, sumexp) pairs of each row.  A block covers 32 consecutive rows; warp g
// of the block takes tiles g, g+8, ... (a warp reads 32 consecutive rows of one tile: 256 B), and
// the eight partial results of a row meet in shared memory in a fixed order (deterministic).
__global__ void __launch_bounds__(256)
ce_row_combine_kernel(const float2* __restrict__ ms, const float* __restrict__ tgt, int tiles_n,
                      int m_pad, int M, const int64_t* __restrict__ labels, int64_t ignore_index,
                      float* __restrict__ loss_tok, float* __restrict__ partials,
                      int64_t label_end, int* __restrict__ status) {
  __shared__ float red[8][32];
  const int r = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int row = blockIdx.x * 32 + r;
  const bool ok = row < M;
  const float2* p = ms + (ok ? row : 0);
  float mx = -INFINITY;
  if (ok) {
#pragma unroll 4
    for (int j = g; j < tiles_n; j += 8) mx = fmaxf(mx, p[(int64_t)j * m_pad].x);
  }
  red[g][r] = mx;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) mx = fmaxf(mx, red[i][r]);
  __syncthreads();
  float s = 0.f;
  if (ok) {
#pragma unroll 4
    for (int j = g; j < tiles_n; j += 8) {
      const float2 v = p[(int64_t)j * m_pad];
      s += v.y * exp2f((v.x - mx) * kLog2e);
    }
  }
  red[g][r] = s;
  __syncthreads();
  if (g != 0 || !ok) return;
  s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += red[i][r];
  const float t = tgt[row];
  if (partials && ARKE_CHK(3 * (int64_t)row, 3 * (int64_t)row + 2, 3 * (int64_t)M)) {
    partials[3 * (int64_t)row + 0] = mx;
    partials[3 * (int64_t)row + 1] = s;
    partials[3 * (int64_t)row + 2] = t;
  }
  if (loss_tok) {
    const int64_t lab = labels[row];
    float loss = (lab == ignore_index) ? 0.f : (logf(s) + mx - t);
    // A call over the whole vocabulary (label_end > 0) has no other slice that could hold the
    // label: a label outside [0, V) is corrupt input.  The reference's F.cross_entropy raises for
    // it; here the row's loss becomes NaN (so does the mean) and the status word records it.
    if (label_end > 0 && lab != ignore_index && (lab < 0 || lab >= label_end)) {
      loss = __int_as_float(0x7fc00000);
      atomicCAS(status, 0, KSTAT_BAD_LABEL);
    }
    if (ARKE_CHK(row, row, M)) loss_tok[row] = loss;
  }
}

// merge G vocabulary-shard partials [G,M,3]
__global__ void __launch_bounds__(256)
ce_shard_combine_kernel(const float* __restrict__ partials, int G, int M,
                        const int64_t* __restrict__ labels, int64_t ignore_index,
                        float* __restrict__ loss_tok) {
  const int row = blockIdx.x * 256 + threadIdx.x;
  if (row >= M) return;
  float mx = -INFINITY;
  for (int g = 0; g < G; ++g) mx = fmaxf(mx, partials[((int64_t)g * M + row) * 3]);
  float s = 0.f, t = 0.f;
  for (int g = 0; g < G; ++g) {
    const float* pr = partials + ((int64_t)g * M + row) * 3;
    s += pr[1] * exp2f((pr[0] - mx) * kLog2e);
    t += pr[2];
  }
  loss_tok[row] = (labels[row] == ignore_index) ? 0.f : (logf(s) + mx - t);
}

// mean over non-ignored rows; one block, fixed summation order (deterministic)
__global__ void __launch_bounds__(1024)
ce_mean_kernel(const float* __restrict__ loss_tok, const int64_t* __restrict__ labels,
               int64_t ignore_index, int M, float* __restrict__ mean_out) {
  __shared__ float ssum[32];
  __shared__ int scnt[32];
  float sum = 0.f;
  int cnt = 0;
  for (int i = threadIdx.x; i < M; i += 1024) {
    if (labels[i] != ignore_index) {
      sum += loss_tok[i];
      cnt += 1;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
    cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  }
  if ((threadIdx.x & 31) == 0) {
    ssum[threadIdx.x >> 5] = sum;
    scnt[threadIdx.x >> 5] = cnt;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float ts = 0.f;
    int tc = 0;
    for (int i = 0; i < 32; ++i) {
      ts += ssum[i];
      tc += scnt[i];
    }
    // F.cross_entropy returns NaN when every row is ignored (0 / 0); keep that behaviour
    *mean_out = ts / (float)tc;
  }
}

struct CeLayout {
  int tiles_m, tiles_n, m_pad;
  size_t off_ms, off_tgt, off_loss, total;
};
static CeLayout ce_layout(int64_t M, int64_t V) {
  CeLayout L;
  L.tiles_m = (int)((M + kGemmBM - 1) / kGemmBM);
  L.tiles_n = (int)((V + kCeBN - 1) / kCeBN);
  L.m_pad = L.tiles_m * kGemmBM;
  L.off_ms = 0;
  L.off_tgt = (size_t)L.tiles_n * L.m_pad * sizeof(float2);
  L.off_loss = L.off_tgt + (size_t)L.m_pad * sizeof(float);
  L.total = L.off_loss + (size_t)L.m_pad * sizeof(float);
  return L;
}

}  // namespace arke

using namespace arke;

extern "C" size_t arke_b200_fused_linear_ce_workspace(int64_t M, int64_t V, int64_t D) {
  (void)D;
  if (M <= 0 || V <= 0) return 0;
  return ce_layout(M, V).total;
}

extern "C" int arke_b200_fused_linear_ce(const void* x, const void* w, const int64_t* labels,
                                         int dtype, int64_t M, int64_t V, int64_t D,
                                         int64_t vocab_offset, int64_t ignore_index,
                                         float* loss_tok, float* mean_loss, float* partials,
                                         void* workspace, size_t workspace_bytes, void* stream) {
  ARKE_API_ENTER("arke_b200_fused_linear_ce");
  const char* op = "fused_linear_ce";
  if (M < 0 || V < 0 || D < 0 || M > INT32_MAX || V > INT32_MAX || D > INT32_MAX) return set_error(ARKE_ERR_SHAPE, "fused_linear_ce: bad shape");
  if (dtype != ARKE_BF16 && dtype != ARKE_F16) return set_error(ARKE_ERR_DTYPE, "fused_linear_ce: x and w must be bf16 or f16");
  if (M == 0) return ARKE_OK;
  if (V == 0 || D == 0) return set_error(ARKE_ERR_SHAPE, "fused_linear_ce: V and D must be positive");
  if (!x || !w || !labels) return set_error(ARKE_ERR_ARG, "fused_linear_ce: null input");
  if (!loss_tok && !mean_loss && !partials) return set_error(ARKE_ERR_ARG, "fused_linear_ce: no output requested");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return set_error(ARKE_ERR_ALIGN, "fused_linear_ce: x and w must be 16-byte aligned");
  if ((D * 2) % 16 != 0) return set_error(ARKE_ERR_ALIGN, "fused_linear_ce: hidden size must be a multiple of 8 (16-byte rows)");
  int rc = require_sm100(op);
  if (rc != ARKE_OK) return rc;
  const CeLayout L = ce_layout(M, V);
  if (!workspace || workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(workspace) & 15)) {
    char buf[160];
    snprintf(buf, sizeof(buf), "fused_linear_ce: workspace needs %zu bytes, 16-byte aligned (got %zu)", L.total, workspace_bytes);
    return set_error(ARKE_ERR_WORKSPACE, buf);
  }
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float2* ms = reinterpret_cast<float2*>(ws + L.off_ms);
  float* tgt = reinterpret_cast<float*>(ws + L.off_tgt);
  float* loss_ws = reinterpret_cast<float*>(ws + L.off_loss);

  cudaError_t e = cudaMemsetAsync(tgt, 0, (size_t)L.m_pad * sizeof(float), st);
  if (e != cudaSuccess) return set_cuda_error("fused_linear_ce: memset", e);

  int* status = kernel_status_ptr();
  if (!status) return ARKE_ERR_CUDA;
  EpiCE::Params ep{labels, vocab_offset, ignore_index, ms, tgt, L.m_pad, dtype == ARKE_BF16 ? 1u : 0u};
  const int sms = sm_count();
  if (sms <= 0) return ARKE_ERR_CUDA;
  bool pair = M >= 1024 && V >= 1024;
  if (const int tm = tuning_options().gemm_tile_m) pair = tm == 256;              // caller's choice
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {(uint64_t)D, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)D * 2};
    uint32_t box[2] = {64, (uint32_t)kGemmBM};
    rc = make_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, x, dims, str, box, 1, op);
    if (rc != ARKE_OK) return rc;
    uint64_t dimsb[2] = {(uint64_t)D, (uint64_t)V};
    uint32_t boxb[2] = {64, (uint32_t)(pair ? kCeBN / 2 : kCeBN)};   // a CTA of a pair stages half the columns
    rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w, dimsb, str, boxb, 1, op);
    if (rc != ARKE_OK) return rc;
  }
  const int band = gemm_band_m((int)M, (int)V, (int)D, 2);
  if (pair) {
    constexpr int STAGES = 6;
    using SM = PairSmem<STAGES>;
    constexpr int smem_bytes = SM::kEpiOffset + EpiCE::kSmemBytes + 1024;
    auto kern = gemm_pair_tcgen05_kernel<KIND_F16, false, STAGES, EpiCE>;
    e = ensure_dynamic_smem(kern, smem_bytes);
    if (e != cudaSuccess) return set_cuda_error("cudaFuncSetAttribute(flce pair smem)", e);
    const int tiles = ((L.tiles_m + 1) / 2) * L.tiles_n;
    int grid = sms & ~1;
    if (2 * tiles < grid) grid = 2 * tiles;
    kern<<<grid, kPairThreads, smem_bytes, st>>>(ta, tb, ep, (int)M, (int)V, (int)D, (band + 1) / 2, status, pair_sched_counter(tiles, grid / 2), SplitTail{});
  } else {
    using SM = GemmSmem<kCeBN, kCeStages>;
    constexpr int smem_bytes = SM::kEpiOffset + EpiCE::kSmemBytes + 1024;
    auto kern = gemm_tcgen05_kernel<KIND_F16, false, kCeBN, kCeStages, EpiCE>;
    e = ensure_dynamic_smem(kern, smem_bytes);
    if (e != cudaSuccess) return set_cuda_error("cudaFuncSetAttribute(flce smem)", e);
    const int tiles = L.tiles_m * L.tiles_n;
    int grid = sms;
    if (tiles < grid) grid = tiles;
    kern<<<grid, kGemmThreads, smem_bytes, st>>>(ta, tb, ep, (int)M, (int)V, (int)D, band, status);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error("fused_linear_ce: gemm launch", e);

  float* loss_dst = loss_tok ? loss_tok : ((mean_loss != nullptr) ? loss_ws : nullptr);
  // labels are range-checked only when this call covers the whole vocabulary for certain
  const int64_t label_end = (vocab_offset == 0 && partials == nullptr) ? V : 0;
  ce_row_combine_kernel<<<(int)((M + 31) / 32), 256, 0, st>>>(ms, tgt, L.tiles_n, L.m_pad, (int)M, labels,
                                                             ignore_index, loss_dst, partials, label_end, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error("fused_linear_ce: combine launch", e);
  if (mean_loss) {
    ce_mean_kernel<<<1, 1024, 0, st>>>(loss_dst, labels, ignore_index, (int)M, mean_loss);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_cuda_error("fused_linear_ce: mean launch", e);
  }
  return ARKE_OK;
}

extern "C" int arke_b200_ce_combine(const float* partials, int64_t G, int64_t M,
                                    const int64_t* labels, int64_t ignore_index, float* loss_tok,
                                    float* mean_loss, void* stream) {
  ARKE_API_ENTER("arke_b200_ce_combine");
  if (G <= 0 || M < 0 || M > INT32_MAX || G > 4096) return set_error(ARKE_ERR_SHAPE, "ce_combine: bad shape");
  if (M == 0) return ARKE_OK;
  if (!partials || !labels || !loss_tok) return set_error(ARKE_ERR_ARG, "ce_combine: null pointer (loss_tok is required)");
  cudaStream_t st = (cudaStream_t)stream;
  ce_shard_combine_kernel<<<(int)((M + 255) / 256), 256, 0, st>>>(partials, (int)G, (int)M, labels, ignore_index, loss_tok);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error("ce_combine launch", e);
  if (mean_loss) {
    ce_mean_kernel<<<1, 1024, 0, st>>>(loss_tok, labels, ignore_index, (int)M, mean_loss);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_cuda_error("ce_combine mean launch", e);
  }
  return ARKE_OK;
}

// --------------------------------------------------------------------------------------------
// Variant of fused_linear_ce for callers that cannot provide a workspace
// --------------------------------------------------------------------------------------------
// The per-tile (max, sumexp) pairs, the target logits and the per-token staging normally live in
// a caller-allocated workspace.  Some hosts cannot allocate one: every byte of device memory is
// already owned by their own pool, so a cudaMalloc (theirs or torch's) would fail or stall the
// device, or they sit in a serving loop where an allocation's implicit synchronisation is not
// acceptable.  For them the scratch is this fixed array; it costs kStaticScratchBytes of device
// memory on every GPU that loads the library, for the lifetime of the process.
constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_ce_static_scratch[kStaticScratchBytes];

namespace {
std::mutex g_static_mu;
void* g_static_ptr[64];  // device address of g_ce_static_scratch, per device ordinal
}  // namespace

// In host code `g_ce_static_scratch` is only a handle for the runtime, not an address a kernel
// can use; the device address is looked up once per device (with that device current).
static int static_scratch_ptr(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_cuda_error("fused_linear_ce_static: cudaGetDevice", e);
  if (dev < 0 || dev >= 64) return set_error(ARKE_ERR_DEVICE, "fused_linear_ce_static: device ordinal out of range");
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_ce_static_scratch);
    if (e != cudaSuccess) return set_cuda_error("fused_linear_ce_static: cudaGetSymbolAddress", e);
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return ARKE_OK;
}

// The first call on a device looks up the array's device address (keep that call outside any
// stream capture); later calls only read the cached pointer.  All calls share the one array and
// it keeps whatever the previous call left: the part that must start at zero (the target-logit
// slots) is cleared on `stream` by every call, and two calls whose work overlaps on the GPU
// (different streams without an ordering between them) would race on it.
extern "C" int arke_b200_fused_linear_ce_static(const void* x, const void* w, const int64_t* labels,
                                                int dtype, int64_t M, int64_t V, int64_t D,
                                                int64_t vocab_offset, int64_t ignore_index,
                                                float* loss_tok, float* mean_loss, float* partials,
                                                void* stream) {
  if (M > 0 && V > 0 && M <= INT32_MAX && V <= INT32_MAX) {
    const size_t need = ce_layout(M, V).total;
    if (need > kStaticScratchBytes) {
      char buf[256];
      snprintf(buf, sizeof(buf),
               "fused_linear_ce_static: M=%lld, V=%lld needs %zu bytes of scratch but the built-in array "
               "holds %zu; use arke_b200_fused_linear_ce with a caller-provided workspace",
               (long long)M, (long long)V, need, kStaticScratchBytes);
      return set_error(ARKE_ERR_WORKSPACE, buf);
    }
  }
  void* scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);
  if (rc != ARKE_OK) return rc;
  return arke_b200_fused_linear_ce(x, w, labels, dtype, M, V, D, vocab_offset, ignore_index, loss_tok,
                                   mean_loss, partials, scratch, kStaticScratchBytes, stream);
}
