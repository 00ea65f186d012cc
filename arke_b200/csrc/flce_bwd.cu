// Backward of fused linear + cross-entropy: gradients of the mean loss with respect to the hidden
// states X and the projection W, without ever holding fp32 logits.
//
// The reference defines only the forward (ref_fused_linear_cross_entropy,
// arke/ir/ops/reference_impls.py:211-213); its operator documentation lists a `logits_grad` output
// (docs/benchmark/benchmark-ops.md:582-593) that no backend of it produces.  The definition used
// here is the derivative of that forward:
//   p      = softmax(X W^T)                      (per row, over the whole vocabulary)
//   G[i,j] = p[i,j] - [j == label_i]      for label_i != ignore_index, else 0
//   dX = (grad / n_valid) G W ,   dW = (grad / n_valid) G^T X
//
// Three launches on the tcgen05 GEMM main loop:
//   1. logits tiles are recomputed like in the forward and the epilogue turns each 128 x 256 tile
//      into G (16-bit) with the row's log-sum-exp from the forward: exp(l - lse) - onehot;
//   2. dX[M,D] = G[M,V] . W[V,D]          (W as given = N-contiguous B operand)
//   3. dW[V,D] = G[M,V]^T . X[M,D]        (G as M-contiguous ("MN-major") A operand, X as given)
// G is the only intermediate: M x V 16-bit values in a caller-provided workspace.  It is stored
// UNSCALED, in [-1, 1]: multiplied by grad / n_valid first (1e-4 at 8192 tokens) most of the
// softmax tail would fall below the smallest f16 normal (6.1e-5) or flush to zero, and the
// sum_j p_j W_j term of dX / dW would be lost.  The fp32 scalar grad / n_valid is applied to the
// fp32 accumulators in the epilogue of launches 2 and 3 instead.
#include "gemm_core.cuh"
#include "gemm_pair_core.cuh"
#include "capi_internal.h"
#include <stdio.h>
#include <stdlib.h>

namespace arke {

int gemm_band_m(int M, int N, int K, int elem_bytes);  // gemm.cu

constexpr int kGradBN = 256;
constexpr float kGradLog2e = 1.4426950408889634f;

struct EpiGrad {
  static constexpr bool kSplitN = false;   // narrow last-wave units are not wired into this policy
  struct Params {
    const int64_t* labels;   // [M] global vocabulary indices
    const float* lse;        // [M] natural-log logsumexp of the full-vocabulary logits
    int64_t vocab_offset;    // global index of this W slice's first row
    int64_t ignore_index;
    uint16_t* g;             // [M, ldg] 16-bit
    int64_t ldg;
    uint32_t ab_format;      // 0 = f16, 1 = bf16 (operands and G)
  };
  static constexpr int kSmemBytes = 16;

  static __device__ void tile(const Params& p, uint8_t*, uint32_t tmem_acc, int tile_m, int tile_n,
                              int M, int N, int) {
    const int q = (threadIdx.x >> 5) & 3;
    const int lane = threadIdx.x & 31;
    const int row = tile_m * kGemmBM + q * 32 + lane;
    const bool row_ok = row < M;
    const int col_base = tile_n * kGradBN;
    const uint32_t taddr = tmem_acc + (static_cast<uint32_t>(q * 32) << 16);
    const int64_t lab = row_ok ? p.labels[row] : p.ignore_index;
    int lcol = -1;
    float sc = 0.f;
    if (lab != p.ignore_index) {
      sc = 1.f;              // rows with an ignored label contribute nothing
      const int64_t l = lab - p.vocab_offset;
      if (l >= 0 && l < N) lcol = (int)l;
    }
    const float nlse2 = row_ok ? -p.lse[row] * kGradLog2e : 0.f;
    const bool bf = p.ab_format != 0;
    uint16_t* grow = p.g + (int64_t)(row_ok ? row : 0) * p.ldg;
#pragma unroll 1
    for (int c = 0; c < kGradBN / 32; ++c) {
      const int col0 = col_base + c * 32;
      if (col0 >= N) break;  // uniform over the CTA
      uint32_t v[32];
      tmem_ld32(taddr + c * 32, v);
      tmem_ld_wait();
      float f[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = ex2_approx(fmaf(__uint_as_float(v[i]), kGradLog2e, nlse2));
      if (static_cast<unsigned>(lcol - col0) < 32u) {
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] = (lcol - col0 == i) ? f[i] - 1.f : f[i];
      }
      uint16_t* dst = grow + col0;
      if (row_ok && !ARKE_CHK((int64_t)row * p.ldg + col0, (int64_t)row * p.ldg + (col0 + 31 < N ? col0 + 31 : N - 1), span_elems(M, N, p.ldg))) {
        // checked build: the range is outside G; nothing is stored
      } else if (!row_ok) {
        // nothing to store for rows past M (the warp stays together for the next tcgen05.ld)
      } else if (col0 + 32 <= N) {   // rows of G are 16-byte aligned (ldg a multiple of 8)
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          w[i] = bf ? pack_bf16x2(f[2 * i] * sc, f[2 * i + 1] * sc) : pack_f16x2(f[2 * i] * sc, f[2 * i + 1] * sc);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (col0 + i < N)
            dst[i] = bf ? __bfloat16_as_ushort(__float2bfloat16_rn(f[i] * sc)) : __half_as_ushort(__float2half_rn(f[i] * sc));
      }
    }
  }
};

// scale = grad / max(1, number of rows whose label is not ignore_index); one block, deterministic
__global__ void __launch_bounds__(1024)
ce_grad_scale_kernel(const int64_t* __restrict__ labels, int64_t ignore_index, int M, float grad,
                     const float* __restrict__ grad_dev, float* __restrict__ out) {
  __shared__ int scnt[32];
  int cnt = 0;
  for (int i = threadIdx.x; i < M; i += 1024) cnt += labels[i] != ignore_index;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if ((threadIdx.x & 31) == 0) scnt[threadIdx.x >> 5] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int tot = 0;
    for (int i = 0; i < 32; ++i) tot += scnt[i];
    const float g = grad_dev != nullptr ? grad * grad_dev[0] : grad;
    out[0] = g / (float)(tot > 0 ? tot : 1);
  }
}

struct GradLayout {
  int64_t ldg;          // row stride of G in elements (V rounded up to 8)
  size_t off_scale;     // device scalar behind G
  size_t total;
};
static GradLayout grad_layout(int64_t M, int64_t V) {
  GradLayout L;
  L.ldg = (V + 7) & ~int64_t(7);
  L.off_scale = (((size_t)M * (size_t)L.ldg * 2) + 255) & ~size_t(255);
  L.total = L.off_scale + 256;
  return L;
}

}  // namespace arke

using namespace arke;

extern "C" size_t arke_b200_fused_linear_ce_backward_workspace(int64_t M, int64_t V) {
  if (M <= 0 || V <= 0) return 0;
  return grad_layout(M, V).total;
}

extern "C" int arke_b200_fused_linear_ce_backward(const void* x, const void* w, const int64_t* labels,
                                                  const float* lse, int dtype, int64_t M, int64_t V,
                                                  int64_t D, int64_t vocab_offset, int64_t ignore_index,
                                                  float grad, const float* grad_dev, void* dx, int dx_dtype,
                                                  void* dw, void* workspace, size_t workspace_bytes,
                                                  void* stream) {
  ARKE_API_ENTER("arke_b200_fused_linear_ce_backward");
  const char* op = "fused_linear_ce_backward";
  if (M < 0 || V < 0 || D < 0 || M > INT32_MAX || V > INT32_MAX || D > INT32_MAX) return set_error(ARKE_ERR_SHAPE, "fused_linear_ce_backward: bad shape");
  if (dtype != ARKE_BF16 && dtype != ARKE_F16) return set_error(ARKE_ERR_DTYPE, "fused_linear_ce_backward: x and w must be bf16 or f16");
  if (dx && dx_dtype != dtype && dx_dtype != ARKE_F32)
    return set_error(ARKE_ERR_DTYPE, "fused_linear_ce_backward: dx must have the operands' dtype or be f32");
  if (M == 0 || V == 0) return ARKE_OK;
  if (D == 0) return set_error(ARKE_ERR_SHAPE, "fused_linear_ce_backward: D must be positive");
  if (!x || !w || !labels || !lse) return set_error(ARKE_ERR_ARG, "fused_linear_ce_backward: null input");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(dx) |
       reinterpret_cast<uintptr_t>(dw)) & 15)
    return set_error(ARKE_ERR_ALIGN, "fused_linear_ce_backward: x, w, dx, dw must be 16-byte aligned");
  if ((D * 2) % 16 != 0) return set_error(ARKE_ERR_ALIGN, "fused_linear_ce_backward: hidden size must be a multiple of 8 (16-byte rows)");
  int rc = require_sm100(op);
  if (rc != ARKE_OK) return rc;
  const GradLayout L = grad_layout(M, V);
  if (!workspace || workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    char buf[176];
    snprintf(buf, sizeof(buf), "fused_linear_ce_backward: workspace needs %zu bytes, 256-byte aligned (got %zu)", L.total, workspace_bytes);
    return set_error(ARKE_ERR_WORKSPACE, buf);
  }
  cudaStream_t st = (cudaStream_t)stream;
  uint16_t* g = static_cast<uint16_t*>(workspace);
  float* scale = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + L.off_scale);

  ce_grad_scale_kernel<<<1, 1024, 0, st>>>(labels, ignore_index, (int)M, grad, grad_dev, scale);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error("fused_linear_ce_backward: scale launch", e);

  // ---- 1. G = softmax(X W^T) - onehot ----
  int* status = kernel_status_ptr();
  if (!status) return ARKE_ERR_CUDA;
  EpiGrad::Params ep{labels, lse, vocab_offset, ignore_index, g, L.ldg, dtype == ARKE_BF16 ? 1u : 0u};
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
    uint32_t boxb[2] = {64, (uint32_t)(pair ? kGradBN / 2 : kGradBN)};
    rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w, dimsb, str, boxb, 1, op);
    if (rc != ARKE_OK) return rc;
  }
  const int tiles_m = (int)((M + kGemmBM - 1) / kGemmBM), tiles_n = (int)((V + kGradBN - 1) / kGradBN);
  const int band = gemm_band_m((int)M, (int)V, (int)D, 2);
  if (pair) {
    constexpr int STAGES = 6;
    using SM = PairSmem<STAGES>;
    constexpr int smem_bytes = SM::kEpiOffset + EpiGrad::kSmemBytes + 1024;
    auto kern = gemm_pair_tcgen05_kernel<KIND_F16, false, STAGES, EpiGrad>;
    e = ensure_dynamic_smem(kern, smem_bytes);
    if (e != cudaSuccess) return set_cuda_error("cudaFuncSetAttribute(flce backward pair smem)", e);
    const int tiles = ((tiles_m + 1) / 2) * tiles_n;
    int grid = sms & ~1;
    if (2 * tiles < grid) grid = 2 * tiles;
    kern<<<grid, kPairThreads, smem_bytes, st>>>(ta, tb, ep, (int)M, (int)V, (int)D, (band + 1) / 2, status, pair_sched_counter(tiles, grid / 2), SplitTail{});
  } else {
    using SM = GemmSmem<kGradBN, 4>;
    constexpr int smem_bytes = SM::kEpiOffset + EpiGrad::kSmemBytes + 1024;
    auto kern = gemm_tcgen05_kernel<KIND_F16, false, kGradBN, 4, EpiGrad>;
    e = ensure_dynamic_smem(kern, smem_bytes);
    if (e != cudaSuccess) return set_cuda_error("cudaFuncSetAttribute(flce backward smem)", e);
    const int tiles = tiles_m * tiles_n;
    int grid = sms;
    if (tiles < grid) grid = tiles;
    kern<<<grid, kGemmThreads, smem_bytes, st>>>(ta, tb, ep, (int)M, (int)V, (int)D, band, status);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error("fused_linear_ce_backward: logits-gradient launch", e);

  // ---- 2. dX = G W ;  3. dW = G^T X ----
  if (dx) {
    rc = gemm_16bit(g, L.ldg, 0, w, D, 1, dtype, (int)M, (int)D, (int)V, dx, dx_dtype, D, st, "fused_linear_ce_backward: dX", scale);
    if (rc != ARKE_OK) return rc;
  }
  if (dw) {
    rc = gemm_16bit(g, L.ldg, 1, x, D, 1, dtype, (int)V, (int)D, (int)M, dw, dtype, D, st, "fused_linear_ce_backward: dW", scale);
    if (rc != ARKE_OK) return rc;
  }
  return ARKE_OK;
}
