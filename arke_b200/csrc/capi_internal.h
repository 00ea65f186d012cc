// Host-side plumbing shared by the .cu files: error reporting, the per-device kernel status
// word and the cuTensorMapEncodeTiled wrapper (resolved at run time, so the library links
// against the CUDA runtime only and loads on machines without a driver).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <nvtx3/nvToolsExt.h>
#include "../../include/arke_b200.h"

namespace arke {

int set_error(int code, const char* msg);
int set_cuda_error(const char* what, cudaError_t e);

// Device pointer to the current device's 32-bit kernel status word (zero-initialised device
// global; kernels atomically record the first expired wait there).  Returns nullptr and sets
// the error on failure.
int* kernel_status_ptr();

// Checks that the current device is compute capability 10.x; sets the error otherwise.
int require_sm100(const char* op);

// Number of SMs of the current device (cached per device).
int sm_count();
// 16-bit GEMM on the tcgen05 main loop (gemm.cu): C[M,N] = op(A) op(B), fp32 accumulate.
//   a_mn = 0: A is [M,K] (K contiguous);  a_mn = 1: A is [K,M] (M contiguous)
//   b_mn = 1: B is [K,N] (N contiguous);  b_mn = 0: B is [N,K] (K contiguous)
// `alpha` (device scalar, may be null) multiplies the fp32 accumulators before they are rounded.
int gemm_16bit(const void* a, int64_t lda, int a_mn, const void* b, int64_t ldb, int b_mn, int dtype,
               int M, int N, int K, void* c, int c_dtype, int64_t ldc, cudaStream_t st, const char* op,
               const float* alpha = nullptr);
// Device counter for the CTA-pair kernel's dynamic tile assignment (gemm.cu), nullptr = round robin.
unsigned* pair_sched_counter(int tiles, int pairs);
// Per-thread tuning options set through arke_b200_set_option (0 = the library's own choice).
struct TuningOptions {
  int gemm_tile_m = 0;    // 128: one-CTA 128-row tiles, 256: CTA-pair 256-row tiles
  int gemm_band_mb = 0;   // MB of the A operand kept L2-resident per band of tiles
  int gemm_static_sched = 0;  // 1: CTA pairs take tiles round robin instead of from the device counter
  int gemm_no_pdl = 0;    // 1: launch the GEMM kernels without programmatic stream serialization
  int gemm_no_split = 0;  // 1: the last wave of a CTA-pair GEMM keeps whole tiles (no narrow units)
};
TuningOptions& tuning_options();
// Two device counters (zero between launches: the last CTA pair to leave a kernel clears them)
// for one launch's tile scheduler; slots rotate over 64 launches per device.  nullptr on error.
unsigned* sched_counter_slot();
// Zeroes every counter slot of the current device (after a kernel reported a failed wait).
void sched_counters_clear(cudaStream_t st);
// Whether the GEMM kernels are launched with programmatic stream serialization (default yes;
// option gemm_no_pdl = 1 turns it off for the calling thread).
bool pdl_enabled();

// Tiled tensor map over a row-major tensor of rank 2 or 3 (dims[0] innermost), element size
// `elem_bytes`, 128-byte swizzle when swizzle128 != 0 (box inner extent must then be 128 B).
// strides_bytes[i] is the byte stride of dims[i+1].
int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dt, uint32_t rank, const void* base,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    int swizzle128, const char* what);

// Raises a kernel's dynamic shared-memory limit once per (kernel, device): the attribute belongs
// to the function in that device's context, and asking again on every launch costs a microsecond
// of host time, a tenth of a small op's latency.  Keyed by the kernel's address (instantiations
// with the same parameter list share one function-pointer type).
cudaError_t ensure_dynamic_smem_impl(const void* kern, int bytes);
template <class Kern>
inline cudaError_t ensure_dynamic_smem(Kern kern, int bytes) {
  return ensure_dynamic_smem_impl(reinterpret_cast<const void*>(kern), bytes);
}

// NVTX range around a C-ABI call (header-only NVTX: a no-op unless a profiler is attached), so a
// timeline shows which library call enqueued which kernels.
struct ApiRange {
  explicit ApiRange(const char* name) { nvtxRangePushA(name); }
  ~ApiRange() { nvtxRangePop(); }
  ApiRange(const ApiRange&) = delete;
  ApiRange& operator=(const ApiRange&) = delete;
};
// first statement of every entry point that launches kernels
#define ARKE_API_ENTER(name)               \
  ::arke::ApiRange arke_api_range_(name);  \
  ARKE_CHK_BIND()

#ifdef ARKE_B200_CHECKED
// Points this translation unit's copy of the checked build's status pointer at the current
// device's status word (once per device per translation unit).  Call before launching.
#define ARKE_CHK_BIND()                                                                          \
  do {                                                                                           \
    static bool arke_chk_bound[64];                                                              \
    int arke_chk_dev = 0;                                                                        \
    if (cudaGetDevice(&arke_chk_dev) == cudaSuccess && arke_chk_dev >= 0 && arke_chk_dev < 64 && \
        !arke_chk_bound[arke_chk_dev]) {                                                         \
      int* arke_chk_p = ::arke::kernel_status_ptr();                                             \
      if (arke_chk_p != nullptr &&                                                               \
          cudaMemcpyToSymbol(::arke::g_chk_status, &arke_chk_p, sizeof(arke_chk_p)) == cudaSuccess) \
        arke_chk_bound[arke_chk_dev] = true;                                                     \
    }                                                                                            \
  } while (0)
#else
#define ARKE_CHK_BIND() do { } while (0)
#endif

}  // namespace arke
