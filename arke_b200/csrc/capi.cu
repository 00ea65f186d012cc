// Error reporting, device queries and tensor-map construction for the C ABI.
#include "capi_internal.h"
#include "common.cuh"
#include <stdio.h>
#include <string.h>
#include <stdlib.h>
#include <mutex>

namespace arke {

static thread_local char g_err[512] = "";

int set_error(int code, const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}
int set_cuda_error(const char* what, cudaError_t e) {
  snprintf(g_err, sizeof(g_err), "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return ARKE_ERR_CUDA;
}

__device__ int g_kernel_status;  // one copy per device that loads the module

static constexpr int kMaxDev = 64;
static int* g_status_ptr[kMaxDev];
static int g_sm_count[kMaxDev];
static int g_cc_major[kMaxDev];
static std::mutex g_mu;

static int current_device(int* dev) {
  cudaError_t e = cudaGetDevice(dev);
  if (e != cudaSuccess) return set_cuda_error("cudaGetDevice", e);
  if (*dev < 0 || *dev >= kMaxDev) return set_error(ARKE_ERR_DEVICE, "device ordinal out of range");
  return ARKE_OK;
}

static int ensure_device_info(int dev) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_sm_count[dev] != 0) return ARKE_OK;
  int sms = 0, major = 0;
  cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) return set_cuda_error("cudaDeviceGetAttribute", e);
  g_cc_major[dev] = major;
  g_sm_count[dev] = sms;
  return ARKE_OK;
}

int* kernel_status_ptr() {
  int dev;
  if (current_device(&dev) != ARKE_OK) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_kernel_status);
    if (e != cudaSuccess) {
      set_cuda_error("cudaGetSymbolAddress(kernel status)", e);
      return nullptr;
    }
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

int require_sm100(const char* op) {
  int dev;
  int rc = current_device(&dev);
  if (rc != ARKE_OK) return rc;
  rc = ensure_device_info(dev);
  if (rc != ARKE_OK) return rc;
  if (g_cc_major[dev] != 10) {
    char buf[256];
    snprintf(buf, sizeof(buf), "%s: needs an sm_100 (B200) device, found compute capability %d.x",
             op, g_cc_major[dev]);
    return set_error(ARKE_ERR_DEVICE, buf);
  }
  return ARKE_OK;
}

bool pdl_enabled() { return tuning_options().gemm_no_pdl == 0; }

__device__ unsigned g_sched_ctr[128];

void sched_counters_clear(cudaStream_t st) {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_sched_ctr) == cudaSuccess) cudaMemsetAsync(p, 0, sizeof(unsigned) * 128, st);
}

unsigned* sched_counter_slot() {
  static std::mutex mu;
  static unsigned* base[64];
  static unsigned seq[64];
  int dev;
  if (current_device(&dev) != ARKE_OK || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!base[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_sched_ctr) != cudaSuccess) return nullptr;
    base[dev] = static_cast<unsigned*>(p);
  }
  return base[dev] + 2 * (seq[dev]++ % 64);
}

cudaError_t ensure_dynamic_smem_impl(const void* kern, int bytes) {
  struct Entry { const void* kern; unsigned long long devs; };
  static Entry table[256];
  static int n = 0;
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool track = dev >= 0 && dev < 64;
  std::lock_guard<std::mutex> lock(mu);
  Entry* ent = nullptr;
  for (int i = 0; i < n; ++i)
    if (table[i].kern == kern) { ent = &table[i]; break; }
  if (ent && track && (ent->devs >> dev) & 1ull) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return e;
  if (track) {
    if (!ent && n < 256) { table[n] = Entry{kern, 0ull}; ent = &table[n++]; }
    if (ent) ent->devs |= 1ull << dev;
  }
  return cudaSuccess;
}

TuningOptions& tuning_options() {
  static thread_local TuningOptions opt;
  return opt;
}

int sm_count() {
  int dev;
  if (current_device(&dev) != ARKE_OK) return 0;
  if (ensure_device_info(dev) != ARKE_OK) return 0;
  return g_sm_count[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static int resolve_encode() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return ARKE_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return set_cuda_error("cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)", e);
  if (qres != cudaDriverEntryPointSuccess || !fn)
    return set_error(ARKE_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return ARKE_OK;
}

int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dt, uint32_t rank, const void* base,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    int swizzle128, const char* what) {
  int rc = resolve_encode();
  if (rc != ARKE_OK) return rc;
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], estr[5];
  for (uint32_t i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
  }
  for (uint32_t i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = g_encode(out, dt, rank, const_cast<void*>(base), gdim, gstr, bx, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[384];
    snprintf(buf, sizeof(buf),
             "%s: cuTensorMapEncodeTiled failed (CUresult %d) rank=%u dims=[%llu,%llu,%llu] "
             "stride0=%llu box=[%u,%u,%u] base=%p",
             what, (int)r, rank, (unsigned long long)dims[0],
             (unsigned long long)(rank > 1 ? dims[1] : 0), (unsigned long long)(rank > 2 ? dims[2] : 0),
             (unsigned long long)(rank > 1 ? strides_bytes[0] : 0), box[0], rank > 1 ? box[1] : 0,
             rank > 2 ? box[2] : 0, base);
    return set_error(ARKE_ERR_CUDA, buf);
  }
  return ARKE_OK;
}

}  // namespace arke

using namespace arke;

#ifdef ARKE_B200_CHECKED
extern "C" const char* arke_b200_version(void) { return "arke_b200 0.1 (sm_100a, checked build)"; }
#else
extern "C" const char* arke_b200_version(void) { return "arke_b200 0.1 (sm_100a)"; }
#endif
extern "C" const char* arke_b200_last_error(void) { return g_err; }

// One CTA waits (bounded) on an mbarrier that nothing ever completes, records the expiry in the
// status word like the production kernels do, and returns normally.
__global__ void selftest_wait_kernel(long long limit_cycles, int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
    const long long t0 = clock64();
    bool done = false;
    while (!(done = mbar_try_wait(&bar, 0))) {
      if (clock64() - t0 > limit_cycles) break;
    }
    if (!done) atomicCAS(status, 0, KSTAT_TIMEOUT_EPILOGUE);
  }
}

extern "C" int arke_b200_selftest_wait_timeout(int64_t limit_cycles, void* stream) {
  if (limit_cycles <= 0 || limit_cycles > 2000000000LL)
    return set_error(ARKE_ERR_ARG, "selftest_wait_timeout: limit must be in (0, 2e9] cycles");
  int* status = kernel_status_ptr();
  if (!status) return ARKE_ERR_CUDA;
  selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((long long)limit_cycles, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? ARKE_OK : set_cuda_error("selftest_wait_timeout launch", e);
}

// Checked build only: one thread evaluates the index check on an index equal to the extent (one
// past the end) — no memory is touched — so a test can see the status code the check records.
__global__ void selftest_bounds_kernel(int extent) {
  (void)ARKE_CHK(extent, extent, extent);
}

extern "C" int arke_b200_selftest_bounds_check(void* stream) {
#ifdef ARKE_B200_CHECKED
  ARKE_API_ENTER("arke_b200_selftest_bounds_check");
  if (!kernel_status_ptr()) return ARKE_ERR_CUDA;
  selftest_bounds_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(1024);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? ARKE_OK : set_cuda_error("selftest_bounds_check launch", e);
#else
  (void)stream;
  return set_error(ARKE_ERR_ARG, "selftest_bounds_check: this library was built without -DARKE_B200_CHECKED");
#endif
}

extern "C" int arke_b200_kernel_status(void* stream) {
  int* p = kernel_status_ptr();
  if (!p) return ARKE_ERR_CUDA;
  int h = 0;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(&h, p, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return set_cuda_error("kernel status read", e);
  if (h != 0) {
    sched_counters_clear(st);   // a kernel that gave up may have left its tile counter non-zero
    e = cudaMemsetAsync(p, 0, sizeof(int), st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return set_cuda_error("kernel status clear", e);
  }
  return h;
}

extern "C" int arke_b200_set_option(const char* name, int64_t value) {
  if (!name) return set_error(ARKE_ERR_ARG, "set_option: null name");
  TuningOptions& o = tuning_options();
  if (strcmp(name, "gemm_tile_m") == 0) {
    if (value != 0 && value != 128 && value != 256) return set_error(ARKE_ERR_ARG, "set_option: gemm_tile_m must be 0 (auto), 128 or 256");
    o.gemm_tile_m = (int)value;
    return ARKE_OK;
  }
  if (strcmp(name, "gemm_band_mb") == 0) {
    if (value < 0 || value > 4096) return set_error(ARKE_ERR_ARG, "set_option: gemm_band_mb must be in [0, 4096]");
    o.gemm_band_mb = (int)value;
    return ARKE_OK;
  }
  if (strcmp(name, "gemm_static_sched") == 0) {
    if (value != 0 && value != 1) return set_error(ARKE_ERR_ARG, "set_option: gemm_static_sched must be 0 or 1");
    o.gemm_static_sched = (int)value;
    return ARKE_OK;
  }
  if (strcmp(name, "gemm_no_pdl") == 0) {
    if (value != 0 && value != 1) return set_error(ARKE_ERR_ARG, "set_option: gemm_no_pdl must be 0 or 1");
    o.gemm_no_pdl = (int)value;
    return ARKE_OK;
  }
  if (strcmp(name, "gemm_no_split") == 0) {
    if (value != 0 && value != 1) return set_error(ARKE_ERR_ARG, "set_option: gemm_no_split must be 0 or 1");
    o.gemm_no_split = (int)value;
    return ARKE_OK;
  }
  return set_error(ARKE_ERR_ARG, "set_option: unknown option (known: gemm_tile_m, gemm_band_mb, gemm_static_sched, gemm_no_pdl, gemm_no_split)");
}

extern "C" int64_t arke_b200_get_option(const char* name) {
  if (!name) return -1;
  const TuningOptions& o = tuning_options();
  if (strcmp(name, "gemm_tile_m") == 0) return o.gemm_tile_m;
  if (strcmp(name, "gemm_band_mb") == 0) return o.gemm_band_mb;
  if (strcmp(name, "gemm_static_sched") == 0) return o.gemm_static_sched;
  if (strcmp(name, "gemm_no_pdl") == 0) return o.gemm_no_pdl;
  if (strcmp(name, "gemm_no_split") == 0) return o.gemm_no_split;
  return -1;
}
