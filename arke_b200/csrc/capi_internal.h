// Host-side plumbing shared by the .cu files: error reporting, the per-device kernel status
// word and the cuTensorMapEncodeTiled wrapper (resolved at run time, so the library links
// against the CUDA runtime only and loads on machines without a driver).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
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
// Whether the GEMM kernels are launched with programmatic stream serialization (default yes;
// environment ARKE_B200_PDL=0 turns it off, a measurement knob).
bool pdl_enabled();

// Tiled tensor map over a row-major tensor of rank 2 or 3 (dims[0] innermost), element size
// `elem_bytes`, 128-byte swizzle when swizzle128 != 0 (box inner extent must then be 128 B).
// strides_bytes[i] is the byte stride of dims[i+1].
int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dt, uint32_t rank, const void* base,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    int swizzle128, const char* what);

}  // namespace arke
