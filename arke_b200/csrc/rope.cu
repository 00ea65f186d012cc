// Rotary position embedding (rotate-half form) and the split of a packed QKV projection into the
// [B, H, S, D] tensors attention reads — one HBM-bound pass.
//
// Semantics: ref_rope (arke/ir/ops/reference_impls.py:197-206; schema arke/ir/ops/catalog.py:425-435)
//   y[..., :D/2] = x1*cos - x2*sin,   y[..., D/2:] = x2*cos + x1*sin,   cos/sin [S, D/2]
// evaluated like the interpreter's eager tensor expression: every product and every sum is rounded
// to the tensors' dtype (no fused multiply-add), which makes the result bit-identical to it for
// bf16, f16 and f32.
//
// Work unit = one head of one token: the thread that owns elements [j, j+VEC) of the first half
// also owns the same elements of the second half, so each input element is read once and each
// output element written once (16-byte accesses; a head row of D = 128 16-bit values is 256 B
// contiguous on both sides).  Source addressing is (batch, position, head) strided, so the same
// kernel serves a contiguous [B, H, S, D] tensor (seen as B*H batches of one head) and the packed
// projection output [B*S, (Hq + 2 Hkv) * D] (heads Hq.. go to K, heads Hq+Hkv.. to V un-rotated).
#include "common.cuh"
#include "capi_internal.h"
#include "../../include/arke_b200.h"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace arke {

struct RopeParams {
  const void* x;
  const void* cos;
  const void* sin;
  void* q;
  void* k;
  void* v;
  int64_t sxb, sxs, sxh;   // source strides in elements: batch, position, head
  int64_t units;           // B * S * Htot
  int S, Htot, Hq, Hkv, D;
};

template <typename T> struct RopeVec;
template <> struct RopeVec<__nv_bfloat16> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ void apply(const uint4& a, const uint4& b, const uint4& c, const uint4& s, uint4& o1, uint4& o2) {
    const __nv_bfloat162* x1 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&b);
    const __nv_bfloat162* cc = reinterpret_cast<const __nv_bfloat162*>(&c);
    const __nv_bfloat162* ss = reinterpret_cast<const __nv_bfloat162*>(&s);
    __nv_bfloat162* y1 = reinterpret_cast<__nv_bfloat162*>(&o1);
    __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(&o2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      y1[i] = __hsub2_rn(__hmul2_rn(x1[i], cc[i]), __hmul2_rn(x2[i], ss[i]));
      y2[i] = __hadd2_rn(__hmul2_rn(x2[i], cc[i]), __hmul2_rn(x1[i], ss[i]));
    }
  }
};
template <> struct RopeVec<__half> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ void apply(const uint4& a, const uint4& b, const uint4& c, const uint4& s, uint4& o1, uint4& o2) {
    const __half2* x1 = reinterpret_cast<const __half2*>(&a);
    const __half2* x2 = reinterpret_cast<const __half2*>(&b);
    const __half2* cc = reinterpret_cast<const __half2*>(&c);
    const __half2* ss = reinterpret_cast<const __half2*>(&s);
    __half2* y1 = reinterpret_cast<__half2*>(&o1);
    __half2* y2 = reinterpret_cast<__half2*>(&o2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      y1[i] = __hsub2_rn(__hmul2_rn(x1[i], cc[i]), __hmul2_rn(x2[i], ss[i]));
      y2[i] = __hadd2_rn(__hmul2_rn(x2[i], cc[i]), __hmul2_rn(x1[i], ss[i]));
    }
  }
};
template <> struct RopeVec<float> {
  static constexpr int kVec = 4;
  static __device__ __forceinline__ void apply(const uint4& a, const uint4& b, const uint4& c, const uint4& s, uint4& o1, uint4& o2) {
    const float* x1 = reinterpret_cast<const float*>(&a);
    const float* x2 = reinterpret_cast<const float*>(&b);
    const float* cc = reinterpret_cast<const float*>(&c);
    const float* ss = reinterpret_cast<const float*>(&s);
    float* y1 = reinterpret_cast<float*>(&o1);
    float* y2 = reinterpret_cast<float*>(&o2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      y1[i] = __fsub_rn(__fmul_rn(x1[i], cc[i]), __fmul_rn(x2[i], ss[i]));
      y2[i] = __fadd_rn(__fmul_rn(x2[i], cc[i]), __fmul_rn(x1[i], ss[i]));
    }
  }
};

template <typename T> __device__ __forceinline__ T rope_mul(T a, T b);
template <> __device__ __forceinline__ __nv_bfloat16 rope_mul(__nv_bfloat16 a, __nv_bfloat16 b) { return __hmul_rn(a, b); }
template <> __device__ __forceinline__ __half rope_mul(__half a, __half b) { return __hmul_rn(a, b); }
template <> __device__ __forceinline__ float rope_mul(float a, float b) { return __fmul_rn(a, b); }
template <typename T> __device__ __forceinline__ T rope_add(T a, T b);
template <> __device__ __forceinline__ __nv_bfloat16 rope_add(__nv_bfloat16 a, __nv_bfloat16 b) { return __hadd_rn(a, b); }
template <> __device__ __forceinline__ __half rope_add(__half a, __half b) { return __hadd_rn(a, b); }
template <> __device__ __forceinline__ float rope_add(float a, float b) { return __fadd_rn(a, b); }
template <typename T> __device__ __forceinline__ T rope_sub(T a, T b);
template <> __device__ __forceinline__ __nv_bfloat16 rope_sub(__nv_bfloat16 a, __nv_bfloat16 b) { return __hsub_rn(a, b); }
template <> __device__ __forceinline__ __half rope_sub(__half a, __half b) { return __hsub_rn(a, b); }
template <> __device__ __forceinline__ float rope_sub(float a, float b) { return __fsub_rn(a, b); }

// Where unit (b, s, h) goes: destination row pointer and whether it is rotated.
template <typename T>
__device__ __forceinline__ T* rope_dst(const RopeParams& p, int64_t b, int s, int h, bool& rotate) {
  if (h < p.Hq) {
    rotate = true;
    return reinterpret_cast<T*>(p.q) + ((b * p.Hq + h) * p.S + s) * p.D;
  }
  if (h < p.Hq + p.Hkv) {
    rotate = true;
    return reinterpret_cast<T*>(p.k) + ((b * p.Hkv + (h - p.Hq)) * p.S + s) * p.D;
  }
  rotate = false;
  return reinterpret_cast<T*>(p.v) + ((b * p.Hkv + (h - p.Hq - p.Hkv)) * p.S + s) * p.D;
}

// Checked build: the source, table and destination element ranges of one thread, re-derived from
// the launch parameters, must lie inside their tensors (see ARKE_CHK in common.cuh).
#ifdef ARKE_B200_CHECKED
__device__ __forceinline__ bool rope_chk(const RopeParams& p, int64_t b, int s, int h, int j, int n) {
  const int half = p.D >> 1;
  const long long nb = p.units / ((long long)p.S * p.Htot);
  const long long ext_src = (nb - 1) * p.sxb + (long long)(p.S - 1) * p.sxs + (long long)(p.Htot - 1) * p.sxh + p.D;
  const long long so = b * p.sxb + (long long)s * p.sxs + (long long)h * p.sxh + j;
  const bool ok = ARKE_CHK(so, so + half + n - 1, ext_src) &&
                  ARKE_CHK((long long)s * half + j, (long long)s * half + j + n - 1, (long long)p.S * half);
  long long doff, dext;
  if (h < p.Hq) {
    doff = ((b * p.Hq + h) * p.S + s) * (long long)p.D + j;
    dext = nb * p.Hq * (long long)p.S * p.D;
  } else {
    const int hk = h < p.Hq + p.Hkv ? h - p.Hq : h - p.Hq - p.Hkv;
    doff = ((b * p.Hkv + hk) * p.S + s) * (long long)p.D + j;
    dext = nb * p.Hkv * (long long)p.S * p.D;
  }
  return ok && ARKE_CHK(doff, doff + half + n - 1, dext);
}
#define ARKE_ROPE_CHK(p, b, s, h, j, n) rope_chk(p, b, s, h, j, n)
#else
#define ARKE_ROPE_CHK(p, b, s, h, j, n) (true)
#endif

// VEC = RopeVec<T>::kVec: 16-byte accesses (D/2 a multiple of VEC, everything 16-byte aligned).
template <typename T>
__global__ void __launch_bounds__(256) rope_vec_kernel(const RopeParams p) {
  constexpr int VEC = RopeVec<T>::kVec;
  const int half = p.D >> 1;
  const int vpu = half / VEC;                       // vectors per unit and half
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t u = idx / vpu;
  if (u >= p.units) return;
  const int j = (int)(idx - u * vpu) * VEC;
  const int h = (int)(u % p.Htot);
  const int64_t tok = u / p.Htot;
  const int s = (int)(tok % p.S);
  const int64_t b = tok / p.S;
  if (!ARKE_ROPE_CHK(p, b, s, h, j, VEC)) return;
  const T* src = reinterpret_cast<const T*>(p.x) + b * p.sxb + (int64_t)s * p.sxs + (int64_t)h * p.sxh + j;
  bool rotate;
  T* dst = rope_dst<T>(p, b, s, h, rotate) + j;
  const uint4 a = __ldcs(reinterpret_cast<const uint4*>(src));
  const uint4 bb = __ldcs(reinterpret_cast<const uint4*>(src + half));
  uint4 o1 = a, o2 = bb;
  if (rotate) {
    const uint4 c = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.cos) + (int64_t)s * half + j));
    const uint4 sn = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.sin) + (int64_t)s * half + j));
    RopeVec<T>::apply(a, bb, c, sn, o1, o2);
  }
  *reinterpret_cast<uint4*>(dst) = o1;              // plain stores: attention reads these next (L2)
  *reinterpret_cast<uint4*>(dst + half) = o2;
}

// any even D, any alignment: one element pair per thread
template <typename T>
__global__ void __launch_bounds__(256) rope_scalar_kernel(const RopeParams p) {
  const int half = p.D >> 1;
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t u = idx / half;
  if (u >= p.units) return;
  const int j = (int)(idx - u * half);
  const int h = (int)(u % p.Htot);
  const int64_t tok = u / p.Htot;
  const int s = (int)(tok % p.S);
  const int64_t b = tok / p.S;
  if (!ARKE_ROPE_CHK(p, b, s, h, j, 1)) return;
  const T* src = reinterpret_cast<const T*>(p.x) + b * p.sxb + (int64_t)s * p.sxs + (int64_t)h * p.sxh + j;
  bool rotate;
  T* dst = rope_dst<T>(p, b, s, h, rotate) + j;
  const T x1 = src[0], x2 = src[half];
  if (rotate) {
    const T c = reinterpret_cast<const T*>(p.cos)[(int64_t)s * half + j];
    const T sn = reinterpret_cast<const T*>(p.sin)[(int64_t)s * half + j];
    dst[0] = rope_sub<T>(rope_mul<T>(x1, c), rope_mul<T>(x2, sn));
    dst[half] = rope_add<T>(rope_mul<T>(x2, c), rope_mul<T>(x1, sn));
  } else {
    dst[0] = x1;
    dst[half] = x2;
  }
}

static inline bool al16(const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
static int launch_rope(const RopeParams& p, cudaStream_t st, const char* op) {
  constexpr int VEC = RopeVec<T>::kVec;
  const int half = p.D / 2;
  const bool vec_ok = half % VEC == 0 && p.sxb % VEC == 0 && p.sxs % VEC == 0 && p.sxh % VEC == 0 &&
                      al16(p.x) && al16(p.cos) && al16(p.sin) && al16(p.q) && al16(p.k) && al16(p.v);
  const int64_t threads = p.units * (vec_ok ? half / VEC : half);
  const int64_t blocks = (threads + 255) / 256;
  if (blocks > 0x7fffffffLL) return set_error(ARKE_ERR_SHAPE, "rope: too many elements for one launch");
  if (vec_ok) rope_vec_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(p);
  else rope_scalar_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? ARKE_OK : set_cuda_error(op, e);
}

static int dispatch_rope(const RopeParams& p, int dtype, cudaStream_t st, const char* op) {
  ARKE_API_ENTER("arke_b200_rope");
  switch (dtype) {
    case ARKE_BF16: return launch_rope<__nv_bfloat16>(p, st, op);
    case ARKE_F16: return launch_rope<__half>(p, st, op);
    case ARKE_F32: return launch_rope<float>(p, st, op);
    default: return set_error(ARKE_ERR_DTYPE, "rope: dtype must be bf16, f16 or f32 (x, cos, sin and the outputs share it)");
  }
}

}  // namespace arke

using namespace arke;

extern "C" int arke_b200_rope(const void* x, const void* cos, const void* sin, void* y, int dtype,
                              int64_t B, int64_t H, int64_t S, int64_t D, void* stream) {
  if (B < 0 || H < 0 || S < 0 || D <= 0 || (D & 1) || D > (1 << 20) || S > INT32_MAX || B * H > INT32_MAX)
    return set_error(ARKE_ERR_SHAPE, "rope: need B, H, S >= 0 and an even head_dim");
  if (B == 0 || H == 0 || S == 0) return ARKE_OK;
  if (!x || !cos || !sin || !y) return set_error(ARKE_ERR_ARG, "rope: null pointer");
  int rc = require_sm100("rope");
  if (rc != ARKE_OK) return rc;
  RopeParams p{};
  p.x = x; p.cos = cos; p.sin = sin; p.q = y; p.k = nullptr; p.v = nullptr;
  p.sxb = S * D; p.sxs = D; p.sxh = 0;               // [B*H] batches of one head each
  p.units = B * H * S;
  p.S = (int)S; p.Htot = 1; p.Hq = 1; p.Hkv = 0; p.D = (int)D;
  return dispatch_rope(p, dtype, (cudaStream_t)stream, "rope launch");
}

extern "C" int arke_b200_qkv_rope_split(const void* qkv, int64_t ld, const void* cos, const void* sin,
                                        void* q, void* k, void* v, int dtype, int64_t B, int64_t S,
                                        int64_t Hq, int64_t Hkv, int64_t D, void* stream) {
  if (B < 0 || S < 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || (D & 1) || D > (1 << 20) || S > INT32_MAX ||
      Hq + 2 * Hkv > 65535)
    return set_error(ARKE_ERR_SHAPE, "qkv_rope_split: need B, S >= 0, Hq, Hkv > 0 and an even head_dim");
  if (ld < (Hq + 2 * Hkv) * D) return set_error(ARKE_ERR_SHAPE, "qkv_rope_split: row stride smaller than (Hq + 2 Hkv) * D");
  if (B == 0 || S == 0) return ARKE_OK;
  if (!qkv || !cos || !sin || !q || !k || !v) return set_error(ARKE_ERR_ARG, "qkv_rope_split: null pointer");
  int rc = require_sm100("qkv_rope_split");
  if (rc != ARKE_OK) return rc;
  RopeParams p{};
  p.x = qkv; p.cos = cos; p.sin = sin; p.q = q; p.k = k; p.v = v;
  p.sxb = S * ld; p.sxs = ld; p.sxh = D;
  p.Htot = (int)(Hq + 2 * Hkv);
  p.units = B * S * p.Htot;
  p.S = (int)S; p.Hq = (int)Hq; p.Hkv = (int)Hkv; p.D = (int)D;
  return dispatch_rope(p, dtype, (cudaStream_t)stream, "qkv_rope_split launch");
}
