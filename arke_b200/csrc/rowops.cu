// Row-wise HBM-bound kernels: per-token quantization (int8 / e4m3) and packed SwiGLU with
// optional e4m3 re-quantization.  One row (token) is owned by a group of TPR threads that
// keeps the whole row in registers between the amax reduction and the quantising pass, so
// every input byte is read from HBM exactly once; all fast-path accesses are 128-bit and the
// per-element work is branch-free (about seven instructions), which is what lets the kernels
// run at the measured HBM copy rate.
//
// Semantics follow the reference interpreter:
//   quantize_per_token : arke/ir/ops/reference_impls.py:215-218 evaluated on X.float()
//   silu_and_mul       : arke/ir/ops/reference_impls.py:167-171 (each op rounds to the input dtype)
#include "common.cuh"
#include "capi_internal.h"

namespace arke {

// --------------------------------------------------------------------------------------------
// element-type helpers
// --------------------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__nv_bfloat16> {
  using V2 = __nv_bfloat162;
  static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) { return pack_bf16x2(a, b); }
  static __device__ __forceinline__ float round(float a) { return __bfloat162float(__float2bfloat16_rn(a)); }
};
template <> struct Elem<__half> {
  using V2 = __half2;
  static __device__ __forceinline__ float lo(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w & 0xffff))); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w >> 16))); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) { return pack_f16x2(a, b); }
  static __device__ __forceinline__ float round(float a) { return __half2float(__float2half_rn(a)); }
};
template <> struct Elem<float> {
  static __device__ __forceinline__ float round(float a) { return a; }
};

template <typename T>
__device__ __forceinline__ uint32_t absmax2(uint32_t acc, uint32_t w) {
  using V2 = typename Elem<T>::V2;
  V2 a = *reinterpret_cast<V2*>(&acc);
  V2 b = *reinterpret_cast<V2*>(&w);
  V2 r = __hmax2(a, __habs2(b));
  return *reinterpret_cast<uint32_t*>(&r);
}
template <typename T>
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
  using V2 = typename Elem<T>::V2;
  V2 r = __hmul2(*reinterpret_cast<V2*>(&a), *reinterpret_cast<V2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(uint2* p, uint2 v) { __stcs(p, v); }

// Max over the TPR threads that share a row. `red` holds 8 floats (one per warp of the CTA).
template <int TPR>
__device__ __forceinline__ float group_max(float v, float* red) {
  constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;  // warps per row
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) red[warp] = v;
    __syncthreads();
    const int base = (warp / WPR) * WPR;
    v = red[base];
#pragma unroll
    for (int i = 1; i < WPR; ++i) v = fmaxf(v, red[base + i]);
  }
  return v;
}

// rint(x / scale) as the reference computes it (correctly rounded fp32 quotient, then round
// half to even), clamped to the int8 range.  scale == 0 (an all-zero row) maps to 0.
__device__ __forceinline__ int quant_exact(float x, float scale) {
  if (!(scale > 0.f)) return 0;
  float t = rintf(__fdiv_rn(x, scale));
  t = fminf(fmaxf(t, -128.f), 127.f);
  return (int)t;
}

// Correctly rounded x / s from the correctly rounded reciprocal inv = RN(1/s): q0 = RN(x*inv),
// residual r = x - q0*s by FMA, q1 = RN(q0 + r*inv) (one-step correction of the quotient).
// Three FMA-pipe instructions, no branch.  Rows whose maximum lies outside [2^-60, 2^60] (where
// the reciprocal or the residual could leave the normal fp32 range) do not use it: for them
// fast_quotient_ok() is false and the caller passes inv = NaN-free exact divisions instead.
// Inside that range the quantised code (int8 or e4m3) obtained from this quotient is identical to
// the one obtained from the IEEE division for every 16-bit x with |x| <= amax;
// arke_b200_selftest_quant_division() checks that exhaustively on the device.
__device__ __forceinline__ float div_by_scale(float x, float s, float inv) {
  const float q0 = x * inv;
  const float r = fmaf(-q0, s, x);
  return fmaf(r, inv, q0);
}
__device__ __forceinline__ bool fast_quotient_ok(float amax) {
  return amax >= 8.673617379884035e-19f && amax <= 1.152921504606847e18f;  // 2^-60 .. 2^60
}
// x / s by the fast quotient (FAST) or by the IEEE division; callers branch once per row
template <bool FAST>
__device__ __forceinline__ float row_div(float x, float s, float inv) {
  if constexpr (FAST) return div_by_scale(x, s, inv);
  else return s > 0.f ? __fdiv_rn(x, s) : 0.f;
}

// The interpreter formula rint(x / scale) on 16 values held as 8 packed words: exact quotient
// (above), then round-half-to-even by the 1.5*2^23 adder trick; |x/scale| <= 127 so the low byte
// of the sum is the two's-complement int8 and no clamp is needed.  scale == 0 gives inv == 0 -> 0.
template <typename T, bool FAST>
__device__ __forceinline__ uint4 quant16_i8(const uint32_t (&w)[8], float scale, float inv) {
  constexpr float MAGIC = 12582912.f;  // 1.5 * 2^23
  uint32_t b[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    b[2 * i] = __float_as_uint(row_div<FAST>(Elem<T>::lo(w[i]), scale, inv) + MAGIC);
    b[2 * i + 1] = __float_as_uint(row_div<FAST>(Elem<T>::hi(w[i]), scale, inv) + MAGIC);
  }
  uint4 o;
  uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t lo = __byte_perm(b[4 * i], b[4 * i + 1], 0x0040);      // bytes: b0.0, b1.0
    uint32_t hi = __byte_perm(b[4 * i + 2], b[4 * i + 3], 0x0040);  // bytes: b2.0, b3.0
    po[i] = __byte_perm(lo, hi, 0x5410);
  }
  return o;
}

// The benchmark driver's golden on 16 values (benchmarks/bench_l1.py:443-448, evaluated in the
// input dtype's tensor arithmetic): round(h(h(x / a) * 127)) with h = round-to-input-dtype and
// a = amax clamped below by h(1e-8); IEEE division, NaN (0/0 cannot occur after the clamp) -> 0.
template <typename T>
__device__ __forceinline__ uint4 quant16_i8_golden(const uint32_t (&w)[8], float a) {
  uint32_t b[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float x0 = Elem<T>::lo(w[i]), x1 = Elem<T>::hi(w[i]);
    float r0 = rintf(Elem<T>::round(Elem<T>::round(__fdiv_rn(x0, a)) * 127.f));
    float r1 = rintf(Elem<T>::round(Elem<T>::round(__fdiv_rn(x1, a)) * 127.f));
    r0 = (r0 == r0) ? fminf(fmaxf(r0, -128.f), 127.f) : 0.f;
    r1 = (r1 == r1) ? fminf(fmaxf(r1, -128.f), 127.f) : 0.f;
    b[2 * i] = (uint32_t)(int)r0;
    b[2 * i + 1] = (uint32_t)(int)r1;
  }
  uint4 o;
  uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lo = __byte_perm(b[4 * i], b[4 * i + 1], 0x0040);
    const uint32_t hi = __byte_perm(b[4 * i + 2], b[4 * i + 3], 0x0040);
    po[i] = __byte_perm(lo, hi, 0x5410);
  }
  return o;
}

template <typename T, bool FAST>
__device__ __forceinline__ uint4 quant16_e4m3(const uint32_t (&w)[8], float scale, float inv) {
  uint4 o;
  uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint16_t a = pack_e4m3x2(row_div<FAST>(Elem<T>::lo(w[2 * i]), scale, inv),
                             row_div<FAST>(Elem<T>::hi(w[2 * i]), scale, inv));
    uint16_t c = pack_e4m3x2(row_div<FAST>(Elem<T>::lo(w[2 * i + 1]), scale, inv),
                             row_div<FAST>(Elem<T>::hi(w[2 * i + 1]), scale, inv));
    po[i] = (uint32_t)a | ((uint32_t)c << 16);
  }
  return o;
}

// eight values (one 16-byte input vector) -> eight quantised bytes
template <typename T, bool FAST>
__device__ __forceinline__ uint2 quant8_i8(const uint4 v, float scale, float inv) {
  constexpr float MAGIC = 12582912.f;
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t b[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    b[2 * i] = __float_as_uint(row_div<FAST>(Elem<T>::lo(w[i]), scale, inv) + MAGIC);
    b[2 * i + 1] = __float_as_uint(row_div<FAST>(Elem<T>::hi(w[i]), scale, inv) + MAGIC);
  }
  uint2 o;
  o.x = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
  o.y = __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410);
  return o;
}
template <typename T, bool FAST>
__device__ __forceinline__ uint2 quant8_e4m3(const uint4 v, float scale, float inv) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint16_t h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    h[i] = pack_e4m3x2(row_div<FAST>(Elem<T>::lo(w[i]), scale, inv), row_div<FAST>(Elem<T>::hi(w[i]), scale, inv));
  return make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
}

// --------------------------------------------------------------------------------------------
// quantize_per_token, register-resident fast path (N % 16 == 0, 16-byte aligned rows)
//   OUT = 0: int8 with scale = amax / 127 ; OUT = 1: e4m3 with scale = amax / 448
//   FORMULA = 1 (int8 only): the benchmark driver's golden, scale output = clamped amax
// --------------------------------------------------------------------------------------------
template <typename T, int TPR, int VPT, int OUT, int FORMULA = 0>
__global__ void __launch_bounds__(256)
quant_rows_kernel(const T* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q, int64_t ldq,
                  float* __restrict__ scale_out, int M, int N) {
  constexpr int RPB = 256 / TPR;
  __shared__ float red[8];
  // A GEMM launched behind this kernel with programmatic stream serialization may start its
  // set-up now.  (Launching this kernel itself that way, behind a GEMM, measured 1 % slower.)
  pdl_launch_dependents();
  const int t = threadIdx.x % TPR;
  const int64_t row = (int64_t)blockIdx.x * RPB + threadIdx.x / TPR;
  const bool row_ok = row < M;
  const int nvec = N >> 4;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (row_ok ? row : 0) * ldx);

  uint4 v[VPT][2];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = t + i * TPR;
    if (row_ok && vi < nvec && ARKE_CHK(row * ldx + 16 * vi, row * ldx + 16 * vi + 15, span_elems(M, N, ldx))) {
      v[i][0] = ld_stream(xr + 2 * vi);
      v[i][1] = ld_stream(xr + 2 * vi + 1);
    } else {
      v[i][0] = make_uint4(0, 0, 0, 0);
      v[i][1] = make_uint4(0, 0, 0, 0);
    }
  }
  uint32_t m2 = 0;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m2 = absmax2<T>(m2, v[i][h].x);
      m2 = absmax2<T>(m2, v[i][h].y);
      m2 = absmax2<T>(m2, v[i][h].z);
      m2 = absmax2<T>(m2, v[i][h].w);
    }
  }
  float amax = fmaxf(Elem<T>::lo(m2), Elem<T>::hi(m2));
  amax = group_max<TPR>(amax, red);

  const float scale = FORMULA == 0 ? __fdiv_rn(amax, OUT == 0 ? 127.f : 448.f) : fmaxf(amax, Elem<T>::round(1e-8f));
  const float inv = scale > 0.f ? __fdiv_rn(1.f, scale) : 0.f;
  const bool fast = fast_quotient_ok(amax);
  if (row_ok && t == 0 && ARKE_CHK(row, row, M)) scale_out[row] = scale;

  uint4* qr = reinterpret_cast<uint4*>(q + (row_ok ? row : 0) * ldq);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = t + i * TPR;
    if (row_ok && vi < nvec && ARKE_CHK(row * ldq + 16 * vi, row * ldq + 16 * vi + 15, span_elems(M, N, ldq))) {
      uint32_t w[8] = {v[i][0].x, v[i][0].y, v[i][0].z, v[i][0].w,
                       v[i][1].x, v[i][1].y, v[i][1].z, v[i][1].w};
      uint4 o;
      if constexpr (FORMULA == 1) {
        o = quant16_i8_golden<T>(w, scale);
      } else if (fast) {
        if constexpr (OUT == 0) o = quant16_i8<T, true>(w, scale, inv);
        else o = quant16_e4m3<T, true>(w, scale, inv);
      } else {
        if constexpr (OUT == 0) o = quant16_i8<T, false>(w, scale, inv);
        else o = quant16_e4m3<T, false>(w, scale, inv);
      }
      st_stream(qr + vi, o);
    }
  }
}

// --------------------------------------------------------------------------------------------
// quantize_per_token, any shape / alignment / dtype (one CTA per row, two passes, exact
// division everywhere).  FORMULA 0 = interpreter (see above); FORMULA 1 = the benchmark
// driver's golden, benchmarks/bench_l1.py:443-448: round(h(h(x / amax) * 127)) with h =
// round-to-input-dtype, returning amax (clamped below by h(1e-8)) as the scale.
// --------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float load_f(const T* p) { return (float)*p; }
template <> __device__ __forceinline__ float load_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float load_f<__half>(const __half* p) { return __half2float(*p); }

template <typename T, int OUT, int FORMULA>
__global__ void __launch_bounds__(256)
quant_rows_generic_kernel(const T* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q,
                          int64_t ldq, float* __restrict__ scale_out, int M, int N) {
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * ldx;
  float amax = 0.f;
  for (int j = threadIdx.x; j < N; j += 256)
    if (ARKE_CHK(row * ldx + j, row * ldx + j, span_elems(M, N, ldx))) amax = fmaxf(amax, fabsf(load_f<T>(xr + j)));
  amax = group_max<256>(amax, red);
  uint8_t* qr = q + row * ldq;
  if constexpr (FORMULA == 0) {
    const float scale = __fdiv_rn(amax, OUT == 0 ? 127.f : 448.f);
    if (threadIdx.x == 0) scale_out[row] = scale;
    for (int j = threadIdx.x; j < N; j += 256) {
      if (!ARKE_CHK(row * ldq + j, row * ldq + j, span_elems(M, N, ldq))) continue;
      const float xv = load_f<T>(xr + j);
      if constexpr (OUT == 0) {
        qr[j] = (uint8_t)(int8_t)quant_exact(xv, scale);
      } else {
        const float tq = scale > 0.f ? __fdiv_rn(xv, scale) : 0.f;
        qr[j] = (uint8_t)(pack_e4m3x2(tq, 0.f) & 0xff);
      }
    }
  } else {
    const float a = fmaxf(amax, Elem<T>::round(1e-8f));
    if (threadIdx.x == 0) scale_out[row] = a;
    for (int j = threadIdx.x; j < N; j += 256) {
      if (!ARKE_CHK(row * ldq + j, row * ldq + j, span_elems(M, N, ldq))) continue;
      const float xv = load_f<T>(xr + j);
      float t1 = Elem<T>::round(__fdiv_rn(xv, a));   // 0/0 -> NaN -> 0 below
      float t2 = Elem<T>::round(t1 * 127.f);
      float r = rintf(t2);
      r = (r == r) ? fminf(fmaxf(r, -128.f), 127.f) : 0.f;
      qr[j] = (uint8_t)(int8_t)(int)r;
    }
  }
}

// --------------------------------------------------------------------------------------------
// silu_and_mul on a packed [M, 2N] input (gate = cols [0,N), up = cols [N,2N)), with optional
// bf16/fp16 output Y and optional fused per-row e4m3 re-quantization of Y (scale = amax/448).
// silu is evaluated in fp32, rounded to the input dtype, multiplied by `up` in the input dtype
// (one more rounding) exactly like the eager reference; amax / quantisation act on that
// rounded Y so the fused result equals the two-step one.
// --------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ uint32_t silu_mul2(uint32_t g, uint32_t u) {
  constexpr float NLOG2E = -1.4426950408889634f;
  const float g0 = Elem<T>::lo(g), g1 = Elem<T>::hi(g);
  const float s0 = g0 * rcp_approx(1.f + ex2_approx(g0 * NLOG2E));
  const float s1 = g1 * rcp_approx(1.f + ex2_approx(g1 * NLOG2E));
  return mul2<T>(Elem<T>::pack(s0, s1), u);
}

template <typename T, int TPR, int VPT, bool WRITE_Y, bool WRITE_Q>
__global__ void __launch_bounds__(TPR)
swiglu_rows_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y, int64_t ldy,
                   uint8_t* __restrict__ q, int64_t ldq, float* __restrict__ scale_out, int M,
                   int N) {
  __shared__ float red[32];
  const int t = threadIdx.x;
  const int64_t row = blockIdx.x;
  const int nvec = N >> 4;
  const uint4* gr = reinterpret_cast<const uint4*>(x + row * ldx);
  const uint4* ur = reinterpret_cast<const uint4*>(x + row * ldx + N);

  uint32_t yv[VPT][8];
  {
    uint4 g[VPT][2], u[VPT][2];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = t + i * TPR;
      if (vi < nvec && ARKE_CHK(row * ldx + N + 16 * vi, row * ldx + N + 16 * vi + 15, span_elems(M, 2 * (long long)N, ldx))) {
        g[i][0] = ld_stream(gr + 2 * vi);
        g[i][1] = ld_stream(gr + 2 * vi + 1);
        u[i][0] = ld_stream(ur + 2 * vi);
        u[i][1] = ld_stream(ur + 2 * vi + 1);
      } else {
        g[i][0] = g[i][1] = u[i][0] = u[i][1] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        yv[i][4 * h + 0] = silu_mul2<T>(g[i][h].x, u[i][h].x);
        yv[i][4 * h + 1] = silu_mul2<T>(g[i][h].y, u[i][h].y);
        yv[i][4 * h + 2] = silu_mul2<T>(g[i][h].z, u[i][h].z);
        yv[i][4 * h + 3] = silu_mul2<T>(g[i][h].w, u[i][h].w);
      }
    }
  }
  if constexpr (WRITE_Y) {
    uint4* yr = reinterpret_cast<uint4*>(y + row * ldy);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = t + i * TPR;
      if (vi < nvec && ARKE_CHK(row * ldy + 16 * vi, row * ldy + 16 * vi + 15, span_elems(M, N, ldy))) {
        st_stream(yr + 2 * vi, make_uint4(yv[i][0], yv[i][1], yv[i][2], yv[i][3]));
        st_stream(yr + 2 * vi + 1, make_uint4(yv[i][4], yv[i][5], yv[i][6], yv[i][7]));
      }
    }
  }
  if constexpr (WRITE_Q) {
    uint32_t m2 = 0;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int k = 0; k < 8; ++k) m2 = absmax2<T>(m2, yv[i][k]);
    float amax = fmaxf(Elem<T>::lo(m2), Elem<T>::hi(m2));
    // block-wide max (TPR threads, one row per CTA)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((t & 31) == 0) red[t >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < TPR / 32; ++i) amax = fmaxf(amax, red[i]);
    const float scale = __fdiv_rn(amax, 448.f);
    const float inv = scale > 0.f ? __fdiv_rn(1.f, scale) : 0.f;
    const bool fast = fast_quotient_ok(amax);
    if (t == 0 && ARKE_CHK(row, row, M)) scale_out[row] = scale;
    uint4* qr = reinterpret_cast<uint4*>(q + row * ldq);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = t + i * TPR;
      if (vi < nvec && ARKE_CHK(row * ldq + 16 * vi, row * ldq + 16 * vi + 15, span_elems(M, N, ldq))) st_stream(qr + vi, fast ? quant16_e4m3<T, true>(yv[i], scale, inv) : quant16_e4m3<T, false>(yv[i], scale, inv));
    }
  }
}

// any-shape fallback: one CTA per row, scalar accesses, Y recomputed in the second pass
template <typename T>
__device__ __forceinline__ float silu_mul1(float g, float u) {
  const float s = Elem<T>::round(g / (1.f + expf(-g)));
  return Elem<T>::round(s * u);
}
template <typename T>
__device__ __forceinline__ void store_t(T* p, float v);
template <> __device__ __forceinline__ void store_t<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void store_t<__half>(__half* p, float v) { *p = __float2half_rn(v); }
template <> __device__ __forceinline__ void store_t<float>(float* p, float v) { *p = v; }

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_rows_generic_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y, int64_t ldy,
                           uint8_t* __restrict__ q, int64_t ldq, float* __restrict__ scale_out,
                           int M, int N) {
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  const T* gr = x + row * ldx;
  const T* ur = gr + N;
  float amax = 0.f;
  for (int j = threadIdx.x; j < N; j += 256) {
    if (!ARKE_CHK(row * ldx + j, row * ldx + N + j, span_elems(M, 2 * (long long)N, ldx))) continue;
    const float v = silu_mul1<T>(load_f<T>(gr + j), load_f<T>(ur + j));
    if (y && ARKE_CHK(row * ldy + j, row * ldy + j, span_elems(M, N, ldy))) store_t<T>(y + row * ldy + j, v);
    amax = fmaxf(amax, fabsf(v));
  }
  if (!q) return;
  amax = group_max<256>(amax, red);
  const float scale = __fdiv_rn(amax, 448.f);
  if (threadIdx.x == 0) scale_out[row] = scale;
  for (int j = threadIdx.x; j < N; j += 256) {
    const float v = silu_mul1<T>(load_f<T>(gr + j), load_f<T>(ur + j));
    const float tq = scale > 0.f ? __fdiv_rn(v, scale) : 0.f;
    q[row * ldq + j] = (uint8_t)(pack_e4m3x2(tq, 0.f) & 0xff);
  }
}

// --------------------------------------------------------------------------------------------
// rmsnorm / rmsnorm_residual (arke/ir/ops/reference_impls.py:85-90 and ref_rmsnorm_residual):
//   h = x (+ residual);  y = T(h / sqrt(mean(h^2) + eps) * w)   with fp32 math on 16-bit inputs,
// optionally fused with the per-token quantisation of the rounded y (the op that follows it in a
// W8A8 layer), so that y never has to be written or re-read.  One group of TPR threads per row,
// the row stays in registers across the two reductions (sum of squares, then amax).
// --------------------------------------------------------------------------------------------
template <int TPR>
__device__ __forceinline__ float group_sum(float v, float* red) {
  constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) red[warp] = v;
    __syncthreads();
    const int base = (warp / WPR) * WPR;
    v = red[base];
#pragma unroll
    for (int i = 1; i < WPR; ++i) v += red[base + i];
  }
  return v;
}

// QOUT: -1 no quantised output, 0 int8, 1 e4m3
template <typename T, int TPR, int VPT, bool HAS_RES, bool WRITE_Y, int QOUT>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ res, int64_t ldr,
                    const T* __restrict__ w, float eps, T* __restrict__ y, int64_t ldy,
                    uint8_t* __restrict__ q, int64_t ldq, float* __restrict__ scale_out, int M, int N) {
  constexpr int RPB = 256 / TPR;
  __shared__ float red_a[8], red_b[8];
  const int t = threadIdx.x % TPR;
  const int64_t row = (int64_t)blockIdx.x * RPB + threadIdx.x / TPR;
  const bool row_ok = row < M;
  const int nvec = N >> 3;  // 16-byte vectors of 8 elements
  const uint4* xr = reinterpret_cast<const uint4*>(x + (row_ok ? row : 0) * ldx);
  const uint4* rr = HAS_RES ? reinterpret_cast<const uint4*>(res + (row_ok ? row : 0) * ldr) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(w);

  float h[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = t + i * TPR;
    uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
    if (row_ok && vi < nvec && ARKE_CHK(row * ldx + 8 * vi, row * ldx + 8 * vi + 7, span_elems(M, N, ldx)) &&
        (!HAS_RES || ARKE_CHK(row * ldr + 8 * vi, row * ldr + 8 * vi + 7, span_elems(M, N, ldr)))) {
      a = ld_stream(xr + vi);
      if constexpr (HAS_RES) b = ld_stream(rr + vi);
    }
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float v0 = Elem<T>::lo(aw[k]), v1 = Elem<T>::hi(aw[k]);
      if constexpr (HAS_RES) {
        v0 += Elem<T>::lo(bw[k]);
        v1 += Elem<T>::hi(bw[k]);
      }
      h[i][2 * k] = v0;
      h[i][2 * k + 1] = v1;
      ss = fmaf(v0, v0, ss);
      ss = fmaf(v1, v1, ss);
    }
  }
  ss = group_sum<TPR>(ss, red_a);
  const float inv_rms = __fdiv_rn(1.f, sqrtf(__fdiv_rn(ss, (float)N) + eps));

  uint32_t yv[VPT][4];
  uint32_t m2 = 0;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = t + i * TPR;
    uint4 wv = make_uint4(0, 0, 0, 0);
    if (vi < nvec && ARKE_CHK(8 * vi, 8 * vi + 7, N)) wv = __ldg(wr + vi);
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float y0 = (h[i][2 * k] * inv_rms) * Elem<T>::lo(ww[k]);
      const float y1 = (h[i][2 * k + 1] * inv_rms) * Elem<T>::hi(ww[k]);
      yv[i][k] = Elem<T>::pack(y0, y1);
      if constexpr (QOUT >= 0) m2 = absmax2<T>(m2, yv[i][k]);
    }
    if constexpr (WRITE_Y) {
      if (row_ok && vi < nvec && ARKE_CHK(row * ldy + 8 * vi, row * ldy + 8 * vi + 7, span_elems(M, N, ldy)))
        st_stream(reinterpret_cast<uint4*>(y + row * ldy) + vi, make_uint4(yv[i][0], yv[i][1], yv[i][2], yv[i][3]));
    }
  }
  if constexpr (QOUT >= 0) {
    float amax = fmaxf(Elem<T>::lo(m2), Elem<T>::hi(m2));
    amax = group_max<TPR>(amax, red_b);
    const float scale = __fdiv_rn(amax, QOUT == 0 ? 127.f : 448.f);
    const float inv = scale > 0.f ? __fdiv_rn(1.f, scale) : 0.f;
    const bool fast = fast_quotient_ok(amax);
    if (row_ok && t == 0 && ARKE_CHK(row, row, M)) scale_out[row] = scale;
    uint2* qr = reinterpret_cast<uint2*>(q + (row_ok ? row : 0) * ldq);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = t + i * TPR;
      if (row_ok && vi < nvec && ARKE_CHK(row * ldq + 8 * vi, row * ldq + 8 * vi + 7, span_elems(M, N, ldq))) {
        const uint4 d = make_uint4(yv[i][0], yv[i][1], yv[i][2], yv[i][3]);
        uint2 o;
        if (fast) {
          if constexpr (QOUT == 0) o = quant8_i8<T, true>(d, scale, inv);
          else o = quant8_e4m3<T, true>(d, scale, inv);
        } else {
          if constexpr (QOUT == 0) o = quant8_i8<T, false>(d, scale, inv);
          else o = quant8_e4m3<T, false>(d, scale, inv);
        }
        st_stream(qr + vi, o);
      }
    }
  }
}

// any shape / alignment / dtype: one CTA per row, scalar accesses, three passes over the row
template <typename T, bool HAS_RES, int QOUT>
__global__ void __launch_bounds__(256)
rmsnorm_rows_generic_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ res, int64_t ldr,
                            const T* __restrict__ w, float eps, T* __restrict__ y, int64_t ldy,
                            uint8_t* __restrict__ q, int64_t ldq, float* __restrict__ scale_out, int M, int N) {
  __shared__ float red_a[8], red_b[8];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * ldx;
  const T* rr = HAS_RES ? res + row * ldr : nullptr;
  auto hval = [&](int j) {
    if (!ARKE_CHK(row * ldx + j, row * ldx + j, span_elems(M, N, ldx))) return 0.f;
    float v = load_f<T>(xr + j);
    if constexpr (HAS_RES) {
      if (ARKE_CHK(row * ldr + j, row * ldr + j, span_elems(M, N, ldr))) v += load_f<T>(rr + j);
    }
    return v;
  };
  float ss = 0.f;
  for (int j = threadIdx.x; j < N; j += 256) { const float v = hval(j); ss = fmaf(v, v, ss); }
  ss = group_sum<256>(ss, red_a);
  const float inv_rms = __fdiv_rn(1.f, sqrtf(__fdiv_rn(ss, (float)N) + eps));
  float amax = 0.f;
  for (int j = threadIdx.x; j < N; j += 256) {
    const float yy = Elem<T>::round((hval(j) * inv_rms) * load_f<T>(w + j));
    if (y && ARKE_CHK(row * ldy + j, row * ldy + j, span_elems(M, N, ldy))) store_t<T>(y + row * ldy + j, yy);
    amax = fmaxf(amax, fabsf(yy));
  }
  if constexpr (QOUT >= 0) {
    amax = group_max<256>(amax, red_b);
    const float scale = __fdiv_rn(amax, QOUT == 0 ? 127.f : 448.f);
    if (threadIdx.x == 0) scale_out[row] = scale;
    for (int j = threadIdx.x; j < N; j += 256) {
      const float yy = Elem<T>::round((hval(j) * inv_rms) * load_f<T>(w + j));
      if (!ARKE_CHK(row * ldq + j, row * ldq + j, span_elems(M, N, ldq))) continue;
      if constexpr (QOUT == 0) q[row * ldq + j] = (uint8_t)(int8_t)quant_exact(yy, scale);
      else q[row * ldq + j] = (uint8_t)(pack_e4m3x2(scale > 0.f ? __fdiv_rn(yy, scale) : 0.f, 0.f) & 0xff);
    }
  }
}

// --------------------------------------------------------------------------------------------
// dequantize_per_channel (arke/ir/ops/reference_impls.py:220-224): Y[i,j] = (X[i,j] - zp[j]) * s[j]
// in fp32, X int8, zero point optional (fp32 values), output fp32 / bf16 / f16.  Flat elementwise
// kernel, 16 elements per thread (one 128-bit load), grid-stride.
// --------------------------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256)
dequant_per_channel_kernel(const int8_t* __restrict__ x, int64_t ldx, const float* __restrict__ scale,
                           const float* __restrict__ zp, TO* __restrict__ y, int64_t ldy, int M, int N) {
  const int nvec = (N + 15) >> 4;
  const int64_t total = (int64_t)M * nvec;
  const bool vec = (N & 15) == 0 && (ldx & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  for (int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * 256) {
    const int64_t row = idx / nvec;
    const int c0 = (int)(idx - row * nvec) << 4;
    int8_t v[16];
    if (!ARKE_CHK(row * ldx + c0, row * ldx + min(c0 + 15, N - 1), span_elems(M, N, ldx))) continue;
    if (vec) {
      *reinterpret_cast<uint4*>(v) = ld_stream(reinterpret_cast<const uint4*>(x + row * ldx + c0));
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = (c0 + i < N) ? x[row * ldx + c0 + i] : (int8_t)0;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int c = c0 + i;
      if (c < N && ARKE_CHK(row * ldy + c, row * ldy + c, span_elems(M, N, ldy))) {
        const float z = zp ? __ldg(zp + c) : 0.f;
        store_t<TO>(y + row * ldy + c, ((float)v[i] - z) * __ldg(scale + c));
      }
    }
  }
}

// --------------------------------------------------------------------------------------------
// Exhaustive device-side check of div_by_scale against the IEEE division over the whole domain
// the fast kernels use it on: every finite 16-bit x, every positive finite 16-bit amax >= |x|.
// --------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float bits16_to_float(uint32_t b) {
  return Elem<T>::lo(b & 0xffffu);
}
template <typename T>
__global__ void __launch_bounds__(256)
selftest_div_kernel(float denom, unsigned long long* mismatches, unsigned long long* checked) {
  // blockIdx.x enumerates the 2^15 positive amax bit patterns; threads sweep all 2^16 x patterns
  const float amax = bits16_to_float<T>(blockIdx.x);
  unsigned bad = 0, n = 0;
  if (amax > 0.f && amax < INFINITY && fast_quotient_ok(amax)) {
    const float scale = __fdiv_rn(amax, denom);
    if (scale > 0.f) {
      const float inv = __fdiv_rn(1.f, scale);
      for (uint32_t xb = threadIdx.x; xb < 65536u; xb += 256) {
        const float xv = bits16_to_float<T>(xb);
        if (!(fabsf(xv) <= amax)) continue;  // also skips NaN
        const float a = div_by_scale(xv, scale, inv);
        const float e = __fdiv_rn(xv, scale);
        if (denom == 127.f) {
          constexpr float MAGIC = 12582912.f;
          bad += ((__float_as_uint(a + MAGIC) ^ __float_as_uint(e + MAGIC)) & 0xffu) != 0;
        } else {
          const uint32_t ca = pack_e4m3x2(a, 0.f) & 0xff, ce = pack_e4m3x2(e, 0.f) & 0xff;
          bad += (ca != ce) && (((ca | ce) & 0x7f) != 0);  // +0 and -0 count as equal
        }
        ++n;
      }
    }
  }
  bad = __reduce_add_sync(0xffffffffu, bad);
  n = __reduce_add_sync(0xffffffffu, n);
  if ((threadIdx.x & 31) == 0) {
    if (bad) atomicAdd(mismatches, (unsigned long long)bad);
    atomicAdd(checked, (unsigned long long)n);
  }
}

// --------------------------------------------------------------------------------------------
// host-side dispatch
// --------------------------------------------------------------------------------------------
// threads per row / 16-byte vectors per thread for the 4096-wide rows of the benchmark shapes
#ifndef ARKE_Q256_TPR
#define ARKE_Q256_TPR 64
#define ARKE_Q256_VPT 4
#endif
#ifndef ARKE_R512_TPR
#define ARKE_R512_TPR 128
#define ARKE_R512_VPT 4
#endif
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T, int OUT, int FORMULA = 0>
static cudaError_t launch_quant_fast(const T* x, int64_t ldx, uint8_t* q, int64_t ldq, float* s,
                                     int M, int N, cudaStream_t st) {
  const int nvec = N / 16;
#define ARKE_Q(TPR, VPT)                                                                              \
  do {                                                                                                \
    constexpr int RPB = 256 / TPR;                                                                    \
    quant_rows_kernel<T, TPR, VPT, OUT, FORMULA><<<(M + RPB - 1) / RPB, 256, 0, st>>>(x, ldx, q, ldq, \
                                                                                      s, M, N);       \
    return cudaGetLastError();                                                                        \
  } while (0)
  if (nvec <= 32) ARKE_Q(32, 1);
  if (nvec <= 64) ARKE_Q(32, 2);
  if (nvec <= 128) ARKE_Q(32, 4);
  if (nvec <= 256) ARKE_Q(ARKE_Q256_TPR, ARKE_Q256_VPT);
  if (nvec <= 512) ARKE_Q(128, 4);
  if (nvec <= 1024) ARKE_Q(256, 4);
  if (nvec <= 2048) ARKE_Q(256, 8);
#undef ARKE_Q
  return cudaErrorInvalidValue;
}

template <typename T>
static int quant_dispatch(const T* x, int64_t ldx, uint8_t* q, int64_t ldq, float* s, int M, int N,
                          int out_kind, int formula, cudaStream_t st) {
  const bool vec_ok = sizeof(T) == 2 && N % 16 == 0 && N / 16 <= 2048 &&
                      aligned16(x) && aligned16(q) && ldx % 8 == 0 && ldq % 16 == 0;
  cudaError_t e;
  if constexpr (sizeof(T) == 2) {
    if (vec_ok) {
      if (formula == 1) e = launch_quant_fast<T, 0, 1>(x, ldx, q, ldq, s, M, N, st);
      else e = out_kind == 0 ? launch_quant_fast<T, 0>(x, ldx, q, ldq, s, M, N, st)
                             : launch_quant_fast<T, 1>(x, ldx, q, ldq, s, M, N, st);
      return e == cudaSuccess ? ARKE_OK : set_cuda_error("quantize_per_token launch", e);
    }
  }
  if (formula == 0 && out_kind == 0)
    quant_rows_generic_kernel<T, 0, 0><<<M, 256, 0, st>>>(x, ldx, q, ldq, s, M, N);
  else if (formula == 0)
    quant_rows_generic_kernel<T, 1, 0><<<M, 256, 0, st>>>(x, ldx, q, ldq, s, M, N);
  else
    quant_rows_generic_kernel<T, 0, 1><<<M, 256, 0, st>>>(x, ldx, q, ldq, s, M, N);
  e = cudaGetLastError();
  return e == cudaSuccess ? ARKE_OK : set_cuda_error("quantize_per_token launch", e);
}

template <typename T>
static int swiglu_dispatch(const T* x, int64_t ldx, T* y, int64_t ldy, uint8_t* q, int64_t ldq,
                           float* s, int M, int N, cudaStream_t st) {
  cudaError_t e;
  const int nvec = N / 16;
  bool vec_ok = sizeof(T) == 2 && N % 16 == 0 && nvec <= 4096 && aligned16(x) && ldx % 8 == 0 &&
                (!y || (aligned16(y) && ldy % 8 == 0)) && (!q || (aligned16(q) && ldq % 16 == 0));
  if constexpr (sizeof(T) == 2) {
    if (vec_ok) {
#define ARKE_S(TPR, VPT)                                                                          \
  do {                                                                                            \
    if (y && q) swiglu_rows_kernel<T, TPR, VPT, true, true><<<M, TPR, 0, st>>>(x, ldx, y, ldy, q, ldq, s, M, N); \
    else if (q) swiglu_rows_kernel<T, TPR, VPT, false, true><<<M, TPR, 0, st>>>(x, ldx, y, ldy, q, ldq, s, M, N); \
    else swiglu_rows_kernel<T, TPR, VPT, true, false><<<M, TPR, 0, st>>>(x, ldx, y, ldy, q, ldq, s, M, N); \
  } while (0)
      if (nvec <= 32) ARKE_S(32, 1);
      else if (nvec <= 128) ARKE_S(64, 2);
      else if (nvec <= 256) ARKE_S(128, 2);
      else if (nvec <= 512) ARKE_S(256, 2);
      else if (nvec <= 1024) ARKE_S(256, 4);
      else if (nvec <= 2048) ARKE_S(512, 4);
      else ARKE_S(1024, 4);
#undef ARKE_S
      e = cudaGetLastError();
      return e == cudaSuccess ? ARKE_OK : set_cuda_error("silu_and_mul launch", e);
    }
  }
  swiglu_rows_generic_kernel<T><<<M, 256, 0, st>>>(x, ldx, y, ldy, q, ldq, s, M, N);
  e = cudaGetLastError();
  return e == cudaSuccess ? ARKE_OK : set_cuda_error("silu_and_mul launch", e);
}

}  // namespace arke

using namespace arke;

extern "C" int arke_b200_quantize_per_token(const void* x, int x_dtype, int64_t M, int64_t N,
                                            int64_t ldx, void* q, int64_t ldq, float* scale,
                                            int out_kind, int formula, void* stream) {
  ARKE_API_ENTER("arke_b200_quantize_per_token");
  if (M < 0 || N < 0 || M > INT32_MAX || N > INT32_MAX) return set_error(ARKE_ERR_SHAPE, "quantize_per_token: bad shape");
  if (M == 0 || N == 0) return ARKE_OK;
  if (!x || !q || !scale) return set_error(ARKE_ERR_ARG, "quantize_per_token: null pointer");
  if (out_kind != ARKE_QUANT_INT8 && out_kind != ARKE_QUANT_E4M3) return set_error(ARKE_ERR_ARG, "quantize_per_token: out_kind must be int8 (0) or e4m3 (1)");
  if (formula != 0 && formula != 1) return set_error(ARKE_ERR_ARG, "quantize_per_token: formula must be 0 (interpreter) or 1 (bench golden)");
  if (formula == 1 && out_kind != ARKE_QUANT_INT8) return set_error(ARKE_ERR_ARG, "quantize_per_token: formula 1 is int8 only");
  if (ldx < N || ldq < N) return set_error(ARKE_ERR_SHAPE, "quantize_per_token: row stride smaller than N");
  cudaStream_t st = (cudaStream_t)stream;
  switch (x_dtype) {
    case ARKE_BF16: return quant_dispatch((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, scale, (int)M, (int)N, out_kind, formula, st);
    case ARKE_F16: return quant_dispatch((const __half*)x, ldx, (uint8_t*)q, ldq, scale, (int)M, (int)N, out_kind, formula, st);
    case ARKE_F32: return quant_dispatch((const float*)x, ldx, (uint8_t*)q, ldq, scale, (int)M, (int)N, out_kind, formula, st);
    default: return set_error(ARKE_ERR_DTYPE, "quantize_per_token: input dtype must be bf16, f16 or f32");
  }
}

namespace arke {
template <typename T, bool HAS_RES, bool WRITE_Y, int QOUT>
static cudaError_t launch_rmsnorm_fast(const T* x, int64_t ldx, const T* res, int64_t ldr, const T* w, float eps,
                                       T* y, int64_t ldy, uint8_t* q, int64_t ldq, float* s, int M, int N,
                                       cudaStream_t st) {
  const int nvec = N / 8;
#define ARKE_R(TPR, VPT)                                                                            \
  do {                                                                                              \
    constexpr int RPB = 256 / TPR;                                                                  \
    rmsnorm_rows_kernel<T, TPR, VPT, HAS_RES, WRITE_Y, QOUT><<<(M + RPB - 1) / RPB, 256, 0, st>>>(  \
        x, ldx, res, ldr, w, eps, y, ldy, q, ldq, s, M, N);                                         \
    return cudaGetLastError();                                                                      \
  } while (0)
  if (nvec <= 32) ARKE_R(32, 1);
  if (nvec <= 64) ARKE_R(32, 2);
  if (nvec <= 128) ARKE_R(64, 2);
  if (nvec <= 256) ARKE_R(128, 2);
  if (nvec <= 512) ARKE_R(ARKE_R512_TPR, ARKE_R512_VPT);
  if (nvec <= 1024) ARKE_R(256, 4);
#undef ARKE_R
  return cudaErrorInvalidValue;
}

template <typename T>
static int rmsnorm_dispatch(const T* x, int64_t ldx, const T* res, int64_t ldr, const T* w, float eps, T* y,
                            int64_t ldy, uint8_t* q, int64_t ldq, float* s, int M, int N, int qout,
                            cudaStream_t st) {
  cudaError_t e = cudaErrorInvalidValue;
  bool launched = false;
  if constexpr (sizeof(T) == 2) {
    const bool vec_ok = N % 8 == 0 && N / 8 <= 1024 && aligned16(x) && ldx % 8 == 0 && aligned16(w) &&
                        (!res || (aligned16(res) && ldr % 8 == 0)) && (!y || (aligned16(y) && ldy % 8 == 0)) &&
                        (!q || ((reinterpret_cast<uintptr_t>(q) & 7) == 0 && ldq % 8 == 0));
    if (vec_ok) {
      launched = true;
#define ARKE_RD(HR, WY, QO) e = launch_rmsnorm_fast<T, HR, WY, QO>(x, ldx, res, ldr, w, eps, y, ldy, q, ldq, s, M, N, st)
      if (res) {
        if (y && qout < 0) ARKE_RD(true, true, -1);
        else if (y && qout == 0) ARKE_RD(true, true, 0);
        else if (y) ARKE_RD(true, true, 1);
        else if (qout == 0) ARKE_RD(true, false, 0);
        else ARKE_RD(true, false, 1);
      } else {
        if (y && qout < 0) ARKE_RD(false, true, -1);
        else if (y && qout == 0) ARKE_RD(false, true, 0);
        else if (y) ARKE_RD(false, true, 1);
        else if (qout == 0) ARKE_RD(false, false, 0);
        else ARKE_RD(false, false, 1);
      }
#undef ARKE_RD
    }
  }
  if (!launched) {
#define ARKE_RG(HR, QO) rmsnorm_rows_generic_kernel<T, HR, QO><<<M, 256, 0, st>>>(x, ldx, res, ldr, w, eps, y, ldy, q, ldq, s, M, N)
    if (res) {
      if (qout < 0) ARKE_RG(true, -1);
      else if (qout == 0) ARKE_RG(true, 0);
      else ARKE_RG(true, 1);
    } else {
      if (qout < 0) ARKE_RG(false, -1);
      else if (qout == 0) ARKE_RG(false, 0);
      else ARKE_RG(false, 1);
    }
#undef ARKE_RG
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? ARKE_OK : set_cuda_error("rmsnorm launch", e);
}
}  // namespace arke

extern "C" int arke_b200_rmsnorm(const void* x, const void* residual, const void* w, int dtype, int64_t M,
                                 int64_t N, int64_t ldx, int64_t ldr, float eps, void* y, int64_t ldy, void* q,
                                 int64_t ldq, float* scale, int out_kind, void* stream) {
  ARKE_API_ENTER("arke_b200_rmsnorm");
  if (M < 0 || N < 0 || M > INT32_MAX || N > INT32_MAX) return set_error(ARKE_ERR_SHAPE, "rmsnorm: bad shape");
  if (M == 0 || N == 0) return ARKE_OK;
  if (!x || !w) return set_error(ARKE_ERR_ARG, "rmsnorm: null input");
  if (!y && !q) return set_error(ARKE_ERR_ARG, "rmsnorm: no output requested");
  if (q && !scale) return set_error(ARKE_ERR_ARG, "rmsnorm: quantised output needs a scale buffer");
  if (q && out_kind != ARKE_QUANT_INT8 && out_kind != ARKE_QUANT_E4M3) return set_error(ARKE_ERR_ARG, "rmsnorm: out_kind must be int8 (0) or e4m3 (1)");
  if (ldx < N || (residual && ldr < N) || (y && ldy < N) || (q && ldq < N)) return set_error(ARKE_ERR_SHAPE, "rmsnorm: row stride smaller than N");
  const int qout = q ? out_kind : -1;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case ARKE_BF16: return rmsnorm_dispatch((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)residual, ldr, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)y, ldy, (uint8_t*)q, ldq, scale, (int)M, (int)N, qout, st);
    case ARKE_F16: return rmsnorm_dispatch((const __half*)x, ldx, (const __half*)residual, ldr, (const __half*)w, eps, (__half*)y, ldy, (uint8_t*)q, ldq, scale, (int)M, (int)N, qout, st);
    case ARKE_F32: return rmsnorm_dispatch((const float*)x, ldx, (const float*)residual, ldr, (const float*)w, eps, (float*)y, ldy, (uint8_t*)q, ldq, scale, (int)M, (int)N, qout, st);
    default: return set_error(ARKE_ERR_DTYPE, "rmsnorm: dtype must be bf16, f16 or f32");
  }
}

extern "C" int arke_b200_dequantize_per_channel(const void* x, int64_t M, int64_t N, int64_t ldx, const float* scale,
                                                const float* zero_point, void* y, int y_dtype, int64_t ldy,
                                                void* stream) {
  ARKE_API_ENTER("arke_b200_dequantize_per_channel");
  if (M < 0 || N < 0 || M > INT32_MAX || N > INT32_MAX) return set_error(ARKE_ERR_SHAPE, "dequantize_per_channel: bad shape");
  if (M == 0 || N == 0) return ARKE_OK;
  if (!x || !scale || !y) return set_error(ARKE_ERR_ARG, "dequantize_per_channel: null pointer");
  if (ldx < N || ldy < N) return set_error(ARKE_ERR_SHAPE, "dequantize_per_channel: row stride smaller than N");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t work = M * ((N + 15) / 16);
  int grid = (int)((work + 255) / 256);
  const int cap = sm_count() * 16;
  if (cap > 0 && grid > cap) grid = cap;
  const int8_t* xi = (const int8_t*)x;
  switch (y_dtype) {
    case ARKE_F32: dequant_per_channel_kernel<float><<<grid, 256, 0, st>>>(xi, ldx, scale, zero_point, (float*)y, ldy, (int)M, (int)N); break;
    case ARKE_BF16: dequant_per_channel_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(xi, ldx, scale, zero_point, (__nv_bfloat16*)y, ldy, (int)M, (int)N); break;
    case ARKE_F16: dequant_per_channel_kernel<__half><<<grid, 256, 0, st>>>(xi, ldx, scale, zero_point, (__half*)y, ldy, (int)M, (int)N); break;
    default: return set_error(ARKE_ERR_DTYPE, "dequantize_per_channel: output dtype must be f32, bf16 or f16");
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? ARKE_OK : set_cuda_error("dequantize_per_channel launch", e);
}

extern "C" int arke_b200_selftest_quant_division(int x_dtype, int out_kind, unsigned long long* counters,
                                                 void* stream) {
  if (!counters) return set_error(ARKE_ERR_ARG, "selftest_quant_division: null counters");
  if (x_dtype != ARKE_BF16 && x_dtype != ARKE_F16) return set_error(ARKE_ERR_DTYPE, "selftest_quant_division: dtype must be bf16 or f16");
  if (out_kind != ARKE_QUANT_INT8 && out_kind != ARKE_QUANT_E4M3) return set_error(ARKE_ERR_ARG, "selftest_quant_division: bad out_kind");
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(counters, 0, 2 * sizeof(unsigned long long), st);
  if (e != cudaSuccess) return set_cuda_error("selftest_quant_division memset", e);
  const float denom = out_kind == ARKE_QUANT_INT8 ? 127.f : 448.f;
  if (x_dtype == ARKE_BF16) selftest_div_kernel<__nv_bfloat16><<<32768, 256, 0, st>>>(denom, counters, counters + 1);
  else selftest_div_kernel<__half><<<32768, 256, 0, st>>>(denom, counters, counters + 1);
  e = cudaGetLastError();
  return e == cudaSuccess ? ARKE_OK : set_cuda_error("selftest_quant_division launch", e);
}

extern "C" int arke_b200_silu_and_mul(const void* x, int x_dtype, int64_t M, int64_t N,
                                      int64_t ldx, void* y, int64_t ldy, void* yq, int64_t ldq,
                                      float* scale, void* stream) {
  ARKE_API_ENTER("arke_b200_silu_and_mul");
  if (M < 0 || N < 0 || M > INT32_MAX || N > INT32_MAX) return set_error(ARKE_ERR_SHAPE, "silu_and_mul: bad shape");
  if (M == 0 || N == 0) return ARKE_OK;
  if (!x || (!y && !yq)) return set_error(ARKE_ERR_ARG, "silu_and_mul: null input or no output requested");
  if (yq && !scale) return set_error(ARKE_ERR_ARG, "silu_and_mul: e4m3 output needs a scale buffer");
  if (ldx < 2 * N || (y && ldy < N) || (yq && ldq < N)) return set_error(ARKE_ERR_SHAPE, "silu_and_mul: row stride too small");
  cudaStream_t st = (cudaStream_t)stream;
  switch (x_dtype) {
    case ARKE_BF16: return swiglu_dispatch((const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)y, ldy, (uint8_t*)yq, ldq, scale, (int)M, (int)N, st);
    case ARKE_F16: return swiglu_dispatch((const __half*)x, ldx, (__half*)y, ldy, (uint8_t*)yq, ldq, scale, (int)M, (int)N, st);
    case ARKE_F32: return swiglu_dispatch((const float*)x, ldx, (float*)y, ldy, (uint8_t*)yq, ldq, scale, (int)M, (int)N, st);
    default: return set_error(ARKE_ERR_DTYPE, "silu_and_mul: input dtype must be bf16, f16 or f32");
  }
}
