// Shared host/device helpers of libksmm_cu: element-type traits, vector
// load/store helpers, status plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ksmm_cu.h"

namespace ksmm {

// ---------------------------------------------------------------------------
// element types
// ---------------------------------------------------------------------------
struct f8e4m3 {
  uint8_t bits;
};

template <typename T>
struct ElemTraits;

template <>
struct ElemTraits<float> {
  static constexpr int kDtype = KSMM_F32;
  __device__ static float to_float(float v) { return v; }
  __device__ static float from_float(float v) { return v; }
};
template <>
struct ElemTraits<__half> {
  static constexpr int kDtype = KSMM_F16;
  __device__ static float to_float(__half v) { return __half2float(v); }
  __device__ static __half from_float(float v) { return __float2half_rn(v); }
};
template <>
struct ElemTraits<__nv_bfloat16> {
  static constexpr int kDtype = KSMM_BF16;
  __device__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct ElemTraits<f8e4m3> {
  static constexpr int kDtype = KSMM_F8E4M3;
  __device__ static float to_float(f8e4m3 v) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(v.bits, __NV_E4M3);
    return __half2float(__half(h));
  }
};

__host__ __device__ inline int dtype_size(int dt) {
  return dt == KSMM_F32 ? 4 : (dt == KSMM_F8E4M3 ? 1 : 2);
}

// ---------------------------------------------------------------------------
// N-wide (N = 1, 2, 4) global loads / stores with conversion to / from float.
// The caller guarantees N * sizeof(T) alignment when N > 1.
// ---------------------------------------------------------------------------
template <typename T, int N>
__device__ __forceinline__ void load_vec(const T* __restrict__ p, float (&out)[N]) {
  if constexpr (N == 1) {
    out[0] = ElemTraits<T>::to_float(*p);
  } else if constexpr (sizeof(T) == 4) {
    if constexpr (N == 4) {
      float4 v = __ldg(reinterpret_cast<const float4*>(p));
      out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
      float2 v = __ldg(reinterpret_cast<const float2*>(p));
      out[0] = v.x; out[1] = v.y;
    }
  } else if constexpr (sizeof(T) == 2) {
    if constexpr (N == 4) {
      uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
      T tmp[4];
      *reinterpret_cast<uint2*>(tmp) = raw;
#pragma unroll
      for (int e = 0; e < 4; ++e) out[e] = ElemTraits<T>::to_float(tmp[e]);
    } else {
      uint32_t raw = __ldg(reinterpret_cast<const uint32_t*>(p));
      T tmp[2];
      *reinterpret_cast<uint32_t*>(tmp) = raw;
      out[0] = ElemTraits<T>::to_float(tmp[0]);
      out[1] = ElemTraits<T>::to_float(tmp[1]);
    }
  } else {
    if constexpr (N == 4) {
      uint32_t raw = __ldg(reinterpret_cast<const uint32_t*>(p));
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        T t; t.bits = (raw >> (8 * e)) & 0xffu;
        out[e] = ElemTraits<T>::to_float(t);
      }
    } else {
      uint16_t raw = __ldg(reinterpret_cast<const uint16_t*>(p));
      T t0, t1; t0.bits = raw & 0xffu; t1.bits = raw >> 8;
      out[0] = ElemTraits<T>::to_float(t0);
      out[1] = ElemTraits<T>::to_float(t1);
    }
  }
}

template <typename T, int N>
__device__ __forceinline__ void store_vec(T* __restrict__ p, const float (&v)[N]) {
  if constexpr (N == 1) {
    *p = ElemTraits<T>::from_float(v[0]);
  } else if constexpr (sizeof(T) == 4) {
    if constexpr (N == 4) {
      *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
    }
  } else {
    T tmp[N];
#pragma unroll
    for (int e = 0; e < N; ++e) tmp[e] = ElemTraits<T>::from_float(v[e]);
    if constexpr (N == 4) {
      *reinterpret_cast<uint2*>(p) = *reinterpret_cast<uint2*>(tmp);
    } else {
      *reinterpret_cast<uint32_t*>(p) = *reinterpret_cast<uint32_t*>(tmp);
    }
  }
}

// ---------------------------------------------------------------------------
// problem description handed to every kernel family
// ---------------------------------------------------------------------------
struct Problem {
  const void* in;
  const void* w;
  void* out;
  const void* bias;
  int64_t batch;
  int a, b, c, d;
  int in_dtype, out_dtype;
  int bs_last;             // layout of the input (and of the output unless out_bs_last says otherwise)
  int out_bs_last = -1;    // -1: same as the input; 0 / 1: batch-first / batch-last output (d = 1 factors)
  float alpha;
  // Chains only.  out_regroup_d > 0: store the output regrouped by the blocks of the next factor
  // (c = out_regroup_c, d = out_regroup_d): feature (i2*c + k)*d + l goes to (i2*d + l)*c + k.
  // in_regrouped: the input already has that order for this factor's own (c, d).
  int out_regroup_d = 0, out_regroup_c = 0;
  int in_regrouped = 0;
  int activation = 0;  // ksmm_activation_t, applied after alpha and bias
  // optional tensor of the output's shape, layout and type, added last:
  // out = act(alpha * K x + bias) + residual
  const void* residual = nullptr;
  // Caller-provided memory for the paths that need a second copy of a tensor (layout conversion,
  // regrouping).  With scratch == nullptr the library's own per-stream scratch is used, unless
  // no_alloc is set: then the call fails with KSMM_ERR_WORKSPACE instead of allocating.
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  int no_alloc = 0;
  // groups > 1: that many problems of this pattern in one call.  Weights (groups, a*d*c, b) and
  // outputs (groups, ...) are stacked; the input is one tensor shared by all groups, or stacked
  // like the output when group_shared_input == 0.  The bias, if any, holds groups * a*b*d elements.
  int groups = 1;
  int group_shared_input = 1;
};

// element-wise epilogue function (ksmm_activation_t)
// erf by the rational approximation 7.1.26 of Abramowitz and Stegun (absolute error below
// 1.5e-7, i.e. fp32 rounding level for a GELU): one reciprocal, one exponential, six FMAs.
__device__ __forceinline__ float fast_erf(float x) {
  const float ax = fabsf(x);
  const float t = __frcp_rn(fmaf(0.3275911f, ax, 1.f));
  float p = fmaf(1.061405429f, t, -1.453152027f);
  p = fmaf(p, t, 1.421413741f);
  p = fmaf(p, t, -0.284496736f);
  p = fmaf(p, t, 0.254829592f);
  const float r = 1.f - p * t * __expf(-ax * ax);
  return copysignf(r, x);
}
__device__ __forceinline__ float apply_activation(float v, int act) {
  if (act == 1) return 0.5f * v * (1.f + fast_erf(v * 0.70710678118654752f));
  if (act == 2) return fmaxf(v, 0.f);
  return v;
}
// GELU for results that are rounded to 16 bits: erf(z) = tanh(z (c1 + c3 z^2 + c5 z^4)) to 4e-5
// (least-squares fit on [0, 4]; beyond it both sides are 1 to that accuracy), with the hardware's
// tanh.approx (relative error 2^-11).  The absolute error of the GELU stays below 5e-5 |x| + 2e-5,
// under half an fp16 / bf16 rounding step of the result; six FMA-pipe instructions and one
// special-function instruction per value, against fifteen and two for the form above.
__device__ __forceinline__ float gelu_16bit(float x) {
  // the coefficients below are c1 / sqrt 2, c3 / (2 sqrt 2), c5 / (4 sqrt 2): the polynomial is in x^2
  // (beyond |x| = 7 the fit is no longer meant to hold: the argument of the tanh is frozen there,
  // where tanh is 1 to fp32 accuracy, so that the negative x^4 term can never turn its sign)
  const float u = fminf(x * x, 49.f);
  float p = fmaf(u, -3.2060774e-4f, 3.6819428e-2f);
  p = fmaf(p, u, 7.9770428e-1f);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x * p));
  const float h = 0.5f * x;
  return fmaf(h, t, h);
}

// host-side error plumbing (defined in ksmm_cu.cu)
int set_error(int status, const char* fmt, ...);
void count_launch();
// Device memory of at least `bytes` for the layout-conversion and regrouping paths: the
// problem's own scratch when it has one, else a library-owned buffer per (device, stream) that
// grows on demand (never during a stream capture).  Work on one stream is ordered, so calls on
// different streams never share a buffer.
int layout_scratch(const Problem& p, size_t bytes, cudaStream_t stream, void** out);

}  // namespace ksmm
