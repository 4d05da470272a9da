// Activation functions and their derivatives, shared by the GEMM epilogue and the element-wise kernels.
#pragma once
#include "gemm_tcgen05.h"

namespace mrk {

// erf-GELU without the special-function unit.  The epilogue warps evaluate the activation for every
// output element while the tensor core works on the next tile, and B200 issues 16 exp/rcp per clock
// per SM against 128 FMAs, so erf(x / sqrt 2) is an odd polynomial of degree 17 in x on [-4, 4]
// (least-squares fit at Chebyshev nodes; clamped outside, where 1 - erf < 6.4e-5): |error| < 6e-5
// in fp32 Horner form, far below the bf16 rounding of the outputs.  10 FMA-pipe instructions.
__device__ __forceinline__ float erf_sqrt2_poly(float x) {
  const float xc = fminf(fmaxf(x, -4.0f), 4.0f);
  const float t = xc * xc;
  float p = 1.91351286e-10f;
  p = fmaf(p, t, -1.605284763e-08f);
  p = fmaf(p, t, 6.00525788e-07f);
  p = fmaf(p, t, -1.344138827e-05f);
  p = fmaf(p, t, 2.050217931e-04f);
  p = fmaf(p, t, -2.30244045e-03f);
  p = fmaf(p, t, 1.984304585e-02f);
  p = fmaf(p, t, -1.329219091e-01f);
  p = fmaf(p, t, 7.978790106e-01f);
  return p * xc;
}
__device__ __forceinline__ float gelu_erf(float x) {
  const float hx = 0.5f * x;
  return fmaf(hx, erf_sqrt2_poly(x), hx);
}
// d/dx [x Phi(x)] = Phi(x) + x phi(x); the normal pdf costs the one exponential
__device__ __forceinline__ float gelu_erf_grad(float x) {
  const float cdf = fmaf(0.5f, erf_sqrt2_poly(x), 0.5f);
  const float pdf = 0.3989422804014327f * exp2f(-0.7213475204444817f * x * x);
  return fmaf(x, pdf, cdf);
}
__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + fast_tanh(u));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  const float t = fast_tanh(u);
  const float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x * x);
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
}
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float silu_grad(float x) {
  const float s = 1.0f / (1.0f + __expf(-x));
  return s * (1.0f + x * (1.0f - s));
}

template <int act>
__device__ __forceinline__ float apply_act(float v) {
  switch (act) {
    case MRK_ACT_GELU_ERF: return gelu_erf(v);
    case MRK_ACT_GELU_TANH: return gelu_tanh(v);
    case MRK_ACT_RELU: return v > 0.f ? v : 0.f;
    case MRK_ACT_SILU: return silu(v);
    default: return v;
  }
}
template <int act>
__device__ __forceinline__ float apply_act_grad(float x) {
  switch (act) {
    case MRK_ACT_GELU_ERF: return gelu_erf_grad(x);
    case MRK_ACT_GELU_TANH: return gelu_tanh_grad(x);
    case MRK_ACT_RELU: return x > 0.f ? 1.f : 0.f;
    case MRK_ACT_SILU: return silu_grad(x);
    default: return 1.f;
  }
}

}  // namespace mrk
