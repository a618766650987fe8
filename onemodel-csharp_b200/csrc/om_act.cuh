// The unary operators and their gradients as device functions: one definition for the element-wise kernels and for
// the product epilogues that apply an activation on the accumulator (om_gemm_ws.cu), so that a fused and an unfused
// path give the same bits.
#pragma once
#include "om_common.cuh"

namespace om {

// The erf GELU of the bfloat16-operand tier (OM_GELU_ERF_FAST, chosen by the callers that also write a bfloat16 copy of
// the result, never by the fp32 entry points): erf without a branch and with few instructions, because a product epilogue
// runs this arithmetic on a handful of warps under the next tile's MMAs. With u = 1 / (1 + 0.39 |z|):
//   erfc(|z|) = exp(-z*z) * u * Q(u),  Q of degree 5  (the form of Abramowitz & Stegun 7.1.26 with one more term; the
//   coefficients are a minimax fit made for this file: 8e-9 in exact arithmetic),  erf(z) = sign(z) (1 - erfc(|z|)).
// exp and the reciprocal are the hardware approximations (ex2.approx, rcp.approx). In fp32 the result is within 4e-7
// absolute of erf over the whole line, far inside the 2^-9 relative rounding of the bfloat16 copy that follows; exp(-z*z)
// is handed back for the Gaussian of the derivative. NaN comes back NaN.
constexpr int OM_GELU_ERF_FAST = 64;
// The argument is x, the value erf(x / sqrt 2): the scaling by 1 / sqrt 2 is folded into the two constants (these run in the
// epilogues of the feed-forward products, whose time is the number of instructions per element).
__device__ __forceinline__ float erf_fast(float x, float* gauss) {
  const float a = fabsf(x);
  float e, u;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"((x * x) * -0.72134752044448170f));   // exp(-x*x / 2)
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(u) : "f"(fmaf(a, 0.39f * 0.70710678f, 1.0f)));
  float q = -2.275369167e-01f;
  q = fmaf(q, u, 8.866635561e-01f);
  q = fmaf(q, u, -6.353989244e-01f);
  q = fmaf(q, u, 6.495583057e-01f);
  q = fmaf(q, u, 9.138885140e-02f);
  q = fmaf(q, u, 2.353251427e-01f);
  *gauss = e;
  return copysignf(1.0f - (q * u) * e, x);
}
__device__ __forceinline__ float gelu_erf_fast(float x) {
  float e;
  return x * fmaf(0.5f, erf_fast(x, &e), 0.5f);
}
__device__ __forceinline__ float gelu_erf(float x) { return (0.5f * x) * (1.0f + erff(x * 0.70710677f)); }
__device__ __forceinline__ float gelu_tanh(float x) {
  float u = 0.79788456f * (x + ((0.044715f * x) * x) * x);
  return (0.5f * x) * (1.0f + tanhf(u));
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

template <int OP>
__device__ __forceinline__ float unary_apply(float x) {
  if (OP == OM_RELU) return x > 0.0f ? x : (x == x ? 0.0f : x);
  if (OP == OM_GELU_ERF) return gelu_erf(x);
  if (OP == OM_GELU_ERF_FAST) return gelu_erf_fast(x);
  if (OP == OM_GELU_TANH) return gelu_tanh(x);
  if (OP == OM_SIGMOID) return sigmoidf_(x);
  if (OP == OM_TANH) return tanhf(x);
  if (OP == OM_NEG) return x * -1.0f;
  if (OP == OM_EXP) return expf(x);
  if (OP == OM_SQRT) return sqrtf(x);
  if (OP == OM_ERF) return erff(x);
  return x;
}

// g = incoming gradient, s = saved tensor (output or input, see the header).
template <int OP>
__device__ __forceinline__ float unary_grad(float g, float s) {
  if (OP == OM_RELU) return s > 0.0f ? g : 0.0f;
  if (OP == OM_SIGMOID) return (g * s) * (1.0f - s);
  if (OP == OM_TANH) return g * (1.0f - s * s);
  if (OP == OM_GELU_ERF) {
    float cdf = 0.5f * (1.0f + erff(s * 0.70710677f));
    float pdf = expf((-0.5f * s) * s) * 0.3989423f;
    return g * (cdf + s * pdf);
  }
  if (OP == OM_GELU_ERF_FAST) {
    // gauss is the Gaussian exp(-s*s / 2) of the density.
    float gauss;
    const float cdf = fmaf(0.5f, erf_fast(s, &gauss), 0.5f);
    return g * fmaf(s * 0.3989423f, gauss, cdf);
  }
  if (OP == OM_GELU_TANH) {
    float u = 0.79788456f * (s + ((0.044715f * s) * s) * s);
    float t = tanhf(u);
    float left = 0.5f * (1.0f + t);
    float right = (((0.5f * s) * (1.0f - t * t)) * 0.79788456f) * (1.0f + ((3.0f * 0.044715f) * s) * s);
    return g * (left + right);
  }
  if (OP == OM_NEG) return g * -1.0f;
  if (OP == OM_EXP) return g * s;                       // s = exp(x)
  if (OP == OM_SQRT) return g / (2.0f * s);             // s = sqrt(x)
  if (OP == OM_ERF) return g * (1.1283791671f * expf(-(s * s)));  // s = x
  return g;
}

// An activation and its derivative at the same point, for a product epilogue that leaves both behind (the derivative is what
// the backward pass multiplies by, so nothing of the activation has to be evaluated again there). deriv equals
// unary_grad<OP>(1, x), bit for bit: the erf form shares its erf and its Gaussian between the two.
template <int OP>
__device__ __forceinline__ void unary_both(float x, float* act, float* deriv) {
  if (OP == OM_GELU_ERF_FAST) {
    float gauss;
    const float cdf = fmaf(0.5f, erf_fast(x, &gauss), 0.5f);
    *act = x * cdf;
    *deriv = fmaf(x * 0.3989423f, gauss, cdf);
  } else {
    *act = unary_apply<OP>(x);
    *deriv = unary_grad<OP>(1.0f, x);
  }
}

}  // namespace om
