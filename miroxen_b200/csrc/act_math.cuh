// The activation functions of the layer ops, shared by the in-place / two-input kernels
// (activations.cu) and by the kernels that quantise the activation as they produce it (blockscale.cu).
#pragma once

#include "common.cuh"

namespace mxk {

// 0.5 v (1 + tanh(u)), u = 0.7978845608 (v + 0.044715 v^3)  (src/kernels/ops.cu:222-224).
// 0.5 (1 + tanh(u)) is the logistic function of 2u, so the value is v / (1 + exp(-2u)) =
// v / (1 + 2^z) with z = -2 log2(e) u = v (B0 + B1 v^2): three multiply-adds, one ex2, one add,
// one reciprocal, one multiply.  There is no cancellation anywhere (the negative tail divides
// by a large number instead of adding 1 to a tanh near -1), and when 2^z overflows for very
// negative v the reciprocal is 0 and the result the correct limit -0.  Seven issue slots per
// element plus unpack and pack; at HBM speed the SM has to retire more than one element per
// clock per scheduler, so every slot counts.
__device__ __forceinline__ float gelu_tanh_f(float v) {
  constexpr float B0 = -2.f * 1.4426950408889634f * 0.7978845608f;
  constexpr float B1 = B0 * 0.044715f;
  const float z = v * fmaf(v * v, B1, B0);
  return v * rcp_approx(1.f + ex2_approx(z));
}

__device__ __forceinline__ float gelu_erf_f(float v) {
  return 0.5f * v * (1.f + erff(v * 0.7071067811865476f));
}

// g / (1 + exp(-g))  (src/kernels/ops.cu:127): exp through ex2, the division as a reciprocal.
__device__ __forceinline__ float silu_f(float g) {
  return g * rcp_approx(1.f + ex2_approx(g * -1.4426950408889634f));
}

// 8 bf16 plus 8 fp32 bias values, rounded back to bf16: what add_bias_bf16 leaves in memory
// (src/kernels/ops.cu:249-262), so the activation sees the same bits as after the separate call.
__device__ __forceinline__ uint4 add_bias8(const uint4& raw, const float* bias) {
  float v[8];
  unpack8(raw, v);
  const float4 b0 = *reinterpret_cast<const float4*>(bias), b1 = *reinterpret_cast<const float4*>(bias + 4);
  v[0] += b0.x, v[1] += b0.y, v[2] += b0.z, v[3] += b0.w, v[4] += b1.x, v[5] += b1.y, v[6] += b1.z, v[7] += b1.w;
  return pack8(v);
}

// Eight elements at a time on packed bf16.  ACT 0: GELU (tanh form) of a; 1: GELU (erf form) of a;
// 2: silu(a) * b.  The result is rounded to bf16 exactly as the stand-alone kernels round it.
enum { ACT_GELU_TANH = 0, ACT_GELU_ERF = 1, ACT_SILU_MUL = 2 };
template <int ACT>
__device__ __forceinline__ uint4 act8(const uint4& a, const uint4& b) {
  float v[8];
  unpack8(a, v);
  if (ACT == ACT_SILU_MUL) {
    float u[8];
    unpack8(b, u);
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = silu_f(v[i]) * u[i];
  } else {
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = ACT == ACT_GELU_TANH ? gelu_tanh_f(v[i]) : gelu_erf_f(v[i]);
  }
  return pack8(v);
}

}  // namespace mxk
