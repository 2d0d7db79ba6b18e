// Device helpers of the MXFP8 block-scale format shared by the stand-alone quantiser (blockscale.cu)
// and the kernels that quantise their own output (norm_mod.cuh): packed bf16 maxima, the ue8m0 scale
// exponent, e4m3 conversion, the address of a scale in cuBLASLt's interleaved layout.
#pragma once

#include <cuda_fp8.h>

#include "common.cuh"

namespace mxk {

__host__ __device__ inline int64_t pad_to(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// Two floats -> two e4m3 bytes (x in the low byte), round to nearest even, saturating.
__device__ __forceinline__ uint32_t e4m3x2(float2 v) {
  return __nv_cvt_float2_to_fp8x2(v, __NV_SATFINITE, __NV_E4M3);
}

// max(|a|, |b|) on both bf16 halves; the sign bits of the result are meaningless.
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t absmax_bf16x2(const uint4& u) {
  return absmax_bf16x2(absmax_bf16x2(u.x, u.y), absmax_bf16x2(u.z, u.w));
}
// Largest magnitude of the two halves, as fp32 (a bf16 value).
__device__ __forceinline__ float bf16x2_max_to_float(uint32_t m) {
  m = absmax_bf16x2(m, __byte_perm(m, 0, 0x1032));
  return __uint_as_float((m << 16) & 0x7fff0000u);
}
__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// Joins the warp's maxima and folds them into the tensor maximum at `out` (fp32, cleared beforehand): non-negative
// floats order like their bit patterns, so an integer atomicMax does it (src/kernels/blockscale.cu:68).  All 32
// lanes must call.
__device__ __forceinline__ void amax_commit(float m, float* out) {
#pragma unroll
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));
}

// ue8m0 scale exponent of a block whose largest magnitude is the bf16 value bmax: the smallest e with
// bmax / 2^e <= 448, clamped to [-127, 127] (src/kernels/blockscale.cu:111-119 computes it as
// frexpf(bmax / 448)).  With bmax = 1.m * 2^E, RN(bmax / 448) = RN(1.m / 1.75) * 2^(E-8), and 1.m / 1.75
// equals 1 only for 1.m = 1.75 and is otherwise more than 2^-8 away from 1: e is E - 8 when
// 1.m <= 1.75 and E - 7 above.  Zero and subnormal maxima clamp to -127.
__device__ __forceinline__ int ue8m0_exponent(float bmax) {
  const uint32_t b = __float_as_uint(bmax);
  const int E = int(b >> 23);
  const int e = E - 127 - 8 + ((b & 0x007fffffu) > 0x00600000u ? 1 : 0);
  return E == 0 ? -127 : max(-127, e);
}
// 2^-e for e in [-127, 120]: the exponent field is -e + 127, in [7, 254].
__device__ __forceinline__ float pow2_neg(int e) { return __uint_as_float(uint32_t(127 - e) << 23); }

// MXFP8 on 16 consecutive elements held by one thread (two vectors of 8 bf16), the two halves of a
// 32-element block sitting in neighbouring lanes.
__device__ __forceinline__ uint32_t mxfp8_block_absmax(const uint4 (&raw)[2]) {
  const uint32_t m = absmax_bf16x2(absmax_bf16x2(raw[0]), absmax_bf16x2(raw[1]));
  return absmax_bf16x2(m, __shfl_xor_sync(0xffffffffu, m, 1));
}
// out = 16 e4m3 bytes; returns the ue8m0 scale byte of the block.
__device__ __forceinline__ uint8_t mxfp8_quant16(const uint4 (&raw)[2], uint32_t packed_max, uint4& out) {
  const uint32_t w[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
  const int e = ue8m0_exponent(bf16x2_max_to_float(packed_max));
  const float inv = pow2_neg(e);
  const float2 inv2 = make_float2(inv, inv);
  uint32_t c[8];
#pragma unroll
  for (int i = 0; i < 8; i++) c[i] = e4m3x2(__fmul2_rn(bf16x2_to_float2(w[i]), inv2));
  out = make_uint4(c[0] | c[1] << 16, c[2] | c[3] << 16, c[4] | c[5] << 16, c[6] | c[7] << 16);
  return uint8_t(e + 127);
}

// Address of the scale of (row r, scale block kb): 128 x 4 tiles of 512 bytes
// (src/kernels/blockscale.cu:83 and :127).
__device__ __forceinline__ int64_t sf_row_offset(uint64_t r, int nkb_pad) {
  return int64_t(r >> 7) * (int64_t(nkb_pad) * 128) + int64_t((r & 31) * 16 + ((r >> 5) & 3) * 4);
}
__device__ __forceinline__ int sf_col_offset(int kb) { return (kb >> 2) * 512 + (kb & 3); }

}  // namespace mxk
