// Shared device/host helpers for the libmxk kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mxk.h"

namespace mxk {

using bf16 = __nv_bfloat16;

// ---- status / error reporting (host) -------------------------------------------------------

// Records a formatted message for mxk_last_error() on this thread and returns `code`.
int fail(int code, const char* fmt, ...);
// Checks cudaGetLastError() after a launch (no synchronisation, like the reference's MX_KCHECK,
// src/core/common.h:48) and counts the launch.
int after_launch(const char* what);
// Number of SMs of the current device (cached per device ordinal).
int sm_count();

// Address, on the current device, of the int the kernels' bounded waits report to (0 = no error).
int* device_error_word();

// CTAs of `kernel` that one SM holds at this CTA size (occupancy API, cached per kernel/size).
// Grids of the persistent kernels are sized to exactly one resident wave with it.
int resident_ctas_lookup(const void* kernel, int threads, size_t smem);
template <class K>
inline int resident_ctas(K kernel, int threads, size_t smem = 0) {
  return resident_ctas_lookup(reinterpret_cast<const void*>(kernel), threads, smem);
}

// Programmatic dependent launch: a kernel launched through launch_pdl() may be scheduled while the
// previous kernel of the stream is still draining; its threads park at pdl_wait() until that kernel
// has completed and its writes are visible, so only work that touches no global memory (barrier
// set-up, index arithmetic) may precede pdl_wait().  Every kernel launched this way calls
// pdl_launch_dependents() at its top so that its own successor can be scheduled early too.  This
// hides the launch latency and CTA ramp between the back-to-back kernels of a block (a few
// microseconds each, which is 10-25 % of these kernels at the smaller shapes).
bool pdl_enabled();
template <class... KArgs, class... Args>
inline void launch_pdl(void (*k)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, k, KArgs(args)...);  // errors surface through cudaGetLastError() in after_launch()
}

inline cudaStream_t as_stream(mxk_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

template <class T>
inline bool aligned(const T* p, size_t bytes) {
  return (reinterpret_cast<uintptr_t>(p) & (bytes - 1)) == 0;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- device helpers -----------------------------------------------------------------------

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the 2^k-lane group the lane belongs to (WIDTH lanes, WIDTH a power of two <= 32).
template <int WIDTH>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = WIDTH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ const float* pick(const MxkRowMod& m, int64_t row) {
  return row < m.prefix_len ? m.prefix : m.target;
}

// 128-bit global accesses.  `ld_stream` / `st_stream` mark data that is touched once
// (activations); modulation vectors and tables go through the default cached path.
__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ uint2 ld_stream(const uint2* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(uint2* p, uint2 v) { __stcs(p, v); }

// bf16 pair <-> fp32.  A bf16 is the high half of an fp32, so unpacking is a shift / mask.
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
// Round-to-nearest-even pack, the same rounding as __float2bfloat16.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_to_f(bf16 v) { return __bfloat162float(v); }

// Single-instruction special functions (MUFU), flush-to-zero: 2^x and 1/x to about 2 ulp.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16_lo(v.x), f[1] = bf16_hi(v.x);
  f[2] = bf16_lo(v.y), f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z), f[5] = bf16_hi(v.z);
  f[6] = bf16_lo(v.w), f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]),
                    pack_bf16(f[6], f[7]));
}
__device__ __forceinline__ void unpack4(const uint2& v, float (&f)[4]) {
  f[0] = bf16_lo(v.x), f[1] = bf16_hi(v.x);
  f[2] = bf16_lo(v.y), f[3] = bf16_hi(v.y);
}
__device__ __forceinline__ uint2 pack4(const float (&f)[4]) {
  return make_uint2(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]));
}

}  // namespace mxk
