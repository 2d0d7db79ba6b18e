// mbarrier + 1-D bulk-copy (TMA) helpers for the pipelined row kernels (sm_100a PTX).
//
// Every wait is bounded: a kernel that runs out of polls records kErrBulkTimeout in
// the device's error word (device_error_word(), readable through mxk_device_error()), drains
// its own copies and returns;
// nothing here can spin forever.
#pragma once

#include "common.cuh"

namespace mxk {

constexpr int kErrBulkTimeout = 1;
// A wait is a bounded number of mbarrier.try_wait calls.  try_wait parks the thread in hardware
// until the phase completes or its time hint expires, so a waiting warp costs no issue slots
// (polling test_wait from every thread was measured to more than double the instruction count of
// the row kernels).  kWaitTries x kWaitHintNs bounds the whole wait to roughly a second.
constexpr unsigned kWaitTries = 1u << 16;
constexpr unsigned kWaitHintNs = 20000;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return unsigned(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kWaitHintNs)
      : "memory");
  return ok != 0;
}
// Bounded wait; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
  if (mbar_try(bar, parity)) return true;
  // try_wait may come back early; sleep between tries so that a waiting warp leaves the issue
  // slots to the warps that have data (these kernels are short of issue slots, not of warps).
  unsigned ns = 32;
  for (unsigned i = 1; i < kWaitTries; i++) {
    __nanosleep(ns);
    if (ns < 256) ns <<= 1;
    if (mbar_try(bar, parity)) return true;
  }
  return false;
}
// 1-D bulk copy global -> this CTA's shared memory; src, dst and bytes are multiples of 16.
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// CTA sum whose barrier also carries a vote: returns the sum, and `all_ok` becomes false for every
// thread if any thread passed ok == false.
__device__ __forceinline__ float cta_sum_vote(float v, float* red, int nwarps, bool ok, bool& all_ok) {
  v = warp_sum(v);
  if (nwarps == 1) {
    all_ok = __all_sync(0xffffffffu, ok);
    return v;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  all_ok = __syncthreads_and(ok) != 0;
  float t = red[0];
  for (int i = 1; i < nwarps; i++) t += red[i];
  return t;
}


}  // namespace mxk
