// Library-wide host plumbing: status strings, launch accounting, device attributes, tuning knobs.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "tuning.h"

namespace mxk {

namespace {
thread_local char g_err[512] = "";
thread_local int64_t g_launches = 0;
constexpr int kMaxDevices = 64;
std::atomic<int> g_sms[kMaxDevices];  // 0 = not yet queried
std::atomic<int> g_tune[TUNE_COUNT];  // 0 = use the built-in default
const char* const kTuneNames[TUNE_COUNT] = {
    "norm_threads", "norm_ctas_per_sm", "rope_threads", "rope_ctas_per_sm", "res_rows_per_cta",
    "res_threads",  "ew_threads",       "ew_unroll",    "act_rows_per_cta", "norm_path",
    "norm_stages",  "rope_path",        "rope_stages",  "ew_ctas_per_sm",   "res_path",     "rope_tokens",
    "stream_warps", "stream_stages",    "stream_ctas_per_sm", "stream_chunk_kb", "act_path",
    "pdl",          "norm_interleave", "pipe_interleave", "quant_rows_per_cta", "quant_path", "rope_unroll", "rope_wide", "rope_wide_regs", "linear_ctas", "linear_group_m",
};
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int after_launch(const char* what) {
  g_launches++;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "%s: CUDA launch failed: %s", what, cudaGetErrorString(e));
  return MXK_OK;
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = g_sms[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  g_sms[dev].store(n, std::memory_order_relaxed);
  return n;
}

__device__ int g_device_error = 0;

namespace {
std::atomic<int*> g_err_word[kMaxDevices];
}  // namespace

int* device_error_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  int* p = g_err_word[dev].load(std::memory_order_acquire);
  if (p) return p;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_device_error) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  g_err_word[dev].store(p, std::memory_order_release);
  return p;
}

namespace {
struct OccEntry {
  std::atomic<const void*> fn{nullptr};
  std::atomic<int> threads{0}, smem{0}, value{0};
};
OccEntry g_occ[256];
}  // namespace

int resident_ctas_lookup(const void* kernel, int threads, size_t smem) {
  // Open-addressed cache; an entry is published by writing `value` last, so a reader that sees
  // value > 0 with matching keys can use it, and a lost race only repeats the (pure) query.
  unsigned h = unsigned((reinterpret_cast<uintptr_t>(kernel) >> 4) * 2654435761u + threads * 40503u + unsigned(smem)) & 255u;
  for (int probe = 0; probe < 256; probe++) {
    OccEntry& e = g_occ[(h + probe) & 255u];
    const void* f = e.fn.load(std::memory_order_acquire);
    if (f == kernel && e.threads.load(std::memory_order_relaxed) == threads &&
        e.smem.load(std::memory_order_relaxed) == int(smem)) {
      int v = e.value.load(std::memory_order_acquire);
      if (v > 0) return v;
    }
    if (f == nullptr) {
      int n = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem) != cudaSuccess || n < 1) {
        cudaGetLastError();
        return 1;
      }
      const void* expect = nullptr;
      if (e.fn.compare_exchange_strong(expect, kernel, std::memory_order_acq_rel)) {
        e.threads.store(threads, std::memory_order_relaxed);
        e.smem.store(int(smem), std::memory_order_relaxed);
        e.value.store(n, std::memory_order_release);
      }
      return n;
    }
  }
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem) != cudaSuccess || n < 1) return 1;
  return n;
}

bool pdl_enabled() { return g_tune[TUNE_PDL].load(std::memory_order_relaxed) != 2; }

int tune(int key, int dflt) {
  int v = g_tune[key].load(std::memory_order_relaxed);
  return v > 0 ? v : dflt;
}

}  // namespace mxk

extern "C" {

const char* mxk_last_error(void) { return mxk::g_err; }
int mxk_version(void) { return 100; }
int64_t mxk_launch_count(void) { return mxk::g_launches; }
void mxk_reset_launch_count(void) { mxk::g_launches = 0; }

int mxk_device_error(int* out_host, int clear) {
  if (!out_host) return mxk::fail(MXK_ERR_INVALID_ARG, "device_error: null out");
  int* p = mxk::device_error_word();
  if (!p) return mxk::fail(MXK_ERR_CUDA, "device_error: no error word on this device");
  cudaError_t e = cudaMemcpy(out_host, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && clear && *out_host != 0) e = cudaMemset(p, 0, sizeof(int));
  if (e != cudaSuccess) return mxk::fail(MXK_ERR_CUDA, "device_error: %s", cudaGetErrorString(e));
  return MXK_OK;
}

int mxk_set_tuning(const char* name, int value) {
  for (int i = 0; i < mxk::TUNE_COUNT; i++)
    if (!strcmp(name, mxk::kTuneNames[i])) {
      mxk::g_tune[i].store(value, std::memory_order_relaxed);
      return MXK_OK;
    }
  return mxk::fail(MXK_ERR_INVALID_ARG, "mxk_set_tuning: unknown knob '%s'", name);
}

}  // extern "C"
