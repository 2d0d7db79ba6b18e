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
    "res_threads",  "ew_threads",       "ew_unroll",    "act_rows_per_cta",
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

int mxk_set_tuning(const char* name, int value) {
  for (int i = 0; i < mxk::TUNE_COUNT; i++)
    if (!strcmp(name, mxk::kTuneNames[i])) {
      mxk::g_tune[i].store(value, std::memory_order_relaxed);
      return MXK_OK;
    }
  return mxk::fail(MXK_ERR_INVALID_ARG, "mxk_set_tuning: unknown knob '%s'", name);
}

}  // extern "C"
