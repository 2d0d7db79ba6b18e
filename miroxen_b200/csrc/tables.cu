// RoPE cos/sin tables, the Qwen-Image timestep embedding and the MiniMax-H3 time basis.
//
// The reference evaluates cosf/sinf/powf/expf of libm on the host for every table entry and
// uploads the result (src/models/qwen_image/dit.cpp:151-185, 219-230;
// src/models/minimax_h3/dit.cpp:166-179, 254-262).  A table entry depends only on
// (position on one axis, frequency), and a sequence has few distinct positions per axis, so the
// host evaluates libm once per distinct (position, frequency) into a small per-axis look-up
// table and a kernel expands it to the [S, rot/2] table.  The values are libm's, bit for bit.
#include <cmath>
#include <vector>

#include "bulk_copy.cuh"
#include "common.cuh"

namespace mxk {
namespace {

constexpr int kMaxAxes = 3;
constexpr int kMaxHalf = 128;  // rot <= D <= 256
constexpr int kRunsPerLaunch = 16;

struct ExpandArgs {
  const float* lut_cos;
  const float* lut_sin;
  int64_t lut_off[kMaxAxes];
  int32_t pairs[kMaxAxes];
  int32_t col0[kMaxAxes];
  uint8_t axis_of[kMaxHalf];
  MxkRopeRun runs[kRunsPerLaunch];
  int n_runs;
  int half;
  float* cos;
  float* sin;
};

// One thread per table entry of one run: blockIdx.y = run, x covers rows * half.
__global__ void __launch_bounds__(256) rope_expand_kernel(const ExpandArgs a) {
  const MxkRopeRun& run = a.runs[blockIdx.y];
  const int64_t rows = int64_t(run.n0) * run.n1 * run.n2;
  const int64_t total = rows * a.half;
  for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += int64_t(gridDim.x) * blockDim.x) {
    const int64_t r = e / a.half;
    const int p = int(e - r * a.half);
    const int64_t i01 = r / run.n2;
    const int i2 = int(r - i01 * run.n2);
    const int i0 = int(i01 / run.n1);
    const int i1 = int(i01 - int64_t(i0) * run.n1);
    const int ax = a.axis_of[p];
    const int64_t idx = run.base[ax] + int64_t(i0) * run.step0[ax] + int64_t(i1) * run.step1[ax] +
                        int64_t(i2) * run.step2[ax];
    const int64_t src = a.lut_off[ax] + idx * a.pairs[ax] + (p - a.col0[ax]);
    const int64_t dst = (run.row0 + r) * a.half + p;
    a.cos[dst] = a.lut_cos[src];
    a.sin[dst] = a.lut_sin[src];
  }
}

struct TimestepArgs {
  float freq[128];
  float ts[2];
  float* out;
};

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16(v)); }

__global__ void timestep_embedding_kernel(const TimestepArgs a) {
  const int r = blockIdx.x, i = threadIdx.x;  // 2 x 128
  const float arg = __fmul_rn(a.ts[r], a.freq[i]);
  a.out[r * 256 + i] = round_bf16(float(cos(double(arg))));
  a.out[r * 256 + 128 + i] = round_bf16(float(sin(double(arg))));
}

__global__ void __launch_bounds__(256)
    h3_time_basis_kernel(const float* __restrict__ ts, int64_t nt, const float* __restrict__ table,
                         int64_t grid, int64_t basis, float* __restrict__ out) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= nt * basis) return;
  const int64_t i = e / basis, j = e - i * basis;
  const float t = fminf(fmaxf(ts[i], 0.f), 1.f);
  const float pos = __fmul_rn(t, float(grid - 1));
  int64_t lo = int64_t(floorf(pos));
  if (lo > grid - 2) lo = grid - 2;
  const float fr = __fsub_rn(pos, float(lo));
  const float a = table[lo * basis + j], b = table[(lo + 1) * basis + j];
  out[e] = __fadd_rn(a, __fmul_rn(__fsub_rn(b, a), fr));
}

// Self-test of the bounded wait: waits on an mbarrier that nothing ever completes, with a small try
// budget, and reports the give-up the same way the pipelined kernels do (error word = 1).
__global__ void bounded_wait_selftest_kernel(int tries, int* err) {
  __shared__ __align__(8) unsigned long long bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  bool done = false;
  for (int i = 0; i < tries && !done; i++) done = mbar_try(smem_u32(&bar), 0);
  if (!__syncthreads_and(done) && threadIdx.x == 0 && err) atomicExch(err, kErrBulkTimeout);
}

const float* timestep_freqs() {
  // f[i] = expf(-logf(10000) * i / 128)  (src/models/qwen_image/dit.cpp:226)
  static const std::vector<float> f = [] {
    std::vector<float> v(128);
    for (int i = 0; i < 128; i++) v[i] = std::exp(-std::log(10000.f) * float(i) / float(128));
    return v;
  }();
  return f.data();
}

float host_round_bf16(float v) { return __bfloat162float(__float2bfloat16(v)); }

}  // namespace
}  // namespace mxk

using namespace mxk;

extern "C" {

int mxk_rope_table_expand(const float* lut_cos, const float* lut_sin, const int64_t* lut_off_host,
                          const int32_t* pairs_host, const int32_t* col0_host, int n_axes,
                          const MxkRopeRun* runs_host, int n_runs, int64_t S, int half, float* cos,
                          float* sin, mxk_stream_t stream) {
  if (S <= 0 || n_runs <= 0 || half <= 0) return MXK_OK;
  if (!lut_cos || !lut_sin || !lut_off_host || !pairs_host || !col0_host || !runs_host || !cos || !sin)
    return fail(MXK_ERR_INVALID_ARG, "rope_table_expand: null argument");
  if (n_axes < 1 || n_axes > kMaxAxes) return fail(MXK_ERR_INVALID_ARG, "rope_table_expand: n_axes=%d (1..3)", n_axes);
  if (half > kMaxHalf) return fail(MXK_ERR_TOO_LARGE, "rope_table_expand: half=%d > %d", half, kMaxHalf);
  ExpandArgs a{};
  a.lut_cos = lut_cos, a.lut_sin = lut_sin, a.half = half, a.cos = cos, a.sin = sin;
  std::vector<int> owner(half, -1);
  for (int ax = 0; ax < n_axes; ax++) {
    a.lut_off[ax] = lut_off_host[ax], a.pairs[ax] = pairs_host[ax], a.col0[ax] = col0_host[ax];
    if (pairs_host[ax] < 0 || col0_host[ax] < 0 || col0_host[ax] + pairs_host[ax] > half)
      return fail(MXK_ERR_INVALID_ARG, "rope_table_expand: axis %d columns [%d, %d) outside [0, %d)", ax,
                  col0_host[ax], col0_host[ax] + pairs_host[ax], half);
    for (int p = col0_host[ax]; p < col0_host[ax] + pairs_host[ax]; p++) owner[p] = ax;
  }
  for (int p = 0; p < half; p++) {
    if (owner[p] < 0) return fail(MXK_ERR_INVALID_ARG, "rope_table_expand: pair column %d belongs to no axis", p);
    a.axis_of[p] = uint8_t(owner[p]);
  }
  for (int i = 0; i < n_runs; i++) {
    const MxkRopeRun& r = runs_host[i];
    if (r.n0 <= 0 || r.n1 <= 0 || r.n2 <= 0 || r.row0 < 0 || r.row0 + int64_t(r.n0) * r.n1 * r.n2 > S)
      return fail(MXK_ERR_INVALID_ARG, "rope_table_expand: run %d lies outside [0, %lld)", i, (long long)S);
  }
  for (int i0 = 0; i0 < n_runs; i0 += kRunsPerLaunch) {
    const int n = n_runs - i0 < kRunsPerLaunch ? n_runs - i0 : kRunsPerLaunch;
    int64_t most = 0;
    for (int i = 0; i < n; i++) {
      a.runs[i] = runs_host[i0 + i];
      const int64_t e = int64_t(a.runs[i].n0) * a.runs[i].n1 * a.runs[i].n2 * half;
      if (e > most) most = e;
    }
    a.n_runs = n;
    int64_t gx = ceil_div(most, 256);
    const int64_t cap = int64_t(sm_count()) * 8;
    if (gx > cap) gx = cap;
    rope_expand_kernel<<<dim3(unsigned(gx), unsigned(n)), 256, 0, as_stream(stream)>>>(a);
    if (int rc = after_launch("rope_table_expand")) return rc;
  }
  return MXK_OK;
}

int mxk_msrope_inv_freq_host(const int32_t* axes_host, int n_axes, float theta, float* out_host) {
  if (!axes_host || !out_host || n_axes <= 0) return fail(MXK_ERR_INVALID_ARG, "msrope_inv_freq_host: null argument");
  int k = 0;
  for (int a = 0; a < n_axes; a++)
    for (int j = 0; j < axes_host[a] / 2; j++)
      out_host[k++] = 1.0f / std::pow(theta, float(2 * j) / float(axes_host[a]));
  return MXK_OK;
}

int mxk_rope_lut_int_host(int64_t pos_min, int64_t pos_max, const float* invf_host, int pairs,
                          float* lut_cos_host, float* lut_sin_host) {
  if (!invf_host || !lut_cos_host || !lut_sin_host || pairs <= 0 || pos_max < pos_min)
    return fail(MXK_ERR_INVALID_ARG, "rope_lut_int_host: bad argument");
  for (int64_t p = pos_min; p <= pos_max; p++)
    for (int j = 0; j < pairs; j++) {
      const float ang = float(p) * invf_host[j];
      lut_cos_host[(p - pos_min) * pairs + j] = std::cos(ang);
      lut_sin_host[(p - pos_min) * pairs + j] = std::sin(ang);
    }
  return MXK_OK;
}

int mxk_rope_lut_f32_host(const float* pos_host, int64_t n, const float* invf_host, int pairs,
                          float* lut_cos_host, float* lut_sin_host) {
  if (!pos_host || !invf_host || !lut_cos_host || !lut_sin_host || pairs <= 0 || n < 0)
    return fail(MXK_ERR_INVALID_ARG, "rope_lut_f32_host: bad argument");
  for (int64_t i = 0; i < n; i++)
    for (int j = 0; j < pairs; j++) {
      const float ang = pos_host[i] * invf_host[j];
      lut_cos_host[i * pairs + j] = std::cos(ang);
      lut_sin_host[i * pairs + j] = std::sin(ang);
    }
  return MXK_OK;
}

int mxk_h3_spatial_grid_host(int64_t dim, int64_t H, int64_t W, float* out_host) {
  if (!out_host || dim <= 0 || dim % 2 || H <= 0 || W <= 0)
    return fail(MXK_ERR_INVALID_ARG, "h3_spatial_grid_host: dim=%lld H=%lld W=%lld", (long long)dim, (long long)H, (long long)W);
  const double sa = std::sqrt(double(H * W));
  const double ratio = double(dim) / sa, left = (1.0 - ratio) / 2.0;
  const int64_t n = dim / 2;
  for (int64_t k = 0; k < n; k++) out_host[k] = float((left + ratio * double(k) / double(n)) * 32.0);
  return MXK_OK;
}

int mxk_h3_frame_times_host(int64_t T, int64_t F_lat, float* out_host) {
  if (!out_host || F_lat < 0) return fail(MXK_ERR_INVALID_ARG, "h3_frame_times_host: bad argument");
  static const int per_latent[5] = {1, 4, 4, 4, 4};
  double acc = double(T);
  for (int64_t f = 0; f < F_lat; f++) {
    out_host[f] = float(acc);
    acc += (5.0 / 3.0) * per_latent[f % 5];
  }
  return MXK_OK;
}

int mxk_qwen_timestep_embedding_host(float t, float* out_host) {
  if (!out_host) return fail(MXK_ERR_INVALID_ARG, "qwen_timestep_embedding_host: null out");
  const float* f = timestep_freqs();
  const float ts[2] = {host_round_bf16(t) * 1000.f, 0.f};
  for (int r = 0; r < 2; r++)
    for (int i = 0; i < 128; i++) {
      const float arg = ts[r] * f[i];
      out_host[r * 256 + i] = host_round_bf16(std::cos(arg));
      out_host[r * 256 + 128 + i] = host_round_bf16(std::sin(arg));
    }
  return MXK_OK;
}

int mxk_qwen_timestep_embedding(float t, float* out, mxk_stream_t stream) {
  if (!out) return fail(MXK_ERR_INVALID_ARG, "qwen_timestep_embedding: null out");
  TimestepArgs a;
  const float* f = timestep_freqs();
  for (int i = 0; i < 128; i++) a.freq[i] = f[i];
  a.ts[0] = host_round_bf16(t) * 1000.f, a.ts[1] = 0.f;
  a.out = out;
  timestep_embedding_kernel<<<2, 128, 0, as_stream(stream)>>>(a);
  return after_launch("qwen_timestep_embedding");
}

int mxk_selftest_bounded_wait(mxk_stream_t stream) {
  bounded_wait_selftest_kernel<<<1, 64, 0, as_stream(stream)>>>(4, device_error_word());
  return after_launch("selftest_bounded_wait");
}

int mxk_h3_time_basis(const float* ts, int64_t nt, const float* table, int64_t grid, int64_t basis,
                      float* out, mxk_stream_t stream) {
  if (nt <= 0 || basis <= 0) return MXK_OK;
  if (!ts || !table || !out) return fail(MXK_ERR_INVALID_ARG, "h3_time_basis: null argument");
  if (grid < 2) return fail(MXK_ERR_INVALID_ARG, "h3_time_basis: grid=%lld < 2", (long long)grid);
  h3_time_basis_kernel<<<unsigned(ceil_div(nt * basis, 256)), 256, 0, as_stream(stream)>>>(ts, nt, table, grid, basis, out);
  return after_launch("h3_time_basis");
}

}  // extern "C"
