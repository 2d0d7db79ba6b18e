// gated_residual (reference: src/kernels/ops.cu:73-84 kernel, 177-189 launcher) and the fused
// gated_residual + norm launcher.
//
// x[r, c] += act(gate[c]) * y[r, c].  Each thread owns CPT consecutive columns for a strip of
// rows, so act(gate) - a tanhf in the Qwen blocks - is evaluated once per column per CTA instead
// of once per element, and every row is one 128-bit y load plus 128-bit x loads and stores.
#include "common.cuh"
#include "norm_dispatch.cuh"
#include "tuning.h"

namespace mxk {
namespace {

constexpr int kResRowsInFlight = 4;

template <int CPT>
struct ResVec;
template <>
struct ResVec<8> {
  using ytype = uint4;
};
template <>
struct ResVec<4> {
  using ytype = uint2;
};

template <int CPT>
__device__ __forceinline__ void res_rows(float* __restrict__ x, const bf16* __restrict__ y,
                                         int64_t r0, int64_t r1, int dim, int col,
                                         const float (&g)[CPT]) {
  using yt = typename ResVec<CPT>::ytype;
  constexpr int U = kResRowsInFlight;
  for (int64_t r = r0; r < r1; r += U) {
    float4 xv[U][CPT / 4];
    yt yv[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      if (r + u < r1) {
        const int64_t off = (r + u) * dim + col;
        yv[u] = ld_stream(reinterpret_cast<const yt*>(y + off));
#pragma unroll
        for (int q = 0; q < CPT / 4; q++) xv[u][q] = ld_stream(reinterpret_cast<const float4*>(x + off) + q);
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      if (r + u < r1) {
        float f[CPT];
        if constexpr (CPT == 8) unpack8(yv[u], f);
        else unpack4(yv[u], f);
        const int64_t off = (r + u) * dim + col;
#pragma unroll
        for (int q = 0; q < CPT / 4; q++) {
          float4 v = xv[u][q];
          v.x = fmaf(f[4 * q + 0], g[4 * q + 0], v.x);
          v.y = fmaf(f[4 * q + 1], g[4 * q + 1], v.y);
          v.z = fmaf(f[4 * q + 2], g[4 * q + 2], v.z);
          v.w = fmaf(f[4 * q + 3], g[4 * q + 3], v.w);
          st_stream(reinterpret_cast<float4*>(x + off) + q, v);
        }
      }
    }
  }
}

template <int CPT>
__device__ __forceinline__ void load_gate(const float* gp, int col, int gate_tanh, float (&g)[CPT]) {
#pragma unroll
  for (int q = 0; q < CPT / 4; q++) {
    float4 v = gp ? *reinterpret_cast<const float4*>(gp + col + 4 * q) : make_float4(1.f, 1.f, 1.f, 1.f);
    if (gp && gate_tanh) v = make_float4(tanhf(v.x), tanhf(v.y), tanhf(v.z), tanhf(v.w));
    g[4 * q] = v.x, g[4 * q + 1] = v.y, g[4 * q + 2] = v.z, g[4 * q + 3] = v.w;
  }
}

template <int CPT>
__global__ void __launch_bounds__(256)
    gated_residual_kernel(float* __restrict__ x, const bf16* __restrict__ y, int64_t rows, int dim,
                          MxkRowMod gate, int gate_tanh, int rows_per_chunk) {
  pdl_launch_dependents();
  pdl_wait();
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * CPT;
  if (col >= dim) return;
  const int64_t plen = gate.target ? gate.prefix_len : 0;
  float g[CPT];
  int have = -1;  // which gate vector g holds: 1 prefix, 0 target
  const int64_t nchunks = (rows + rows_per_chunk - 1) / rows_per_chunk;
  for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const int64_t r0 = c * rows_per_chunk;
    const int64_t r1 = r0 + rows_per_chunk < rows ? r0 + rows_per_chunk : rows;
    const int64_t mid = plen < r0 ? r0 : plen > r1 ? r1 : plen;  // rows [r0, mid) use the prefix vector
    if (mid > r0) {
      if (have != 1) load_gate<CPT>(gate.prefix, col, gate_tanh, g), have = 1;
      res_rows<CPT>(x, y, r0, mid, dim, col, g);
    }
    if (r1 > mid) {
      if (have != 0) load_gate<CPT>(gate.target, col, gate_tanh, g), have = 0;
      res_rows<CPT>(x, y, mid, r1, dim, col, g);
    }
  }
}

// Any dim and alignment; one element per thread, 2-D indexing (no 64-bit division).
__global__ void __launch_bounds__(256)
    gated_residual_scalar_kernel(float* __restrict__ x, const bf16* __restrict__ y, int64_t rows,
                                 int dim, MxkRowMod gate, int gate_tanh) {
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= dim) return;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float g = 1.f;
    if (gate.target) {
      const float gv = pick(gate, row)[i];
      g = gate_tanh ? tanhf(gv) : gv;
    }
    x[row * dim + i] = fmaf(bf16_to_f(y[row * dim + i]), g, x[row * dim + i]);
  }
}

}  // namespace
}  // namespace mxk

using namespace mxk;

extern "C" {

int mxk_gated_residual(float* x, const mxk_bf16* y, int64_t rows, int64_t dim, MxkRowMod gate,
                       int gate_tanh, mxk_stream_t stream) {
  if (rows <= 0) return MXK_OK;
  if (!x || !y) return fail(MXK_ERR_INVALID_ARG, "gated_residual: null x or y");
  if (dim <= 0 || dim > (int64_t(1) << 30)) return fail(MXK_ERR_INVALID_ARG, "gated_residual: dim=%lld", (long long)dim);
  if (gate.target && !gate.prefix && gate.prefix_len > 0)
    return fail(MXK_ERR_INVALID_ARG, "gated_residual: prefix_len > 0 with a null prefix vector");
  cudaStream_t s = as_stream(stream);
  const bf16* yb = reinterpret_cast<const bf16*>(y);
  const bool gate_ok = (!gate.target || aligned(gate.target, 16)) && (!gate.prefix || aligned(gate.prefix, 16));
  const int threads = tune(TUNE_RES_THREADS, 128);
  const int rpc = tune(TUNE_RES_ROWS_PER_CTA, 8);
  const int64_t nchunks = ceil_div(rows, rpc);
  // Preferred: the bulk-copy pipelined row kernel in its residual-only mode.
  if (tune(TUNE_RES_PATH, 1) == 1 && dim % 8 == 0 && dim <= 8192 && rows >= 2 && aligned(x, 16) && aligned(y, 16) && gate_ok) {
    NormArgs a{};
    a.x = x, a.xw = x, a.y = yb, a.gate = gate, a.gate_tanh = gate_tanh;
    a.rows = rows, a.dim = int(dim), a.nvec = int(dim / 4);
    NormPlan p;
    if (plan_norm(a.nvec, rows, p, 256)) {  // the residual-only mode measured best with 256-thread CTAs
      launch_norm<2, float, false, true>(p, a, true, s);
      return after_launch("gated_residual");
    }
  }
  // grid.y covers the columns, grid.x walks row chunks; together exactly one resident wave
  auto wave_x = [&](auto kern, unsigned gy) {
    int64_t gx = ceil_div(int64_t(sm_count()) * resident_ctas(kern, threads), gy);
    return unsigned(gx > nchunks ? nchunks : gx < 1 ? 1 : gx);
  };
  if (dim % 8 == 0 && aligned(x, 16) && aligned(y, 16) && gate_ok) {
    const unsigned gy = unsigned(ceil_div(dim / 8, threads));
    launch_pdl(gated_residual_kernel<8>, dim3(wave_x(gated_residual_kernel<8>, gy), gy), dim3(threads), 0, s, x, yb, rows, int(dim), gate, gate_tanh, rpc);
  } else if (dim % 4 == 0 && aligned(x, 16) && aligned(y, 8) && gate_ok) {
    const unsigned gy = unsigned(ceil_div(dim / 4, threads));
    launch_pdl(gated_residual_kernel<4>, dim3(wave_x(gated_residual_kernel<4>, gy), gy), dim3(threads), 0, s, x, yb, rows, int(dim), gate, gate_tanh, rpc);
  } else {
    const unsigned gy = unsigned(ceil_div(dim, 256));
    int64_t gx = rows < int64_t(sm_count()) * 16 ? rows : int64_t(sm_count()) * 16;
    gated_residual_scalar_kernel<<<dim3(unsigned(gx), gy), 256, 0, s>>>(x, yb, rows, int(dim), gate, gate_tanh);
  }
  return after_launch("gated_residual");
}

int mxk_gated_residual_bias(float* x, const mxk_bf16* y, const float* bias, int64_t rows, int64_t dim, MxkRowMod gate,
                            int gate_tanh, mxk_stream_t stream) {
  if (!bias) return mxk_gated_residual(x, y, rows, dim, gate, gate_tanh, stream);
  if (rows <= 0) return MXK_OK;
  if (!x || !y) return fail(MXK_ERR_INVALID_ARG, "gated_residual_bias: null x or y");
  if (gate.target && !gate.prefix && gate.prefix_len > 0)
    return fail(MXK_ERR_INVALID_ARG, "gated_residual_bias: prefix_len > 0 with a null prefix vector");
  const bool gate_ok = (!gate.target || aligned(gate.target, 16)) && (!gate.prefix || aligned(gate.prefix, 16));
  NormArgs a{};
  a.x = x, a.xw = x, a.y = reinterpret_cast<const bf16*>(y), a.ybias = bias, a.gate = gate, a.gate_tanh = gate_tanh;
  a.rows = rows, a.dim = int(dim), a.nvec = int(dim / 4);
  NormPlan p;
  if (dim <= 0 || dim % 8 != 0 || dim > 8192 || !aligned(x, 16) || !aligned(y, 16) || !aligned(bias, 16) || !gate_ok ||
      !plan_norm(a.nvec, rows, p, 256))
    return fail(MXK_ERR_INVALID_ARG, "gated_residual_bias: dim %lld or an unaligned vector is outside the one-pass kernel; "
                "call mxk_add_bias_bf16 and mxk_gated_residual", (long long)dim);
  launch_norm<2, float, false, true, false, true>(p, a, true, as_stream(stream));
  return after_launch("gated_residual_bias");
}

static int gated_residual_norm_impl(const char* name, float* x, const mxk_bf16* y, int64_t rows, int64_t dim, MxkRowMod gate,
                                    int gate_tanh, int norm_mode, float eps, const float* w, MxkRowMod scale, MxkRowMod shift,
                                    mxk_bf16* out, float* amax_out, mxk_stream_t stream);

int mxk_gated_residual_norm(float* x, const mxk_bf16* y, int64_t rows, int64_t dim, MxkRowMod gate,
                            int gate_tanh, int norm_mode, float eps, const float* w,
                            MxkRowMod scale, MxkRowMod shift, mxk_bf16* out, mxk_stream_t stream) {
  return gated_residual_norm_impl("gated_residual_norm", x, y, rows, dim, gate, gate_tanh, norm_mode, eps, w, scale, shift, out,
                                  nullptr, stream);
}

int mxk_gated_residual_norm_amax(float* x, const mxk_bf16* y, int64_t rows, int64_t dim, MxkRowMod gate, int gate_tanh,
                                 int norm_mode, float eps, const float* w, MxkRowMod scale, MxkRowMod shift, mxk_bf16* out,
                                 float* amax_out, mxk_stream_t stream) {
  if (!amax_out) return fail(MXK_ERR_INVALID_ARG, "gated_residual_norm_amax: null amax_out");
  cudaError_t e = cudaMemsetAsync(amax_out, 0, sizeof(float), as_stream(stream));
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "gated_residual_norm_amax: cudaMemsetAsync: %s", cudaGetErrorString(e));
  return gated_residual_norm_impl("gated_residual_norm_amax", x, y, rows, dim, gate, gate_tanh, norm_mode, eps, w, scale, shift,
                                  out, amax_out, stream);
}

static int gated_residual_norm_impl(const char* name, float* x, const mxk_bf16* y, int64_t rows, int64_t dim, MxkRowMod gate,
                                    int gate_tanh, int norm_mode, float eps, const float* w, MxkRowMod scale, MxkRowMod shift,
                                    mxk_bf16* out, float* amax_out, mxk_stream_t stream) {
  if (rows <= 0) return MXK_OK;
  if (norm_mode != 0 && norm_mode != 1)
    return fail(MXK_ERR_INVALID_ARG, "%s: norm_mode=%d (0 LayerNorm, 1 RMSNorm)", name, norm_mode);
  if (!y) return fail(MXK_ERR_INVALID_ARG, "%s: null y", name);
  if (int rc = check_norm_common(name, x, rows, dim, out, scale, shift)) return rc;
  if (gate.target && !gate.prefix && gate.prefix_len > 0)
    return fail(MXK_ERR_INVALID_ARG, "%s: prefix_len > 0 with a null prefix vector", name);
  NormArgs a{};
  a.x = x, a.xw = x, a.y = reinterpret_cast<const bf16*>(y);
  a.gate = gate, a.gate_tanh = gate_tanh;
  a.rows = rows, a.dim = int(dim), a.nvec = int(dim / 4), a.eps = eps;
  a.w = norm_mode == 1 ? w : nullptr;
  a.scale = scale, a.shift = shift, a.out = reinterpret_cast<bf16*>(out), a.amax = amax_out;
  if (norm_mode == 0) return run_norm<0, float, true>(name, a, as_stream(stream));
  return run_norm<1, float, true>(name, a, as_stream(stream));
}

}  // extern "C"
