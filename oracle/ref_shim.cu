// TEST INFRASTRUCTURE ONLY.  extern "C" doorway to the REFERENCE's own launchers
// (namespace mx, src/kernels/ops.h), so that tests and the benchmark can run the reference's
// kernels - src/kernels/ops.cu compiled unmodified for sm_100a next to this file - on the same
// device buffers as libmxk.  Built only where the reference tree is present (oracle/Makefile,
// target _ref); the product never loads it.
#include <cstring>
#include <stdexcept>

#include "kernels/ops.h"

namespace {
thread_local char g_err[512] = "";
template <class F>
int guard(F f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    strncpy(g_err, e.what(), sizeof(g_err) - 1);
    return -1;
  }
}
cudaStream_t st(void* s) { return reinterpret_cast<cudaStream_t>(s); }
using mx::bf16;
}  // namespace

extern "C" {

const char* ref_last_error() { return g_err; }

int ref_layernorm_mod(const float* x, int64_t rows, int64_t dim, float eps, mx::RowMod scale, mx::RowMod shift, void* out, void* s) {
  return guard([&] { mx::layernorm_mod(x, rows, dim, eps, scale, shift, static_cast<bf16*>(out), st(s)); });
}
int ref_rmsnorm_mod(const float* x, int64_t rows, int64_t dim, float eps, const float* w, mx::RowMod scale, mx::RowMod shift, void* out, void* s) {
  return guard([&] { mx::rmsnorm_mod(x, rows, dim, eps, w, scale, shift, static_cast<bf16*>(out), st(s)); });
}
int ref_rmsnorm_bf16(const void* x, int64_t rows, int64_t dim, float eps, const float* w, void* out, void* s) {
  return guard([&] { mx::rmsnorm_bf16(static_cast<const bf16*>(x), rows, dim, eps, w, static_cast<bf16*>(out), st(s)); });
}
int ref_gated_residual(float* x, const void* y, int64_t rows, int64_t dim, mx::RowMod gate, int gate_tanh, void* s) {
  return guard([&] { mx::gated_residual(x, static_cast<const bf16*>(y), rows, dim, gate, gate_tanh, st(s)); });
}
int ref_add_inplace_bf16(void* x, const void* y, int64_t n, void* s) {
  return guard([&] { mx::add_inplace_bf16(static_cast<bf16*>(x), static_cast<const bf16*>(y), n, st(s)); });
}
int ref_head_norm_rope(const void* in, int64_t S, int64_t in_stride, int64_t col0, int H, int D, const float* norm_w, float eps,
                       const float* cos, const float* sin, int rot, int mode, void* out, void* s) {
  return guard([&] {
    mx::head_norm_rope(static_cast<const bf16*>(in), S, in_stride, col0, H, D, norm_w, eps, cos, sin, rot, mx::RopeMode(mode),
                       static_cast<bf16*>(out), st(s));
  });
}
int ref_silu_mul(const void* gu, int64_t rows, int64_t F, void* out, void* s) {
  return guard([&] { mx::silu_mul(static_cast<const bf16*>(gu), rows, F, static_cast<bf16*>(out), st(s)); });
}
int ref_gelu_tanh_inplace(void* x, int64_t n, void* s) {
  return guard([&] { mx::gelu_tanh_inplace(static_cast<bf16*>(x), n, st(s)); });
}
int ref_gelu_erf_inplace(void* x, int64_t n, void* s) {
  return guard([&] { mx::gelu_erf_inplace(static_cast<bf16*>(x), n, st(s)); });
}
int ref_silu_inplace_f32(float* x, int64_t n, void* s) {
  return guard([&] { mx::silu_inplace_f32(x, n, st(s)); });
}
int ref_scatter_rows(float* x, int64_t dim, const int32_t* rows, const void* src, int64_t n, int add, void* s) {
  return guard([&] { mx::scatter_rows(x, dim, rows, static_cast<const bf16*>(src), n, add, st(s)); });
}
int ref_add_bias_bf16(void* y, const float* bias, int64_t rows, int64_t dim, void* s) {
  return guard([&] { mx::add_bias_bf16(static_cast<bf16*>(y), bias, rows, dim, st(s)); });
}
int ref_add_bias_f32(float* y, const float* bias, int64_t rows, int64_t dim, void* s) {
  return guard([&] { mx::add_bias_f32(y, bias, rows, dim, st(s)); });
}
int ref_f32_to_bf16(const float* x, void* y, int64_t n, void* s) {
  return guard([&] { mx::f32_to_bf16(x, static_cast<bf16*>(y), n, st(s)); });
}
int ref_bf16_to_f32(const void* x, float* y, int64_t n, void* s) {
  return guard([&] { mx::bf16_to_f32(static_cast<const bf16*>(x), y, n, st(s)); });
}
int ref_axpy_f32(float* x, const float* y, float a, int64_t n, void* s) {
  return guard([&] { mx::axpy_f32(x, y, a, n, st(s)); });
}
int ref_axpby_f32(float* x, const float* y, float a, float b, int64_t n, void* s) {
  return guard([&] { mx::axpby_f32(x, y, a, b, n, st(s)); });
}

}  // extern "C"
