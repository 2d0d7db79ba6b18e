// mx_ops.h - drop-in for the reference's src/kernels/ops.h: the same `namespace mx` launcher
// signatures (src/kernels/ops.h:11-61), implemented by calls into libmxk's C ABI.  A non-zero
// status becomes std::runtime_error carrying mxk_last_error(), which is what the reference's
// MX_CHECK / MX_KCHECK macros throw (src/core/common.h:34-48).  Header-only; link with -lmxk.
//
// In the reference tree this header replaces kernels/ops.h (which additionally includes
// core/common.h for the bf16 alias); it defines the alias itself when used stand-alone.
#pragma once

#include <cstdint>
#include <stdexcept>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "mxk.h"

namespace mx {

#ifndef MX_OPS_NO_BF16_ALIAS
using bf16 = __nv_bfloat16;
#endif

struct RowMod {  // src/kernels/ops.h:11-15
  const float* target = nullptr;
  const float* prefix = nullptr;
  int64_t prefix_len = 0;
};
enum RopeMode { ROPE_NONE = 0, ROPE_INTERLEAVED = 1, ROPE_HALF = 2 };  // src/kernels/ops.h:39

namespace detail {
inline void ok(int status) {
  if (status != MXK_OK) throw std::runtime_error(mxk_last_error());
}
inline MxkRowMod c(const RowMod& m) { return MxkRowMod{m.target, m.prefix, m.prefix_len}; }
inline mxk_bf16* p(bf16* x) { return reinterpret_cast<mxk_bf16*>(x); }
inline const mxk_bf16* p(const bf16* x) { return reinterpret_cast<const mxk_bf16*>(x); }
}  // namespace detail

inline void layernorm_mod(const float* x, int64_t rows, int64_t dim, float eps, RowMod scale, RowMod shift, bf16* out,
                          cudaStream_t s) {
  detail::ok(mxk_layernorm_mod(x, rows, dim, eps, detail::c(scale), detail::c(shift), detail::p(out), s));
}
inline void rmsnorm_mod(const float* x, int64_t rows, int64_t dim, float eps, const float* w, RowMod scale, RowMod shift,
                        bf16* out, cudaStream_t s) {
  detail::ok(mxk_rmsnorm_mod(x, rows, dim, eps, w, detail::c(scale), detail::c(shift), detail::p(out), s));
}
inline void rmsnorm_bf16(const bf16* x, int64_t rows, int64_t dim, float eps, const float* w, bf16* out, cudaStream_t s) {
  detail::ok(mxk_rmsnorm_bf16(detail::p(x), rows, dim, eps, w, detail::p(out), s));
}
inline void gated_residual(float* x, const bf16* y, int64_t rows, int64_t dim, RowMod gate, int gate_tanh, cudaStream_t s) {
  detail::ok(mxk_gated_residual(x, detail::p(y), rows, dim, detail::c(gate), gate_tanh, s));
}
inline void add_inplace_bf16(bf16* x, const bf16* y, int64_t n, cudaStream_t s) {
  detail::ok(mxk_add_inplace_bf16(detail::p(x), detail::p(y), n, s));
}
inline void head_norm_rope(const bf16* in, int64_t S, int64_t in_stride, int64_t col0, int H, int D, const float* norm_w,
                           float eps, const float* cos, const float* sin, int rot, RopeMode mode, bf16* out,
                           cudaStream_t s) {
  detail::ok(mxk_head_norm_rope(detail::p(in), S, in_stride, col0, H, D, norm_w, eps, cos, sin, rot, int(mode),
                                detail::p(out), s));
}
inline void silu_mul(const bf16* gu, int64_t rows, int64_t F, bf16* out, cudaStream_t s) {
  detail::ok(mxk_silu_mul(detail::p(gu), rows, F, detail::p(out), s));
}
inline void gelu_tanh_inplace(bf16* x, int64_t n, cudaStream_t s) { detail::ok(mxk_gelu_tanh_inplace(detail::p(x), n, s)); }
inline void gelu_erf_inplace(bf16* x, int64_t n, cudaStream_t s) { detail::ok(mxk_gelu_erf_inplace(detail::p(x), n, s)); }
inline void scatter_rows(float* x, int64_t dim, const int32_t* rows, const bf16* src, int64_t n, int add, cudaStream_t s) {
  detail::ok(mxk_scatter_rows(x, dim, rows, detail::p(src), n, add, s));
}
inline void silu_inplace_f32(float* x, int64_t n, cudaStream_t s) { detail::ok(mxk_silu_inplace_f32(x, n, s)); }
inline void add_bias_bf16(bf16* y, const float* bias, int64_t rows, int64_t dim, cudaStream_t s) {
  detail::ok(mxk_add_bias_bf16(detail::p(y), bias, rows, dim, s));
}
inline void add_bias_f32(float* y, const float* bias, int64_t rows, int64_t dim, cudaStream_t s) {
  detail::ok(mxk_add_bias_f32(y, bias, rows, dim, s));
}
inline void f32_to_bf16(const float* x, bf16* y, int64_t n, cudaStream_t s) { detail::ok(mxk_f32_to_bf16(x, detail::p(y), n, s)); }
inline void bf16_to_f32(const bf16* x, float* y, int64_t n, cudaStream_t s) { detail::ok(mxk_bf16_to_f32(detail::p(x), y, n, s)); }
inline void axpy_f32(float* x, const float* y, float a, int64_t n, cudaStream_t s) { detail::ok(mxk_axpy_f32(x, y, a, n, s)); }
inline void axpby_f32(float* x, const float* y, float a, float b, int64_t n, cudaStream_t s) {
  detail::ok(mxk_axpby_f32(x, y, a, b, n, s));
}

}  // namespace mx
