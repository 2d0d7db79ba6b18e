// layernorm_mod / rmsnorm_mod / rmsnorm_bf16 launchers (reference: src/kernels/ops.cu:153-175).
#include "norm_dispatch.cuh"

using namespace mxk;

namespace {
NormArgs make_args(const void* x, int64_t rows, int64_t dim, float eps, const float* w,
                   MxkRowMod scale, MxkRowMod shift, mxk_bf16* out) {
  NormArgs a{};
  a.x = x;
  a.rows = rows;
  a.dim = int(dim);
  a.nvec = int(dim / 4);
  a.eps = eps;
  a.w = w;
  a.scale = scale;
  a.shift = shift;
  a.out = reinterpret_cast<bf16*>(out);
  return a;
}
}  // namespace

extern "C" {

int mxk_layernorm_mod(const float* x, int64_t rows, int64_t dim, float eps, MxkRowMod scale,
                      MxkRowMod shift, mxk_bf16* out, mxk_stream_t stream) {
  if (rows <= 0) return MXK_OK;
  if (int rc = check_norm_common("layernorm_mod", x, rows, dim, out, scale, shift)) return rc;
  return run_norm<0, float, false>("layernorm_mod", make_args(x, rows, dim, eps, nullptr, scale, shift, out),
                                   as_stream(stream));
}

int mxk_rmsnorm_mod(const float* x, int64_t rows, int64_t dim, float eps, const float* w,
                    MxkRowMod scale, MxkRowMod shift, mxk_bf16* out, mxk_stream_t stream) {
  if (rows <= 0) return MXK_OK;
  if (int rc = check_norm_common("rmsnorm_mod", x, rows, dim, out, scale, shift)) return rc;
  return run_norm<1, float, false>("rmsnorm_mod", make_args(x, rows, dim, eps, w, scale, shift, out),
                                   as_stream(stream));
}

int mxk_rmsnorm_bf16(const mxk_bf16* x, int64_t rows, int64_t dim, float eps, const float* w,
                     mxk_bf16* out, mxk_stream_t stream) {
  if (rows <= 0) return MXK_OK;
  if (int rc = check_norm_common("rmsnorm_bf16", x, rows, dim, out, MxkRowMod{}, MxkRowMod{})) return rc;
  return run_norm<1, bf16, false>("rmsnorm_bf16", make_args(x, rows, dim, eps, w, MxkRowMod{}, MxkRowMod{}, out),
                                  as_stream(stream));
}

// The same launches with the tensor maximum of the bf16 output as a by-product (see mxk.h).
static int clear_amax(const char* name, float* amax_out, cudaStream_t s) {
  if (!amax_out) return fail(MXK_ERR_INVALID_ARG, "%s: null amax_out", name);
  cudaError_t e = cudaMemsetAsync(amax_out, 0, sizeof(float), s);
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "%s: cudaMemsetAsync: %s", name, cudaGetErrorString(e));
  return MXK_OK;
}

int mxk_layernorm_mod_amax(const float* x, int64_t rows, int64_t dim, float eps, MxkRowMod scale, MxkRowMod shift,
                           mxk_bf16* out, float* amax_out, mxk_stream_t stream) {
  if (int rc = clear_amax("layernorm_mod_amax", amax_out, as_stream(stream))) return rc;
  if (rows <= 0) return MXK_OK;
  if (int rc = check_norm_common("layernorm_mod_amax", x, rows, dim, out, scale, shift)) return rc;
  NormArgs a = make_args(x, rows, dim, eps, nullptr, scale, shift, out);
  a.amax = amax_out;
  return run_norm<0, float, false>("layernorm_mod_amax", a, as_stream(stream));
}

int mxk_rmsnorm_mod_amax(const float* x, int64_t rows, int64_t dim, float eps, const float* w, MxkRowMod scale,
                         MxkRowMod shift, mxk_bf16* out, float* amax_out, mxk_stream_t stream) {
  if (int rc = clear_amax("rmsnorm_mod_amax", amax_out, as_stream(stream))) return rc;
  if (rows <= 0) return MXK_OK;
  if (int rc = check_norm_common("rmsnorm_mod_amax", x, rows, dim, out, scale, shift)) return rc;
  NormArgs a = make_args(x, rows, dim, eps, w, scale, shift, out);
  a.amax = amax_out;
  return run_norm<1, float, false>("rmsnorm_mod_amax", a, as_stream(stream));
}

int mxk_norm_path_probe(int op, const void* x, const void* y, const void* out, const float* w, MxkRowMod scale,
                        MxkRowMod shift, MxkRowMod gate, int64_t rows, int64_t dim) {
  if (rows <= 0 || dim <= 0 || dim > (int64_t(1) << 30)) return MXK_ERR_INVALID_ARG;
  NormArgs a = make_args(x, rows, dim, 0.f, w, scale, shift, static_cast<mxk_bf16*>(const_cast<void*>(out)));
  NormPlan p;
  const bool fused = op >= 3;
  if (fused) a.xw = static_cast<float*>(const_cast<void*>(x)), a.y = static_cast<const bf16*>(y), a.gate = gate;
  switch (op) {
    case 0: a.w = nullptr; return choose_norm_path<0, float, false>(a, p);
    case 1: return choose_norm_path<1, float, false>(a, p);
    case 2: return choose_norm_path<1, bf16, false>(a, p);
    case 3: a.w = nullptr; return choose_norm_path<0, float, true>(a, p);
    case 4: return choose_norm_path<1, float, true>(a, p);
    case 5:
    case 6:
      // the one-pass MXFP8 forms: `out` stands for the code buffer q
      a.out = nullptr;
      if (dim % 32 != 0 || !aligned(out, 16)) return MXK_ERR_INVALID_ARG;
      if (op == 5) a.w = nullptr;
      return norm_quant_ok<true>(a, p) ? int(kNormPathBulk) : MXK_ERR_INVALID_ARG;
    default: return MXK_ERR_INVALID_ARG;
  }
}

}  // extern "C"
