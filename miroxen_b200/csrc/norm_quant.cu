// Norm + modulation + MXFP8 quantisation in one pass: layernorm_mod / rmsnorm_mod of src/kernels/ops.cu:153-170
// followed by quantize_blockscaled(MXFP8) of src/kernels/blockscale.cu:147-164, for a normed activation
// whose only readers are block-scaled GEMMs (the q/k/v and MLP-up projections).  The bulk-copy row
// kernel rounds its output to bf16, parks the row in shared memory and quantises it from there instead of storing it: 5 bytes per
// element instead of 6 + 3.
#include "norm_dispatch.cuh"

using namespace mxk;

namespace {

// y != nullptr: the residual update x += act(gate) * y runs first, in the same pass (FUSE_RES).
template <int MODE, bool FUSE_RES = false>
int run_norm_quant(const char* name, const float* x, int64_t rows, int64_t dim, float eps, const float* w, MxkRowMod scale,
                   MxkRowMod shift, void* q, uint8_t* sf, cudaStream_t s, float* xw = nullptr, const mxk_bf16* y = nullptr,
                   MxkRowMod gate = MxkRowMod{}, int gate_tanh = 0) {
  if (rows <= 0) return MXK_OK;
  if (int rc = check_norm_common(name, x, rows, dim, q, scale, shift)) return rc;
  if (FUSE_RES) {
    if (!y) return fail(MXK_ERR_INVALID_ARG, "%s: null y", name);
    if (gate.target && !gate.prefix && gate.prefix_len > 0)
      return fail(MXK_ERR_INVALID_ARG, "%s: prefix_len > 0 with a null prefix vector", name);
  }
  if (!sf) return fail(MXK_ERR_INVALID_ARG, "%s: null scale buffer", name);
  if (dim % 32 != 0 || !aligned(q, 16)) return fail(MXK_ERR_INVALID_ARG, "%s: need dim %% 32 == 0 and a 16-byte aligned q", name);
  NormArgs a{};
  a.x = x, a.rows = rows, a.dim = int(dim), a.nvec = int(dim / 4), a.eps = eps, a.w = w, a.scale = scale, a.shift = shift;
  a.q = static_cast<uint8_t*>(q), a.sf = sf, a.nkb_pad = int(pad_to(dim / 32, 4));
  if (FUSE_RES) a.xw = xw, a.y = reinterpret_cast<const bf16*>(y), a.gate = gate, a.gate_tanh = gate_tanh;
  NormPlan p;
  // The one-pass form exists for the bulk-copy row kernel only, whose copies need x (and y) rows on 16-byte boundaries.
  if (!norm_quant_ok<FUSE_RES>(a, p))
    return fail(MXK_ERR_INVALID_ARG, "%s: dim %lld or an unaligned vector is outside the one-pass kernel; call the norm and "
                "mxk_quantize_blockscaled separately", name, (long long)dim);
  // scale padding, as mxk_quantize_blockscaled clears it
  const int64_t nkb = dim / 32;
  cudaError_t e = cudaSuccess;
  if (nkb % 4 != 0) e = cudaMemsetAsync(sf, 0, size_t(pad_to(rows, 128) * pad_to(nkb, 4)), s);
  else if (rows % 128 != 0) e = cudaMemsetAsync(sf + rows / 128 * nkb * 128, 0, size_t(nkb * 128), s);
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "%s: cudaMemsetAsync: %s", name, cudaGetErrorString(e));
  if constexpr (MODE == 1) {
    if (w) launch_norm<1, float, true, FUSE_RES, true>(p, a, true, s);
    else launch_norm<1, float, false, FUSE_RES, true>(p, a, true, s);
  } else {
    launch_norm<0, float, false, FUSE_RES, true>(p, a, true, s);
  }
  return after_launch(name);
}

}  // namespace

extern "C" {

int mxk_layernorm_mod_quant_mxfp8(const float* x, int64_t rows, int64_t dim, float eps, MxkRowMod scale, MxkRowMod shift,
                                  void* q, uint8_t* sf, mxk_stream_t stream) {
  return run_norm_quant<0>("layernorm_mod_quant_mxfp8", x, rows, dim, eps, nullptr, scale, shift, q, sf, as_stream(stream));
}

int mxk_rmsnorm_mod_quant_mxfp8(const float* x, int64_t rows, int64_t dim, float eps, const float* w, MxkRowMod scale,
                                MxkRowMod shift, void* q, uint8_t* sf, mxk_stream_t stream) {
  return run_norm_quant<1>("rmsnorm_mod_quant_mxfp8", x, rows, dim, eps, w, scale, shift, q, sf, as_stream(stream));
}

int mxk_gated_residual_norm_quant_mxfp8(float* x, const mxk_bf16* y, int64_t rows, int64_t dim, MxkRowMod gate, int gate_tanh,
                                        int norm_mode, float eps, const float* w, MxkRowMod scale, MxkRowMod shift, void* q,
                                        uint8_t* sf, mxk_stream_t stream) {
  if (norm_mode != 0 && norm_mode != 1)
    return fail(MXK_ERR_INVALID_ARG, "gated_residual_norm_quant_mxfp8: norm_mode=%d (0 LayerNorm, 1 RMSNorm)", norm_mode);
  if (norm_mode == 0)
    return run_norm_quant<0, true>("gated_residual_norm_quant_mxfp8", x, rows, dim, eps, nullptr, scale, shift, q, sf,
                                   as_stream(stream), x, y, gate, gate_tanh);
  return run_norm_quant<1, true>("gated_residual_norm_quant_mxfp8", x, rows, dim, eps, w, scale, shift, q, sf,
                                 as_stream(stream), x, y, gate, gate_tanh);
}

}  // extern "C"
