"""Python host mirror of the reference's launcher API (src/kernels/ops.h:18-61) over libmxk.

Same names, argument order and meaning as the reference's `namespace mx` functions; tensors are
torch CUDA tensors (bf16 tensors are torch.bfloat16), the stream defaults to torch's current
stream.  Every function launches asynchronously and raises MxkError on a non-zero status.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import BlockArgs, HeadTensor, RopeRun, RowMod, check, lib

ROPE_NONE, ROPE_INTERLEAVED, ROPE_HALF = 0, 1, 2
ACT_GELU_TANH, ACT_SILU_MUL, ACT_GELU_ERF = 0, 1, 2
Q_MXFP8, Q_NVFP4 = 1, 2  # QMode of src/kernels/blockscale.h:14 (0 = None is not a quantised mode)

__all__ = [
    "ROPE_NONE", "ROPE_INTERLEAVED", "ROPE_HALF", "row_mod", "layernorm_mod", "rmsnorm_mod", "rmsnorm_bf16",
    "gated_residual", "add_inplace_bf16", "head_norm_rope", "silu_mul", "gelu_tanh_inplace", "gelu_erf_inplace",
    "scatter_rows", "silu_inplace_f32", "add_bias_bf16", "add_bias_f32", "f32_to_bf16", "bf16_to_f32", "axpy_f32",
    "axpby_f32", "gated_residual_norm", "qkv_norm_rope", "HeadSpec", "dit_block_ops", "BlockArgs", "RowMod",
    "HostPipeline", "OpTimes", "dit_block_ops_prefix", "dit_block_ops_host_static", "device_error", "launch_count", "reset_launch_count", "set_tuning",
    "Q_MXFP8", "Q_NVFP4", "QMat", "qdata_bytes", "qscale_bytes", "quantize_blockscaled", "act_quantize_mxfp8",
    "ACT_GELU_TANH", "ACT_SILU_MUL", "ACT_GELU_ERF", "layernorm_mod_quant_mxfp8", "rmsnorm_mod_quant_mxfp8", "gated_residual_norm_quant_mxfp8",
    "qwen_latent_encode", "qwen_latent_decode", "h3_latent_video", "h3_latent_audio",
    "bias_gelu_tanh_inplace", "bias_silu_mul", "gated_residual_bias",
    "linear_bf16", "linear_act", "linear_silu_mul", "linear_gated_residual", "linear_qkv_norm_rope", "quantize_nvfp4_known_amax", "layernorm_mod_amax", "rmsnorm_mod_amax", "gated_residual_norm_amax", "act_amax",
    "norm_path_probe", "NORM_PATH_GENERIC", "NORM_PATH_VECTOR", "NORM_PATH_BULK",
]


def _p(t) -> Optional[int]:
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def _stream(stream) -> Optional[int]:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream or None
    if isinstance(stream, int):
        return stream or None
    return stream.cuda_stream or None


def row_mod(target=None, prefix=None, prefix_len: int = 0) -> RowMod:
    """RowMod{target, prefix, prefix_len}; with one vector set pass it as `target` only."""
    if target is not None and prefix is None:
        prefix = target
    return RowMod(_p(target), _p(prefix), int(prefix_len))


_NONE = RowMod(None, None, 0)


def layernorm_mod(x, rows, dim, eps, scale: RowMod, shift: RowMod, out, stream=None):
    check(lib().mxk_layernorm_mod(_p(x), rows, dim, eps, scale or _NONE, shift or _NONE, _p(out), _stream(stream)))


def rmsnorm_mod(x, rows, dim, eps, w, scale: RowMod, shift: RowMod, out, stream=None):
    check(lib().mxk_rmsnorm_mod(_p(x), rows, dim, eps, _p(w), scale or _NONE, shift or _NONE, _p(out), _stream(stream)))


def rmsnorm_bf16(x, rows, dim, eps, w, out, stream=None):
    check(lib().mxk_rmsnorm_bf16(_p(x), rows, dim, eps, _p(w), _p(out), _stream(stream)))


NORM_PATH_GENERIC, NORM_PATH_VECTOR, NORM_PATH_BULK = 0, 1, 2


def norm_path_probe(op, x, y, out, w, rows, dim, scale: RowMod = None, shift: RowMod = None, gate: RowMod = None) -> int:
    """Kernel family a norm call with these pointers and sizes takes (host arithmetic only; see mxk.h)."""
    return lib().mxk_norm_path_probe(int(op), _p(x), _p(y), _p(out), _p(w), scale or _NONE, shift or _NONE, gate or _NONE,
                                     rows, dim)


def gated_residual(x, y, rows, dim, gate: RowMod, gate_tanh, stream=None):
    check(lib().mxk_gated_residual(_p(x), _p(y), rows, dim, gate or _NONE, int(gate_tanh), _stream(stream)))


def add_inplace_bf16(x, y, n, stream=None):
    check(lib().mxk_add_inplace_bf16(_p(x), _p(y), n, _stream(stream)))


def head_norm_rope(in_, S, in_stride, col0, H, D, norm_w, eps, cos, sin, rot, mode, out, stream=None):
    check(lib().mxk_head_norm_rope(_p(in_), S, in_stride, col0, H, D, _p(norm_w), eps, _p(cos), _p(sin), rot, mode,
                                   _p(out), _stream(stream)))


def silu_mul(gu, rows, F, out, stream=None):
    check(lib().mxk_silu_mul(_p(gu), rows, F, _p(out), _stream(stream)))


def gelu_tanh_inplace(x, n, stream=None):
    check(lib().mxk_gelu_tanh_inplace(_p(x), n, _stream(stream)))


def gelu_erf_inplace(x, n, stream=None):
    check(lib().mxk_gelu_erf_inplace(_p(x), n, _stream(stream)))


def scatter_rows(x, dim, rows, src, n, add, stream=None):
    check(lib().mxk_scatter_rows(_p(x), dim, _p(rows), _p(src), n, int(add), _stream(stream)))


def silu_inplace_f32(x, n, stream=None):
    check(lib().mxk_silu_inplace_f32(_p(x), n, _stream(stream)))


def add_bias_bf16(y, bias, rows, dim, stream=None):
    check(lib().mxk_add_bias_bf16(_p(y), _p(bias), rows, dim, _stream(stream)))


def add_bias_f32(y, bias, rows, dim, stream=None):
    check(lib().mxk_add_bias_f32(_p(y), _p(bias), rows, dim, _stream(stream)))


def f32_to_bf16(x, y, n, stream=None):
    check(lib().mxk_f32_to_bf16(_p(x), _p(y), n, _stream(stream)))


def bf16_to_f32(x, y, n, stream=None):
    check(lib().mxk_bf16_to_f32(_p(x), _p(y), n, _stream(stream)))


def axpy_f32(x, y, a, n, stream=None):
    check(lib().mxk_axpy_f32(_p(x), _p(y), a, n, _stream(stream)))


def axpby_f32(x, y, a, b, n, stream=None):
    check(lib().mxk_axpby_f32(_p(x), _p(y), a, b, n, _stream(stream)))


# ---- fused extensions -------------------------------------------------------------------------

def gated_residual_norm(x, y, rows, dim, gate: RowMod, gate_tanh, norm_mode, eps, w, scale: RowMod, shift: RowMod, out,
                        stream=None):
    """gated_residual followed by layernorm_mod (norm_mode 0) / rmsnorm_mod (1) on the same rows."""
    check(lib().mxk_gated_residual_norm(_p(x), _p(y), rows, dim, gate or _NONE, int(gate_tanh), norm_mode, eps, _p(w),
                                        scale or _NONE, shift or _NONE, _p(out), _stream(stream)))


@dataclass
class HeadSpec:
    """One tensor of a qkv_norm_rope launch (the per-tensor arguments of head_norm_rope)."""
    in_: object
    in_stride: int
    col0: int
    norm_w: object
    out: object
    rot: int
    mode: int


def qkv_norm_rope(tensors: Sequence[HeadSpec], S, H, D, eps, cos, sin, stream=None):
    arr = (HeadTensor * len(tensors))(*[
        HeadTensor(_p(t.in_), t.in_stride, t.col0, _p(t.norm_w), _p(t.out), t.rot, t.mode) for t in tensors])
    check(lib().mxk_qkv_norm_rope(arr, len(tensors), S, H, D, eps, _p(cos), _p(sin), _stream(stream)))


def dit_block_ops(args: BlockArgs, stream=None):
    """The op sequence of one DiT block (see MxkBlockArgs in include/mxk.h)."""
    check(lib().mxk_dit_block_ops(C.byref(args), _stream(stream)))


def dit_block_ops_prefix(args: BlockArgs, n_ops: int, stream=None):
    """Only the first n_ops launches of dit_block_ops (measurement aid)."""
    check(lib().mxk_dit_block_ops_prefix(C.byref(args), int(n_ops), _stream(stream)))


class OpTimes:
    """mxk_op_times_*: per-op CUDA-event timing of a block pass."""

    def __init__(self):
        self._h = C.c_void_p()
        check(lib().mxk_op_times_create(C.byref(self._h)))

    def run(self, args: BlockArgs, stream=None):
        check(lib().mxk_dit_block_ops_timed(C.byref(args), _stream(stream), self._h))

    def read(self):
        buf = (C.c_float * 16)()
        n = lib().mxk_op_times_read(self._h, buf, 16)
        if n < 0:
            check(n)
        return [buf[i] for i in range(n)]

    def close(self):
        if self._h:
            lib().mxk_op_times_destroy(self._h)
            self._h = C.c_void_p()


class HostPipeline:
    """mxk_host_pipeline_*: the block sequence on HOST buffers, streamed through the GPU in row chunks."""

    def __init__(self, chunk_rows, dim, F, H, D, rot, with_v=False, act_mode=0):
        self._h = C.c_void_p()
        check(lib().mxk_host_pipeline_create(chunk_rows, dim, F, H, D, rot, int(with_v), act_mode, C.byref(self._h)))

    def run(self, args: BlockArgs):
        up, down = C.c_int64(0), C.c_int64(0)
        check(lib().mxk_dit_block_ops_host(self._h, C.byref(args), C.byref(up), C.byref(down)))
        return up.value, down.value

    def close(self):
        if self._h:
            lib().mxk_host_pipeline_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def dit_block_ops_host_static(args: BlockArgs, stream=None):
    """mxk_dit_block_ops_host_static: the block sequence on HOST buffers for callers that may not allocate
    device memory; staging is a fixed array inside the library (see include/mxk.h for the limit and the
    sharing rules).  Returns (h2d_bytes, d2h_bytes) once the results are in host memory."""
    up, down = C.c_int64(0), C.c_int64(0)
    check(lib().mxk_dit_block_ops_host_static(C.byref(args), _stream(stream), C.byref(up), C.byref(down)))
    return up.value, down.value


@dataclass
class QMat:
    """The reference's QMat (src/kernels/blockscale.h:21-25): quantised data, block scales in
    cuBLASLt's interleaved layout, and for NVFP4 the device fp32 max|x| (tensor scale = amax / 2688)."""
    q: torch.Tensor
    sf: torch.Tensor
    amax: Optional[torch.Tensor] = None


def qdata_bytes(mode: int, rows: int, K: int) -> int:
    return int(lib().mxk_qdata_bytes(mode, rows, K))


def qscale_bytes(mode: int, rows: int, K: int) -> int:
    return int(lib().mxk_qscale_bytes(mode, rows, K))


def quantize_blockscaled(mode: int, x, ldx: int, rows: int, K: int, out: Optional[QMat] = None, stream=None) -> QMat:
    """quantize_blockscaled(QMode, x, ldx, rows, K, out, stream) of src/kernels/blockscale.h:30; allocates
    the QMat on x's device when `out` is None."""
    if out is None:
        dev = x.device
        out = QMat(torch.empty(qdata_bytes(mode, rows, K), dtype=torch.uint8, device=dev),
                   torch.empty(qscale_bytes(mode, rows, K), dtype=torch.uint8, device=dev),
                   torch.empty(1, dtype=torch.float32, device=dev) if mode == Q_NVFP4 else None)
    check(lib().mxk_quantize_blockscaled(mode, _p(x), ldx, rows, K, _p(out.q), _p(out.sf), _p(out.amax), _stream(stream)))
    return out


def act_quantize_mxfp8(act_mode: int, in_, rows: int, F: int, out: Optional[QMat] = None, stream=None, bias=None) -> QMat:
    """The MLP activation (gelu_tanh_inplace / silu_mul / gelu_erf_inplace of src/kernels/ops.h:36-41) and its
    MXFP8 quantisation in one pass; same bytes as the two calls, without writing the bf16 activation."""
    if out is None:
        out = QMat(torch.empty(qdata_bytes(Q_MXFP8, rows, F), dtype=torch.uint8, device=in_.device),
                   torch.empty(qscale_bytes(Q_MXFP8, rows, F), dtype=torch.uint8, device=in_.device))
    check(lib().mxk_act_quantize_mxfp8(act_mode, _p(in_), _p(bias), rows, F, _p(out.q), _p(out.sf), _stream(stream)))
    return out


def quantize_nvfp4_known_amax(x, ldx: int, rows: int, K: int, amax, out: Optional[QMat] = None, stream=None) -> QMat:
    """NVFP4 quantisation in one pass from a tensor maximum the producing op already left on the device
    (`amax`, fp32 [1]; see the *_amax ops).  Same bytes as quantize_blockscaled(Q_NVFP4, ...)."""
    if out is None:
        out = QMat(torch.empty(qdata_bytes(Q_NVFP4, rows, K), dtype=torch.uint8, device=x.device),
                   torch.empty(qscale_bytes(Q_NVFP4, rows, K), dtype=torch.uint8, device=x.device), amax)
    check(lib().mxk_quantize_nvfp4_known_amax(_p(x), ldx, rows, K, _p(out.q), _p(out.sf), _p(amax), _stream(stream)))
    return out


def layernorm_mod_amax(x, rows, dim, eps, scale: RowMod, shift: RowMod, out, amax_out, stream=None):
    check(lib().mxk_layernorm_mod_amax(_p(x), rows, dim, eps, scale or _NONE, shift or _NONE, _p(out), _p(amax_out), _stream(stream)))


def rmsnorm_mod_amax(x, rows, dim, eps, w, scale: RowMod, shift: RowMod, out, amax_out, stream=None):
    check(lib().mxk_rmsnorm_mod_amax(_p(x), rows, dim, eps, _p(w), scale or _NONE, shift or _NONE, _p(out), _p(amax_out),
                                     _stream(stream)))


def gated_residual_norm_amax(x, y, rows, dim, gate: RowMod, gate_tanh, norm_mode, eps, w, scale: RowMod, shift: RowMod, out,
                             amax_out, stream=None):
    check(lib().mxk_gated_residual_norm_amax(_p(x), _p(y), rows, dim, gate or _NONE, int(gate_tanh), norm_mode, eps, _p(w),
                                             scale or _NONE, shift or _NONE, _p(out), _p(amax_out), _stream(stream)))


def act_amax(act_mode: int, in_, rows: int, F: int, out, amax_out, bias=None, stream=None):
    """The MLP activation (0 GELU-tanh, 1 silu_mul, 2 GELU-erf; optional bias first) writing bf16 `out` and the
    tensor maximum of what it wrote."""
    check(lib().mxk_act_amax(act_mode, _p(in_), _p(bias), rows, F, _p(out), _p(amax_out), _stream(stream)))


def linear_bf16(A, W, bias, M, N, K, y, stream=None):
    """y bf16 [M, N] = A [M, K] @ W [N, K]^T (+ bias): the reference's linear() as one tensor-core kernel."""
    check(lib().mxk_linear_bf16(_p(A), _p(W), _p(bias), M, N, K, _p(y), _stream(stream)))


def linear_act(A, W, bias, M, N, K, act_mode, y, stream=None):
    """y bf16 [M, N] = act(A @ W^T (+ bias)), act_mode 0 GELU (tanh form) / 2 GELU (erf form): linear() and
    gelu_tanh_inplace() in one kernel."""
    check(lib().mxk_linear_act(_p(A), _p(W), _p(bias), M, N, K, int(act_mode), _p(y), _stream(stream)))


def linear_silu_mul(A, W, bias, M, F, K, out, stream=None):
    """out bf16 [M, F] = silu(g) * u with [g | u] = A @ W [2F, K]^T (+ bias [2F]): linear(gate_up) and silu_mul() in one
    kernel; the [M, 2F] projection is never written."""
    check(lib().mxk_linear_silu_mul(_p(A), _p(W), _p(bias), M, F, K, _p(out), _stream(stream)))


def linear_gated_residual(A, W, bias, M, N, K, x, gate: RowMod, gate_tanh, stream=None):
    """x fp32 [M, N] += act(gate) * bf16(A @ W^T (+ bias)): linear() and gated_residual() in one kernel."""
    check(lib().mxk_linear_gated_residual(_p(A), _p(W), _p(bias), M, N, K, _p(x), gate or _NONE, int(gate_tanh), _stream(stream)))


def linear_qkv_norm_rope(A, W, bias, M, K, H, D, tensors: Sequence[HeadSpec], eps, cos, sin, stream=None):
    """The QKV projection with per-head RMSNorm + rotary embedding in its epilogue (specs: norm_w, out, rot, mode)."""
    arr = (HeadTensor * len(tensors))(*[HeadTensor(None, 0, 0, _p(t.norm_w), _p(t.out), t.rot, t.mode) for t in tensors])
    check(lib().mxk_linear_qkv_norm_rope(_p(A), _p(W), _p(bias), M, K, H, D, arr, len(tensors), eps, _p(cos), _p(sin), _stream(stream)))


def _qmat_for(x, rows, dim, out):
    if out is not None:
        return out
    return QMat(torch.empty(qdata_bytes(Q_MXFP8, rows, dim), dtype=torch.uint8, device=x.device),
                torch.empty(qscale_bytes(Q_MXFP8, rows, dim), dtype=torch.uint8, device=x.device))


def layernorm_mod_quant_mxfp8(x, rows, dim, eps, scale: RowMod, shift: RowMod, out: Optional[QMat] = None, stream=None) -> QMat:
    """layernorm_mod (src/kernels/ops.h:22) and its MXFP8 quantisation in one pass."""
    out = _qmat_for(x, rows, dim, out)
    check(lib().mxk_layernorm_mod_quant_mxfp8(_p(x), rows, dim, eps, scale or _NONE, shift or _NONE, _p(out.q), _p(out.sf),
                                              _stream(stream)))
    return out


def rmsnorm_mod_quant_mxfp8(x, rows, dim, eps, w, scale: RowMod, shift: RowMod, out: Optional[QMat] = None, stream=None) -> QMat:
    """rmsnorm_mod (src/kernels/ops.h:24) and its MXFP8 quantisation in one pass."""
    out = _qmat_for(x, rows, dim, out)
    check(lib().mxk_rmsnorm_mod_quant_mxfp8(_p(x), rows, dim, eps, _p(w), scale or _NONE, shift or _NONE, _p(out.q), _p(out.sf),
                                            _stream(stream)))
    return out


def bias_gelu_tanh_inplace(x, bias, rows, F, stream=None):
    """add_bias_bf16 (src/kernels/ops.h:53) + gelu_tanh_inplace (ops.h:46) in one pass over x [rows, F]."""
    check(lib().mxk_bias_gelu_tanh_inplace(_p(x), _p(bias), rows, F, _stream(stream)))


def bias_silu_mul(gu, bias, rows, F, out, stream=None):
    """add_bias_bf16 on gu [rows, 2F] + silu_mul (ops.h:44) in one pass."""
    check(lib().mxk_bias_silu_mul(_p(gu), _p(bias), rows, F, _p(out), _stream(stream)))


def gated_residual_bias(x, y, bias, rows, dim, gate: RowMod, gate_tanh, stream=None):
    """add_bias_bf16 on y + gated_residual (ops.h:27) in one pass."""
    check(lib().mxk_gated_residual_bias(_p(x), _p(y), _p(bias), rows, dim, gate or _NONE, int(gate_tanh), _stream(stream)))


def qwen_latent_encode(x, y, n, mean, std, stream=None):
    """mx::qwen_latent::encode (src/kernels/qwen_latent.h:7): [64, n] -> [n, 64], (x - mean) / std."""
    check(lib().mxk_qwen_latent_encode(_p(x), _p(y), n, _p(mean), _p(std), _stream(stream)))


def qwen_latent_decode(x, y, n, mean, std, stream=None):
    """mx::qwen_latent::decode (src/kernels/qwen_latent.h:8): [n, 64] -> [64, n], x * std + mean."""
    check(lib().mxk_qwen_latent_decode(_p(x), _p(y), n, _p(mean), _p(std), _stream(stream)))


def h3_latent_video(rows, z, frames, h, w, stream=None):
    """mx::h3_latent::video (src/kernels/h3_latent.h:6)."""
    check(lib().mxk_h3_latent_video(_p(rows), _p(z), frames, h, w, _stream(stream)))


def h3_latent_audio(rows, z, samples, stream=None):
    """mx::h3_latent::audio (src/kernels/h3_latent.h:7)."""
    check(lib().mxk_h3_latent_audio(_p(rows), _p(z), samples, _stream(stream)))


def gated_residual_norm_quant_mxfp8(x, y, rows, dim, gate: RowMod, gate_tanh, norm_mode, eps, w, scale: RowMod, shift: RowMod,
                                    out: Optional[QMat] = None, stream=None) -> QMat:
    """gated_residual, the norm and its MXFP8 quantisation in one pass (x updated in place)."""
    out = _qmat_for(x, rows, dim, out)
    check(lib().mxk_gated_residual_norm_quant_mxfp8(_p(x), _p(y), rows, dim, gate or _NONE, int(gate_tanh), int(norm_mode), eps,
                                                    _p(w), scale or _NONE, shift or _NONE, _p(out.q), _p(out.sf), _stream(stream)))
    return out


def device_error(clear: bool = True) -> int:
    """0, or the code a kernel left when one of its bounded waits ran out (synchronises)."""
    v = C.c_int(0)
    check(lib().mxk_device_error(C.byref(v), int(clear)))
    return v.value


def launch_count() -> int:
    return lib().mxk_launch_count()


def reset_launch_count() -> None:
    lib().mxk_reset_launch_count()


def set_tuning(name: str, value: int) -> None:
    check(lib().mxk_set_tuning(name.encode(), value))
