"""ctypes binding of libmxk.so: prototypes for every symbol include/mxk.h declares."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
HEADER = PKG.parent / "include" / "mxk.h"


class MxkError(RuntimeError):
    """A libmxk call returned a non-zero status (the reference throws std::runtime_error)."""


class RowMod(C.Structure):
    """MxkRowMod / the reference's RowMod (src/kernels/ops.h:11-15)."""
    _fields_ = [("target", C.c_void_p), ("prefix", C.c_void_p), ("prefix_len", C.c_int64)]


class HeadTensor(C.Structure):
    _fields_ = [("in_", C.c_void_p), ("in_stride", C.c_int64), ("col0", C.c_int64), ("norm_w", C.c_void_p),
                ("out", C.c_void_p), ("rot", C.c_int), ("mode", C.c_int)]


class RopeRun(C.Structure):
    _fields_ = [("row0", C.c_int64), ("n0", C.c_int32), ("n1", C.c_int32), ("n2", C.c_int32),
                ("base", C.c_int32 * 3), ("step0", C.c_int32 * 3), ("step1", C.c_int32 * 3), ("step2", C.c_int32 * 3)]


class BlockArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_int64), ("dim", C.c_int64), ("F", C.c_int64),
        ("H", C.c_int), ("D", C.c_int), ("norm_mode", C.c_int), ("eps", C.c_float),
        ("act_mode", C.c_int), ("fused", C.c_int), ("chunk_rows", C.c_int64),
        ("norm1_w", C.c_void_p), ("norm2_w", C.c_void_p),
        ("shift1", RowMod), ("scale1", RowMod), ("gate1", RowMod),
        ("shift2", RowMod), ("scale2", RowMod), ("gate2", RowMod),
        ("gate_tanh", C.c_int),
        ("q_in", C.c_void_p), ("k_in", C.c_void_p), ("v_in", C.c_void_p),
        ("qkv_stride", C.c_int64), ("q_col0", C.c_int64), ("k_col0", C.c_int64), ("v_col0", C.c_int64),
        ("norm_q", C.c_void_p), ("norm_k", C.c_void_p), ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("rot", C.c_int), ("rope_mode", C.c_int),
        ("q_out", C.c_void_p), ("k_out", C.c_void_p), ("v_out", C.c_void_p),
        ("x", C.c_void_p), ("h1", C.c_void_p), ("h2", C.c_void_p), ("attn_o", C.c_void_p),
        ("act", C.c_void_p), ("act2", C.c_void_p), ("mlp_o", C.c_void_p),
    ]


_P, _I64, _I, _F = C.c_void_p, C.c_int64, C.c_int, C.c_float

# name -> (restype, argtypes); must list every function include/mxk.h declares.
PROTOTYPES = {
    "mxk_last_error": (C.c_char_p, []),
    "mxk_version": (_I, []),
    "mxk_launch_count": (_I64, []),
    "mxk_reset_launch_count": (None, []),
    "mxk_set_tuning": (_I, [C.c_char_p, _I]),
    "mxk_device_error": (_I, [C.POINTER(_I), _I]),
    "mxk_selftest_bounded_wait": (_I, [_P]),
    "mxk_qdata_bytes": (_I64, [_I, _I64, _I64]),
    "mxk_qscale_bytes": (_I64, [_I, _I64, _I64]),
    "mxk_quantize_blockscaled": (_I, [_I, _P, _I64, _I64, _I64, _P, _P, _P, _P]),
    "mxk_layernorm_mod_amax": (_I, [_P, _I64, _I64, _F, RowMod, RowMod, _P, _P, _P]),
    "mxk_rmsnorm_mod_amax": (_I, [_P, _I64, _I64, _F, _P, RowMod, RowMod, _P, _P, _P]),
    "mxk_gated_residual_norm_amax": (_I, [_P, _P, _I64, _I64, RowMod, _I, _I, _F, _P, RowMod, RowMod, _P, _P, _P]),
    "mxk_act_amax": (_I, [_I, _P, _P, _I64, _I64, _P, _P, _P]),
    "mxk_quantize_nvfp4_known_amax": (_I, [_P, _I64, _I64, _I64, _P, _P, _P, _P]),
    "mxk_act_quantize_mxfp8": (_I, [_I, _P, _P, _I64, _I64, _P, _P, _P]),
    "mxk_bias_gelu_tanh_inplace": (_I, [_P, _P, _I64, _I64, _P]),
    "mxk_bias_silu_mul": (_I, [_P, _P, _I64, _I64, _P, _P]),
    "mxk_gated_residual_bias": (_I, [_P, _P, _P, _I64, _I64, RowMod, _I, _P]),
    "mxk_qwen_latent_encode": (_I, [_P, _P, _I64, _P, _P, _P]),
    "mxk_qwen_latent_decode": (_I, [_P, _P, _I64, _P, _P, _P]),
    "mxk_h3_latent_video": (_I, [_P, _P, _I64, _I64, _I64, _P]),
    "mxk_h3_latent_audio": (_I, [_P, _P, _I64, _P]),
    "mxk_layernorm_mod_quant_mxfp8": (_I, [_P, _I64, _I64, _F, RowMod, RowMod, _P, _P, _P]),
    "mxk_rmsnorm_mod_quant_mxfp8": (_I, [_P, _I64, _I64, _F, _P, RowMod, RowMod, _P, _P, _P]),
    "mxk_gated_residual_norm_quant_mxfp8": (_I, [_P, _P, _I64, _I64, RowMod, _I, _I, _F, _P, RowMod, RowMod, _P, _P, _P]),
    "mxk_layernorm_mod": (_I, [_P, _I64, _I64, _F, RowMod, RowMod, _P, _P]),
    "mxk_rmsnorm_mod": (_I, [_P, _I64, _I64, _F, _P, RowMod, RowMod, _P, _P]),
    "mxk_rmsnorm_bf16": (_I, [_P, _I64, _I64, _F, _P, _P, _P]),
    "mxk_norm_path_probe": (_I, [_I, _P, _P, _P, _P, RowMod, RowMod, RowMod, _I64, _I64]),
    "mxk_gated_residual": (_I, [_P, _P, _I64, _I64, RowMod, _I, _P]),
    "mxk_add_inplace_bf16": (_I, [_P, _P, _I64, _P]),
    "mxk_head_norm_rope": (_I, [_P, _I64, _I64, _I64, _I, _I, _P, _F, _P, _P, _I, _I, _P, _P]),
    "mxk_silu_mul": (_I, [_P, _I64, _I64, _P, _P]),
    "mxk_gelu_tanh_inplace": (_I, [_P, _I64, _P]),
    "mxk_gelu_erf_inplace": (_I, [_P, _I64, _P]),
    "mxk_silu_inplace_f32": (_I, [_P, _I64, _P]),
    "mxk_scatter_rows": (_I, [_P, _I64, _P, _P, _I64, _I, _P]),
    "mxk_add_bias_bf16": (_I, [_P, _P, _I64, _I64, _P]),
    "mxk_add_bias_f32": (_I, [_P, _P, _I64, _I64, _P]),
    "mxk_f32_to_bf16": (_I, [_P, _P, _I64, _P]),
    "mxk_bf16_to_f32": (_I, [_P, _P, _I64, _P]),
    "mxk_axpy_f32": (_I, [_P, _P, _F, _I64, _P]),
    "mxk_axpby_f32": (_I, [_P, _P, _F, _F, _I64, _P]),
    "mxk_gated_residual_norm": (_I, [_P, _P, _I64, _I64, RowMod, _I, _I, _F, _P, RowMod, RowMod, _P, _P]),
    "mxk_qkv_norm_rope": (_I, [C.POINTER(HeadTensor), _I, _I64, _I, _I, _F, _P, _P, _P]),
    "mxk_qkv_norm_rope_scatter": (_I, [C.POINTER(HeadTensor), _I, _I64, _I, _I, _F, _P, _P, _I, C.POINTER(_P), _I64, _P]),
    "mxk_gather_head_groups": (_I, [C.POINTER(_P), _I, _I64, _I64, _I, _I, _P, _P]),
    "mxk_peer_buffer_alloc": (_I, [_I64, C.POINTER(_P), _P]),
    "mxk_peer_buffer_open": (_I, [_P, C.POINTER(_P)]),
    "mxk_peer_buffer_close": (_I, [_P]),
    "mxk_peer_buffer_free": (_I, [_P]),
    "mxk_linear_bf16": (_I, [_P, _P, _P, _I64, _I64, _I64, _P, _P]),
    "mxk_linear_act": (_I, [_P, _P, _P, _I64, _I64, _I64, _I, _P, _P]),
    "mxk_linear_silu_mul": (_I, [_P, _P, _P, _I64, _I64, _I64, _P, _P]),
    "mxk_linear_qkv_norm_rope": (_I, [_P, _P, _P, _I64, _I64, _I, _I, C.POINTER(HeadTensor), _I, _F, _P, _P, _P]),
    "mxk_linear_gated_residual": (_I, [_P, _P, _P, _I64, _I64, _I64, _P, RowMod, _I, _P]),
    "mxk_rope_table_expand": (_I, [_P, _P, C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.POINTER(C.c_int32), _I,
                                   C.POINTER(RopeRun), _I, _I64, _I, _P, _P, _P]),
    "mxk_msrope_inv_freq_host": (_I, [C.POINTER(C.c_int32), _I, _F, _P]),
    "mxk_rope_lut_int_host": (_I, [_I64, _I64, _P, _I, _P, _P]),
    "mxk_rope_lut_f32_host": (_I, [_P, _I64, _P, _I, _P, _P]),
    "mxk_h3_spatial_grid_host": (_I, [_I64, _I64, _I64, _P]),
    "mxk_h3_frame_times_host": (_I, [_I64, _I64, _P]),
    "mxk_qwen_timestep_embedding_host": (_I, [_F, _P]),
    "mxk_qwen_timestep_embedding": (_I, [_F, _P, _P]),
    "mxk_h3_time_basis": (_I, [_P, _I64, _P, _I64, _I64, _P, _P]),
    "mxk_dit_block_ops": (_I, [C.POINTER(BlockArgs), _P]),
    "mxk_dit_block_ops_prefix": (_I, [C.POINTER(BlockArgs), _I, _P]),
    "mxk_op_times_create": (_I, [C.POINTER(_P)]),
    "mxk_op_times_destroy": (None, [_P]),
    "mxk_dit_block_ops_timed": (_I, [C.POINTER(BlockArgs), _P, _P]),
    "mxk_op_times_read": (_I, [_P, C.POINTER(C.c_float), _I]),
    "mxk_host_pipeline_create": (_I, [_I64, _I64, _I64, _I, _I, _I, _I, _I, C.POINTER(_P)]),
    "mxk_host_pipeline_destroy": (None, [_P]),
    "mxk_static_stage_bytes": (_I64, []),
    "mxk_dit_block_ops_host_static": (_I, [C.POINTER(BlockArgs), _P, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "mxk_dit_block_ops_host": (_I, [_P, C.POINTER(BlockArgs), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
}

_lib = None


def lib_path() -> Path:
    return PKG / "lib" / "libmxk.so"


def header_symbols() -> list[str]:
    """Every function name declared in include/mxk.h."""
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(mxk_[a-z0-9_]+)\s*\(", text)))


def lib() -> C.CDLL:
    """Loads libmxk.so (once).  Raises if it has not been built: there is no other code path."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not path.exists():
            raise MxkError(f"{path} is missing: build it with `python -m miroxen_b200.build` "
                           "(there is no CPU or PyTorch fallback)")
        handle = C.CDLL(str(path))
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise MxkError(f"libmxk status {status}: {lib().mxk_last_error().decode(errors='replace')}")
