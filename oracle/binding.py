"""TEST INFRASTRUCTURE ONLY: ctypes/numpy doorway to the CPU oracle (oracle/mxk_oracle.cpp) and,
where they were built, to the reference's own code under oracle/_ref/.

Only tests/, the smoke check and the CPU-baseline leg of bench.py import this module.  bf16
arrays are numpy uint16 holding the raw bit patterns.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


class RowMod(C.Structure):
    _fields_ = [("target", C.c_void_p), ("prefix", C.c_void_p), ("prefix_len", C.c_int64)]


class QwenSeg(C.Structure):
    _fields_ = [("is_text", C.c_int32), ("pad", C.c_int32), ("len", C.c_int64), ("ih", C.c_int64), ("iw", C.c_int64)]


def reference_root() -> Path:
    """Where the reference tree is expected: the Makefile's REF variable (environment REF, or its default)."""
    import os
    env = os.environ.get("REF")
    if env:
        return Path(env)
    for line in (HERE / "Makefile").read_text().splitlines():
        if line.startswith("REF ?="):
            return Path(line.split("?=", 1)[1].strip())
    raise RuntimeError("oracle/Makefile has no REF default")


def build(ref: bool = True) -> None:
    """Compiles the oracle (and, when the reference tree is present, oracle/_ref)."""
    subprocess.run(["make", "-s", "-C", str(HERE), "all"], check=True)
    root = reference_root()
    if ref and (root / "src" / "kernels" / "ops.cu").exists():
        subprocess.run(["make", "-s", "-C", str(HERE), "_ref", f"REF={root}"], check=True)


_libs: dict[str, C.CDLL] = {}


def _load(name: str) -> C.CDLL:
    if name not in _libs:
        path = HERE / name
        if not path.exists():
            if name.startswith("_ref"):
                raise FileNotFoundError(f"{path} not built (needs the reference tree: make -C oracle _ref)")
            build(ref=False)
        _libs[name] = C.CDLL(str(path))
    return _libs[name]


def oracle(fast: bool = False) -> C.CDLL:
    return _load("liboracle_fast.so" if fast else "liboracle.so")


def have_ref_ops() -> bool:
    return (HERE / "_ref" / "libmx_ref_ops.so").exists()


def have_ref_layout() -> bool:
    return (HERE / "_ref" / "libmx_ref_layout.so").exists()


def have_ref_blockscale() -> bool:
    return (HERE / "_ref" / "libmx_ref_blockscale.so").exists()


def ref_blockscale() -> C.CDLL:
    """The reference's src/kernels/blockscale.cu built for sm_100a (device pointers; needs a GPU)."""
    return _load("_ref/libmx_ref_blockscale.so")


def have_ref_latent() -> bool:
    return (HERE / "_ref" / "libmx_ref_latent.so").exists()


def ref_latent() -> C.CDLL:
    """The reference's src/kernels/qwen_latent.cu and h3_latent.cu built for sm_100a (device pointers)."""
    return _load("_ref/libmx_ref_latent.so")


def ref_ops() -> C.CDLL:
    """The reference's src/kernels/ops.cu built for sm_100a (device pointers; needs a GPU)."""
    return _load("_ref/libmx_ref_ops.so")


def ref_layout() -> C.CDLL:
    return _load("_ref/libmx_ref_layout.so")


def have_ref_builders() -> bool:
    return (HERE / "_ref" / "libmx_ref_builders.so").exists()


def ref_builders() -> C.CDLL:
    """The reference's own table / embedding builder statements (src/models/qwen_image/dit.cpp,
    src/models/minimax_h3/dit.cpp), cut out and compiled by oracle/Makefile; host only."""
    return _load("_ref/libmx_ref_builders.so")


# ---- bf16 helpers -------------------------------------------------------------------------------

def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _ptr(a):
    return None if a is None else a.ctypes.data


def mod(target=None, prefix=None, prefix_len=0) -> RowMod:
    if target is not None and prefix is None:
        prefix = target
    m = RowMod(_ptr(target), _ptr(prefix), int(prefix_len))
    m._keep = (target, prefix)
    return m


NONE = RowMod(None, None, 0)
_F, _I64, _I, _P = C.c_float, C.c_int64, C.c_int, C.c_void_p


def set_threads(n: int, fast: bool = False) -> None:
    oracle(fast).or_set_threads(int(n))


# ---- ops (each returns a new array or updates in place like the reference) -----------------------

def layernorm_mod(x, eps, scale=NONE, shift=NONE, fast=False):
    rows, dim = x.shape
    out = np.empty((rows, dim), np.uint16)
    f = oracle(fast).or_layernorm_mod
    f.argtypes, f.restype = [_P, _I64, _I64, _F, RowMod, RowMod, _P], None
    f(_ptr(x), rows, dim, eps, scale, shift, _ptr(out))
    return out


def rmsnorm_mod(x, eps, w=None, scale=NONE, shift=NONE, fast=False):
    rows, dim = x.shape
    out = np.empty((rows, dim), np.uint16)
    f = oracle(fast).or_rmsnorm_mod
    f.argtypes, f.restype = [_P, _I64, _I64, _F, _P, RowMod, RowMod, _P], None
    f(_ptr(x), rows, dim, eps, _ptr(w), scale, shift, _ptr(out))
    return out


def rmsnorm_bf16(x, eps, w=None):
    rows, dim = x.shape
    out = np.empty((rows, dim), np.uint16)
    f = oracle().or_rmsnorm_bf16
    f.argtypes, f.restype = [_P, _I64, _I64, _F, _P, _P], None
    f(_ptr(x), rows, dim, eps, _ptr(w), _ptr(out))
    return out


def gated_residual(x, y, gate=NONE, gate_tanh=0, fast=False):
    rows, dim = x.shape
    f = oracle(fast).or_gated_residual
    f.argtypes, f.restype = [_P, _P, _I64, _I64, RowMod, _I], None
    f(_ptr(x), _ptr(y), rows, dim, gate, int(gate_tanh))
    return x


def add_inplace_bf16(x, y):
    f = oracle().or_add_inplace_bf16
    f.argtypes, f.restype = [_P, _P, _I64], None
    f(_ptr(x), _ptr(y), x.size)
    return x


def head_norm_rope(inp, S, in_stride, col0, H, D, norm_w, eps, cos, sin, rot, mode, fast=False):
    out = np.empty((S, H, D), np.uint16)
    f = oracle(fast).or_head_norm_rope
    f.argtypes, f.restype = [_P, _I64, _I64, _I64, _I, _I, _P, _F, _P, _P, _I, _I, _P], _I
    rc = f(_ptr(inp), S, in_stride, col0, H, D, _ptr(norm_w), eps, _ptr(cos), _ptr(sin), rot, mode, _ptr(out))
    if rc != 0:
        raise ValueError(f"head_norm_rope: D={D} rot={rot} rejected")
    return out


def silu_mul(gu, F, fast=False):
    rows = gu.shape[0]
    out = np.empty((rows, F), np.uint16)
    f = oracle(fast).or_silu_mul
    f.argtypes, f.restype = [_P, _I64, _I64, _P], None
    f(_ptr(gu), rows, F, _ptr(out))
    return out


def _inplace(name, x, fast=False):
    f = getattr(oracle(fast), name)
    f.argtypes, f.restype = [_P, _I64], None
    f(_ptr(x), x.size)
    return x


def gelu_tanh_inplace(x, fast=False):
    return _inplace("or_gelu_tanh_inplace", x, fast)


def gelu_erf_inplace(x):
    return _inplace("or_gelu_erf_inplace", x)


def silu_inplace_f32(x):
    return _inplace("or_silu_inplace_f32", x)


def scatter_rows(x, rows, src, add):
    n, dim = src.shape
    f = oracle().or_scatter_rows
    f.argtypes, f.restype = [_P, _I64, _P, _P, _I64, _I], None
    f(_ptr(x), dim, _ptr(rows), _ptr(src), n, int(add))
    return x


def add_bias_bf16(y, bias):
    f = oracle().or_add_bias_bf16
    f.argtypes, f.restype = [_P, _P, _I64, _I64], None
    f(_ptr(y), _ptr(bias), y.shape[0], y.shape[1])
    return y


def add_bias_f32(y, bias):
    f = oracle().or_add_bias_f32
    f.argtypes, f.restype = [_P, _P, _I64, _I64], None
    f(_ptr(y), _ptr(bias), y.shape[0], y.shape[1])
    return y


def f32_to_bf16(x):
    out = np.empty(x.shape, np.uint16)
    f = oracle().or_f32_to_bf16
    f.argtypes, f.restype = [_P, _P, _I64], None
    f(_ptr(x), _ptr(out), x.size)
    return out


def bf16_to_f32(x):
    out = np.empty(x.shape, np.float32)
    f = oracle().or_bf16_to_f32
    f.argtypes, f.restype = [_P, _P, _I64], None
    f(_ptr(x), _ptr(out), x.size)
    return out


def axpy_f32(x, y, a):
    f = oracle().or_axpy_f32
    f.argtypes, f.restype = [_P, _P, _F, _I64], None
    f(_ptr(x), _ptr(y), a, x.size)
    return x


def axpby_f32(x, y, a, b):
    f = oracle().or_axpby_f32
    f.argtypes, f.restype = [_P, _P, _F, _F, _I64], None
    f(_ptr(x), _ptr(y), a, b, x.size)
    return x


# ---- tables ---------------------------------------------------------------------------------------

def qwen_seq_rows(segs) -> int:
    return sum(int(s[1]) if s[0] == "text" else int(s[1]) * int(s[2]) for s in segs)


def qwen_rope_table(segs, axes=(16, 56, 56), theta=10000.0):
    """segs: [("text", len) | ("image", ih, iw), ...], target image last -> (cos, sin) fp32 [S, half]."""
    S, half = qwen_seq_rows(segs), sum(a // 2 for a in axes)
    arr = (QwenSeg * len(segs))(*[
        QwenSeg(1, 0, int(s[1]), 0, 0) if s[0] == "text" else QwenSeg(0, 0, 0, int(s[1]), int(s[2])) for s in segs])
    cos, sin = np.empty((S, half), np.float32), np.empty((S, half), np.float32)
    f = oracle().or_qwen_rope_table
    f.argtypes, f.restype = [C.POINTER(QwenSeg), _I, C.POINTER(C.c_int32), _F, _P, _P], _I64
    n = f(arr, len(segs), (C.c_int32 * 3)(*axes), theta, _ptr(cos), _ptr(sin))
    assert n == S
    return cos, sin


def qwen_segs(T, H, W, conds=()):
    """The segment list of QwenImageDit::prepare (src/models/qwen_image/dit.cpp:128-144) for a text
    sequence of T rows, condition images conds = [(slot0, h, w), ...] (each replaces h*w/4 placeholder
    rows from slot0 on) and an H x W target image: text and image runs in order, the target last."""
    segs, cur = [], 0
    for slot0, h, w in conds:
        if slot0 > cur:
            segs.append(("text", slot0 - cur))
        segs.append(("image", h, w))
        cur = slot0 + h * w // 4
    if T > cur:
        segs.append(("text", T - cur))
    segs.append(("image", H, W))
    return segs


def ref_qwen_rope_table(T, H, W, conds=()):
    """(cos, sin) fp32 [S, 64] from the reference's own statements (QwenImageDit::prepare)."""
    f = ref_builders().ref_qwen_rope_table
    f.argtypes, f.restype = [_I64, _I64, _I64, _P, _I, _P, _P], _I64
    flat = np.array([v for c in conds for v in c], np.int64).reshape(-1)
    S = f(T, H, W, _ptr(flat) if flat.size else None, len(conds), None, None)
    if S < 0:
        raise RuntimeError("the reference rejected the layout")
    cos, sin = np.empty((S, 64), np.float32), np.empty((S, 64), np.float32)
    f(T, H, W, _ptr(flat) if flat.size else None, len(conds), _ptr(cos), _ptr(sin))
    return cos, sin


def ref_qwen_timestep_embedding(t):
    out = np.empty((2, 256), np.float32)
    f = ref_builders().ref_qwen_timestep_embedding
    f.argtypes, f.restype = [_F, _P], None
    f(t, _ptr(out))
    return out


def ref_h3_time_basis(ts, table):
    grid, basis = table.shape
    ts = np.ascontiguousarray(ts, np.float32)
    out = np.empty((ts.size, basis), np.float32)
    f = ref_builders().ref_h3_time_basis
    f.argtypes, f.restype = [_P, _I64, _P, _I64, _I64, _P], None
    f(_ptr(ts), ts.size, _ptr(table), grid, basis, _ptr(out))
    return out


def ref_h3_rope_table(positions, inv_freq, rot=None):
    S, nf = positions.shape[0], inv_freq.size
    rot = 6 * nf if rot is None else rot
    cos, sin = np.empty((S, rot // 2), np.float32), np.empty((S, rot // 2), np.float32)
    f = ref_builders().ref_h3_rope_table
    f.argtypes, f.restype = [_P, _I64, _P, _I64, _I, _P, _P], None
    f(_ptr(positions), S, _ptr(inv_freq), nf, rot, _ptr(cos), _ptr(sin))
    return cos, sin


def h3_positions(T, F_lat, H, W, A, anchors, use_reference=False):
    """fp32 [S, 3] rotary positions; anchors: list of "first"/"last".  use_reference=True calls the
    reference's own h3_build_layout (oracle/_ref/libmx_ref_layout.so)."""
    rpf = (H // 2) * (W // 2)
    S = T + len(anchors) * rpf + 2 * A + F_lat * rpf
    pos = np.empty((S, 3), np.float32)
    codes = (C.c_int32 * max(1, len(anchors)))(*[0 if a == "first" else 1 for a in anchors])
    f = ref_layout().ref_h3_positions if use_reference else oracle().or_h3_positions
    f.argtypes, f.restype = [_I64, _I64, _I64, _I64, _I64, C.POINTER(C.c_int32), _I, _P], _I64
    n = f(T, F_lat, H, W, A, codes, len(anchors), _ptr(pos))
    assert n == S, (n, S)
    return pos


def h3_ref2va_positions(T, refs, F_lat, H, W, A, use_reference=False):
    """fp32 [S, 3] rotary positions of the reference-conditioned layout; refs: list of dicts
    {kind: "image" | "video" | "audio", frames, h, w, audio}.  use_reference=True calls the reference's
    own h3_build_ref2va_layout (oracle/_ref/libmx_ref_layout.so)."""
    kinds = {"image": 0, "video": 1, "audio": 2}
    n = len(refs)
    kind = (C.c_int32 * max(n, 1))(*[kinds[r["kind"]] for r in refs])
    arr = lambda key: (C.c_int64 * max(n, 1))(*[int(r.get(key, 0)) for r in refs])
    fr, rh, rw, au = arr("frames"), arr("h"), arr("w"), arr("audio")
    f = ref_layout().ref_h3_ref2va_positions if use_reference else oracle().or_h3_ref2va_positions
    f.argtypes = [_I64, _I, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _P]
    f.restype = _I64
    S = f(T, n, kind, fr, rh, rw, au, F_lat, H, W, A, None)
    if S < 0:
        raise RuntimeError("the reference rejected the layout")
    pos = np.empty((S, 3), np.float32)
    f(T, n, kind, fr, rh, rw, au, F_lat, H, W, A, _ptr(pos))
    return pos


def h3_rope_table(positions, inv_freq):
    S, nf = positions.shape[0], inv_freq.size
    cos, sin = np.empty((S, 3 * nf), np.float32), np.empty((S, 3 * nf), np.float32)
    f = oracle().or_h3_rope_table
    f.argtypes, f.restype = [_P, _I64, _P, _I, _P, _P], None
    f(_ptr(positions), S, _ptr(inv_freq), nf, _ptr(cos), _ptr(sin))
    return cos, sin


def qwen_timestep_embedding(t):
    out = np.empty((2, 256), np.float32)
    f = oracle().or_qwen_timestep_embedding
    f.argtypes, f.restype = [_F, _P], None
    f(t, _ptr(out))
    return out


def h3_time_basis(ts, table):
    grid, basis = table.shape
    out = np.empty((ts.size, basis), np.float32)
    f = oracle().or_h3_time_basis
    f.argtypes, f.restype = [_P, _I64, _P, _I64, _I64, _P], None
    f(_ptr(ts), ts.size, _ptr(table), grid, basis, _ptr(out))
    return out


_U8 = C.c_uint8


def f32_to_e4m3(v: np.ndarray) -> np.ndarray:
    f = oracle().or_f32_to_e4m3
    f.argtypes, f.restype = [_F], _U8
    return np.array([f(float(a)) for a in np.asarray(v, np.float32).ravel()], np.uint8).reshape(np.shape(v))


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    f = oracle().or_e4m3_to_f32
    f.argtypes, f.restype = [_U8], _F
    return np.array([f(int(a)) for a in np.asarray(b, np.uint8).ravel()], np.float32).reshape(np.shape(b))


def qscale_bytes(mode, rows, K) -> int:
    f = oracle().or_qscale_bytes
    f.argtypes, f.restype = [C.c_int, _I64, _I64], _I64
    return int(f(mode, rows, K))


def sf_offset(r, kb, nkb_pad) -> int:
    f = oracle().or_sf_offset
    f.argtypes, f.restype = [_I64, _I64, _I64], _I64
    return int(f(r, kb, nkb_pad))


def quantize_blockscaled(mode, x, K=None):
    """x: bf16 bits [rows, ldx] (uint16); quantises columns [0, K).  Returns (q, sf, amax)."""
    x = np.ascontiguousarray(x, np.uint16)
    rows, ldx = x.shape
    K = ldx if K is None else K
    q = np.zeros(rows * K // (2 if mode == 2 else 1), np.uint8)
    sf = np.full(qscale_bytes(mode, rows, K), 0xAA, np.uint8)
    amax = np.zeros(1, np.float32)
    f = oracle().or_quantize_blockscaled
    f.argtypes, f.restype = [C.c_int, _P, _I64, _I64, _I64, _P, _P, _P], None
    f(mode, _ptr(x), ldx, rows, K, _ptr(q), _ptr(sf), _ptr(amax))
    return q, sf, float(amax[0])


def dequantize_blockscaled(mode, q, sf, amax, rows, K):
    out = np.empty((rows, K), np.float32)
    f = oracle().or_dequantize_blockscaled
    f.argtypes, f.restype = [C.c_int, _P, _P, _F, _I64, _I64, _P], None
    f(mode, _ptr(q), _ptr(sf), amax, rows, K, _ptr(out))
    return out


def qwen_latent_encode(x, mean, std):
    """x: fp32 [64, n] -> [n, 64]."""
    x = np.ascontiguousarray(x, np.float32)
    n = x.shape[1]
    y = np.empty((n, 64), np.float32)
    f = oracle().or_qwen_latent_encode
    f.argtypes, f.restype = [_P, _P, _I64, _P, _P], None
    f(_ptr(x), _ptr(y), n, _ptr(np.ascontiguousarray(mean, np.float32)), _ptr(np.ascontiguousarray(std, np.float32)))
    return y


def qwen_latent_decode(x, mean, std):
    """x: fp32 [n, 64] -> [64, n]."""
    x = np.ascontiguousarray(x, np.float32)
    n = x.shape[0]
    y = np.empty((64, n), np.float32)
    f = oracle().or_qwen_latent_decode
    f.argtypes, f.restype = [_P, _P, _I64, _P, _P], None
    f(_ptr(x), _ptr(y), n, _ptr(np.ascontiguousarray(mean, np.float32)), _ptr(np.ascontiguousarray(std, np.float32)))
    return y


def h3_latent_video(rows, F, H, W):
    rows = np.ascontiguousarray(rows, np.float32)
    z = np.empty((24, F, H, W), np.float32)
    f = oracle().or_h3_latent_video
    f.argtypes, f.restype = [_P, _P, _I64, _I64, _I64], None
    f(_ptr(rows), _ptr(z), F, H, W)
    return z


def h3_latent_audio(rows, A):
    rows = np.ascontiguousarray(rows, np.float32)
    z = np.empty((2, 32, A), np.float32)
    f = oracle().or_h3_latent_audio
    f.argtypes, f.restype = [_P, _P, _I64], None
    f(_ptr(rows), _ptr(z), A)
    return z
