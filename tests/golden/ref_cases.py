"""Seeded input cases shared by make_ref_kernel_golden.py (which runs the REFERENCE's kernels on them on
a GPU) and by the tests that replay them through the CPU oracle and through libmxk."""
import numpy as np


def _bf16(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def _n(g, shape, std=1.0, mean=0.0):
    return (g.standard_normal(shape, dtype=np.float32) * np.float32(std) + np.float32(mean)).astype(np.float32)


def all_finite_bf16():
    b = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    v = (b.astype(np.uint32) << 16).view(np.float32)
    return b[np.isfinite(v)]


def cases():
    """name -> dict(op=..., arrays and scalars).  Deterministic."""
    out = {}
    g = np.random.default_rng(20260)
    for name, rows, dim in (("ln_3072", 8, 3072), ("ln_100", 5, 100)):
        out[name] = dict(op="layernorm_mod", x=_n(g, (rows, dim), 1.0, 0.3), eps=1e-6, plen=3,
                         sc_t=_n(g, dim, 0.3), sc_p=_n(g, dim, 0.3), sh_t=_n(g, dim, 0.3), sh_p=_n(g, dim, 0.3))
    out["rms_5120"] = dict(op="rmsnorm_mod", x=_n(g, (5, 5120), 2.0), eps=1e-5, plen=2, w=_n(g, 5120, 0.1, 1.0),
                           sc_t=_n(g, 5120, 0.3), sc_p=_n(g, 5120, 0.3), sh_t=_n(g, 5120, 0.3), sh_p=_n(g, 5120, 0.3))
    out["rmsbf_1152"] = dict(op="rmsnorm_bf16", x=_bf16(_n(g, (4, 1152), 1.5)), eps=1e-6, w=_n(g, 1152, 0.1, 1.0))
    for name, S, Hh, D, rot, mode, stride, col0 in (("rope_il", 7, 24, 128, 128, 1, 3072, 0),
                                                    ("rope_half96", 5, 56, 128, 96, 2, 3 * 7168, 7168),
                                                    ("rope_d72", 6, 16, 72, 72, 2, 1152, 0),
                                                    ("rope_copy", 4, 40, 128, 0, 0, 3 * 5120, 10240)):
        half = max(rot // 2, 1)
        ang = g.uniform(-3.1, 3.1, (S, half))
        out[name] = dict(op="head_norm_rope", inp=_bf16(_n(g, (S, stride), 1.3)), S=S, stride=stride, col0=col0, H=Hh, D=D,
                         w=None if mode == 0 else _n(g, D, 0.05, 1.0), eps=1e-6, cos=np.cos(ang).astype(np.float32),
                         sin=np.sin(ang).astype(np.float32), rot=rot, mode=mode)
    out["res_tanh"] = dict(op="gated_residual", x=_n(g, (6, 3072)), y=_bf16(_n(g, (6, 3072))), g_t=_n(g, 3072, 0.7),
                           g_p=_n(g, 3072, 0.7), plen=4, tanh=1)
    out["res_plain"] = dict(op="gated_residual", x=_n(g, (3, 5376)), y=_bf16(_n(g, (3, 5376))), g_t=_n(g, 5376, 0.7),
                            g_p=_n(g, 5376, 0.7), plen=0, tanh=0)
    out["silu_mul"] = dict(op="silu_mul", gu=_bf16(_n(g, (4, 2 * 1536), 2.0)), F=1536)
    out["gelu_tanh_all"] = dict(op="gelu_tanh_inplace", x=all_finite_bf16())
    out["gelu_erf_all"] = dict(op="gelu_erf_inplace", x=all_finite_bf16())
    out["silu_f32"] = dict(op="silu_inplace_f32", x=_n(g, 6147, 3.0))
    out["bias_bf16"] = dict(op="add_bias_bf16", y=_bf16(_n(g, (5, 99))), bias=_n(g, 99))
    out["axpby"] = dict(op="axpby_f32", x=_n(g, 4099), y=_n(g, 4099), a=1.7, b=-0.6)
    return out
