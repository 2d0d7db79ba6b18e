"""Generates tests/golden/ref_ops_sm100a.npz: outputs of the REFERENCE's own kernels.

Runs src/kernels/ops.cu of the reference - compiled unmodified for sm_100a into
oracle/_ref/libmx_ref_ops.so by oracle/Makefile - on the seeded cases of ref_cases.py.  Needs a
B200 and that library (built where the reference tree is present):

    python tests/golden/make_ref_kernel_golden.py [out.npz]
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))
from oracle import binding as orc  # noqa: E402
import ref_cases  # noqa: E402


class RM(C.Structure):
    _fields_ = [("target", C.c_void_p), ("prefix", C.c_void_p), ("prefix_len", C.c_int64)]


def dev(a):
    if a is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t.view(torch.bfloat16) if a.dtype == np.uint16 else t).cuda()


def host(t):
    return (t.view(torch.uint16) if t.dtype == torch.bfloat16 else t).cpu().numpy()


def ptr(t):
    return None if t is None else t.data_ptr()


def run_case(L, c):
    """Runs one case through the reference's launcher; returns the output array."""
    P, I64, I, F = C.c_void_p, C.c_int64, C.c_int, C.c_float
    op = c["op"]
    keep = []

    def rm(t, p, plen):
        td, pd = dev(t), dev(p)
        keep.extend([td, pd])
        return RM(ptr(td), ptr(pd), plen)

    none = RM(None, None, 0)
    if op in ("layernorm_mod", "rmsnorm_mod"):
        x = dev(c["x"])
        rows, dim = c["x"].shape
        out = torch.zeros((rows, dim), dtype=torch.bfloat16, device="cuda")
        sc, sh = rm(c["sc_t"], c["sc_p"], c["plen"]), rm(c["sh_t"], c["sh_p"], c["plen"])
        if op == "layernorm_mod":
            L.ref_layernorm_mod.argtypes = [P, I64, I64, F, RM, RM, P, P]
            rc = L.ref_layernorm_mod(ptr(x), rows, dim, c["eps"], sc, sh, ptr(out), None)
        else:
            w = dev(c["w"])
            L.ref_rmsnorm_mod.argtypes = [P, I64, I64, F, P, RM, RM, P, P]
            rc = L.ref_rmsnorm_mod(ptr(x), rows, dim, c["eps"], ptr(w), sc, sh, ptr(out), None)
    elif op == "rmsnorm_bf16":
        x, w = dev(c["x"]), dev(c["w"])
        rows, dim = c["x"].shape
        out = torch.zeros((rows, dim), dtype=torch.bfloat16, device="cuda")
        L.ref_rmsnorm_bf16.argtypes = [P, I64, I64, F, P, P, P]
        rc = L.ref_rmsnorm_bf16(ptr(x), rows, dim, c["eps"], ptr(w), ptr(out), None)
    elif op == "head_norm_rope":
        inp, w, cs, sn = dev(c["inp"]), dev(c["w"]), dev(c["cos"]), dev(c["sin"])
        out = torch.zeros((c["S"], c["H"], c["D"]), dtype=torch.bfloat16, device="cuda")
        L.ref_head_norm_rope.argtypes = [P, I64, I64, I64, I, I, P, F, P, P, I, I, P, P]
        rc = L.ref_head_norm_rope(ptr(inp), c["S"], c["stride"], c["col0"], c["H"], c["D"], ptr(w), c["eps"], ptr(cs), ptr(sn),
                                  c["rot"], c["mode"], ptr(out), None)
    elif op == "gated_residual":
        out, y = dev(c["x"]), dev(c["y"])
        rows, dim = c["x"].shape
        L.ref_gated_residual.argtypes = [P, P, I64, I64, RM, I, P]
        rc = L.ref_gated_residual(ptr(out), ptr(y), rows, dim, rm(c["g_t"], c["g_p"], c["plen"]), c["tanh"], None)
    elif op == "silu_mul":
        gu = dev(c["gu"])
        rows = c["gu"].shape[0]
        out = torch.zeros((rows, c["F"]), dtype=torch.bfloat16, device="cuda")
        L.ref_silu_mul.argtypes = [P, I64, I64, P, P]
        rc = L.ref_silu_mul(ptr(gu), rows, c["F"], ptr(out), None)
    elif op in ("gelu_tanh_inplace", "gelu_erf_inplace", "silu_inplace_f32"):
        out = dev(c["x"])
        f = getattr(L, "ref_" + op)
        f.argtypes = [P, I64, P]
        rc = f(ptr(out), out.numel(), None)
    elif op == "add_bias_bf16":
        out, b = dev(c["y"]), dev(c["bias"])
        L.ref_add_bias_bf16.argtypes = [P, P, I64, I64, P]
        rc = L.ref_add_bias_bf16(ptr(out), ptr(b), c["y"].shape[0], c["y"].shape[1], None)
    elif op == "axpby_f32":
        out, y = dev(c["x"]), dev(c["y"])
        L.ref_axpby_f32.argtypes = [P, P, F, F, I64, P]
        rc = L.ref_axpby_f32(ptr(out), ptr(y), c["a"], c["b"], out.numel(), None)
    else:
        raise KeyError(op)
    torch.cuda.synchronize()
    if rc:
        raise RuntimeError(L.ref_last_error().decode())
    return host(out)


if __name__ == "__main__":
    L = orc.ref_ops()
    outs = {name: run_case(L, c) for name, c in ref_cases.cases().items()}
    dst = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).with_name("ref_ops_sm100a.npz")
    np.savez_compressed(dst, **outs)
    print("wrote", dst, {k: v.shape for k, v in outs.items()})
