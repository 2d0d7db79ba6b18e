"""libmxk against the REFERENCE's own kernels: replayed on the golden cases (outputs of
src/kernels/ops.cu built for sm_100a, tests/golden/ref_ops_sm100a.npz) and, where
oracle/_ref/libmx_ref_ops.so travelled with the tree, run side by side on the same device buffers."""
import sys
from pathlib import Path

import numpy as np
import pytest

import helpers as H
from oracle import binding as orc

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLD))
import ref_cases  # noqa: E402
from test_cpu_golden_ref import EXACT, compare  # noqa: E402

CASES = ref_cases.cases()


@pytest.fixture(scope="module")
def mx():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import miroxen_b200 as m
    m.lib()
    return m


def mxk_run(mx, c):
    op = c["op"]
    d = lambda a: None if a is None else H.to_dev(torch, a)
    host = lambda t: (t.view(torch.uint16) if t.dtype == torch.bfloat16 else t).cpu().numpy()
    keep = []

    def rm(t, p, plen):
        td, pd = d(t), d(p)
        keep.extend([td, pd])
        return mx.row_mod(td, pd, plen)

    if op in ("layernorm_mod", "rmsnorm_mod"):
        rows, dim = c["x"].shape
        out = torch.zeros((rows, dim), dtype=torch.bfloat16, device="cuda")
        sc, sh = rm(c["sc_t"], c["sc_p"], c["plen"]), rm(c["sh_t"], c["sh_p"], c["plen"])
        if op == "layernorm_mod":
            mx.layernorm_mod(d(c["x"]), rows, dim, c["eps"], sc, sh, out)
        else:
            mx.rmsnorm_mod(d(c["x"]), rows, dim, c["eps"], d(c["w"]), sc, sh, out)
    elif op == "rmsnorm_bf16":
        rows, dim = c["x"].shape
        out = torch.zeros((rows, dim), dtype=torch.bfloat16, device="cuda")
        mx.rmsnorm_bf16(d(c["x"]), rows, dim, c["eps"], d(c["w"]), out)
    elif op == "head_norm_rope":
        out = torch.zeros((c["S"], c["H"], c["D"]), dtype=torch.bfloat16, device="cuda")
        mx.head_norm_rope(d(c["inp"]), c["S"], c["stride"], c["col0"], c["H"], c["D"], d(c["w"]), c["eps"], d(c["cos"]),
                          d(c["sin"]), c["rot"], c["mode"], out)
    elif op == "gated_residual":
        out = d(c["x"])
        mx.gated_residual(out, d(c["y"]), c["x"].shape[0], c["x"].shape[1], rm(c["g_t"], c["g_p"], c["plen"]), c["tanh"])
    elif op == "silu_mul":
        out = torch.zeros((c["gu"].shape[0], c["F"]), dtype=torch.bfloat16, device="cuda")
        mx.silu_mul(d(c["gu"]), c["gu"].shape[0], c["F"], out)
    elif op in ("gelu_tanh_inplace", "gelu_erf_inplace", "silu_inplace_f32"):
        out = d(c["x"])
        getattr(mx, op)(out, out.numel())
    elif op == "add_bias_bf16":
        out = d(c["y"])
        mx.add_bias_bf16(out, d(c["bias"]), c["y"].shape[0], c["y"].shape[1])
    elif op == "axpby_f32":
        out = d(c["x"])
        mx.axpby_f32(out, d(c["y"]), c["a"], c["b"], out.numel())
    else:
        raise KeyError(op)
    torch.cuda.synchronize()
    return host(out)


@pytest.mark.parametrize("name", sorted(CASES))
def test_libmxk_matches_reference_kernel_output(mx, name):
    gold = np.load(GOLD / "ref_ops_sm100a.npz")
    compare(name, mxk_run(mx, CASES[name]), gold[name])


@pytest.mark.skipif(not orc.have_ref_ops(), reason="oracle/_ref/libmx_ref_ops.so not present (built from the reference tree)")
@pytest.mark.parametrize("name", sorted(CASES))
def test_reference_kernels_side_by_side(mx, name):
    """Runs the reference's kernels here and now: they must reproduce the committed fixture bit for bit
    (same binary, same inputs) and agree with libmxk and the oracle within the tolerance."""
    from make_ref_kernel_golden import run_case
    ref = run_case(orc.ref_ops(), CASES[name])
    gold = np.load(GOLD / "ref_ops_sm100a.npz")
    assert np.array_equal(ref, gold[name]), f"{name}: reference kernels no longer reproduce the fixture"
    compare(name, mxk_run(mx, CASES[name]), ref)
