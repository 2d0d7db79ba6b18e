"""Pins the CPU oracle against outputs of the REFERENCE's own kernels: tests/golden/ref_ops_sm100a.npz
holds what src/kernels/ops.cu (compiled unmodified for sm_100a) produced on a B200 for the seeded
cases of tests/golden/ref_cases.py (generator: tests/golden/make_ref_kernel_golden.py)."""
import sys
from pathlib import Path

import numpy as np
import pytest

import helpers as H
from oracle import binding as orc

GOLD = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLD))
import ref_cases  # noqa: E402

CASES = ref_cases.cases()
EXACT = {"rope_copy", "bias_bf16"}


def oracle_run(c):
    op = c["op"]
    if op == "layernorm_mod":
        return orc.layernorm_mod(c["x"], c["eps"], orc.mod(c["sc_t"], c["sc_p"], c["plen"]), orc.mod(c["sh_t"], c["sh_p"], c["plen"]))
    if op == "rmsnorm_mod":
        return orc.rmsnorm_mod(c["x"], c["eps"], c["w"], orc.mod(c["sc_t"], c["sc_p"], c["plen"]), orc.mod(c["sh_t"], c["sh_p"], c["plen"]))
    if op == "rmsnorm_bf16":
        return orc.rmsnorm_bf16(c["x"], c["eps"], c["w"])
    if op == "head_norm_rope":
        return orc.head_norm_rope(c["inp"], c["S"], c["stride"], c["col0"], c["H"], c["D"], c["w"], c["eps"], c["cos"], c["sin"],
                                  c["rot"], c["mode"])
    if op == "gated_residual":
        return orc.gated_residual(c["x"].copy(), c["y"], orc.mod(c["g_t"], c["g_p"], c["plen"]), c["tanh"])
    if op == "silu_mul":
        return orc.silu_mul(c["gu"], c["F"])
    if op == "gelu_tanh_inplace":
        return orc.gelu_tanh_inplace(c["x"].copy())
    if op == "gelu_erf_inplace":
        return orc.gelu_erf_inplace(c["x"].copy())
    if op == "silu_inplace_f32":
        return orc.silu_inplace_f32(c["x"].copy())
    if op == "add_bias_bf16":
        return orc.add_bias_bf16(c["y"].copy(), c["bias"])
    if op == "axpby_f32":
        return orc.axpby_f32(c["x"].copy(), c["y"], c["a"], c["b"])
    raise KeyError(op)


def compare(name, got, want):
    assert got.shape == want.shape
    if name in EXACT:
        assert np.array_equal(got, want), name
    elif want.dtype == np.uint16:
        H.assert_bf16_close(got, want, name)
    else:
        H.assert_f32_close(got, want, name, rel=2.0 ** -18)


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_reference_kernel_output(name):
    gold = np.load(GOLD / "ref_ops_sm100a.npz")
    assert set(gold.files) == set(CASES)
    compare(name, oracle_run(CASES[name]), gold[name])
