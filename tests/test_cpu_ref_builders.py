"""The host-side table and embedding builders, pinned against the reference's own statements.

tests/golden/ref_builders.npz was produced by running the reference's statements themselves
(QwenImageDit::prepare / time_mod, H3Dit::time_basis / prepare, cut out of its model files and
compiled by oracle/Makefile) on the cases of tests/golden/ref_builder_cases.py.  Here the CPU oracle
must reproduce those bits exactly; where the reference's statements were built in this checkout
they also run side by side on random cases; and the library's host-side timestep embedding is held
to the same bits (its device-side builders are checked against the fixture in the GPU tests)."""
import hashlib
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import binding as orc

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import ref_builder_cases as cases  # noqa: E402

GOLD = np.load(Path(__file__).resolve().parent / "golden" / "ref_builders.npz")


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest(), np.uint8)


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))


@pytest.mark.parametrize("i", range(len(cases.QWEN_ROPE_FULL)))
def test_oracle_qwen_rope_table_equals_the_reference_small(i):
    T, H, W, conds = cases.QWEN_ROPE_FULL[i]
    cos, sin = orc.qwen_rope_table(orc.qwen_segs(T, H, W, conds))
    assert same_bits(cos, GOLD[f"qwen_rope_full{i}_cos"]) and same_bits(sin, GOLD[f"qwen_rope_full{i}_sin"])


@pytest.mark.parametrize("i", range(len(cases.QWEN_ROPE_DIGEST)))
def test_oracle_qwen_rope_table_equals_the_reference_at_benchmark_sizes(i):
    T, H, W, conds = cases.QWEN_ROPE_DIGEST[i]
    cos, sin = orc.qwen_rope_table(orc.qwen_segs(T, H, W, conds))
    assert cos.shape[0] == int(GOLD[f"qwen_rope_digest{i}_rows"][0])
    assert np.array_equal(digest(cos, sin), GOLD[f"qwen_rope_digest{i}"])


def test_oracle_timestep_embedding_equals_the_reference():
    got = np.stack([orc.qwen_timestep_embedding(float(t)) for t in cases.TIMESTEPS_FULL])
    assert same_bits(got, GOLD["timestep_full"])
    assert np.array_equal(digest(*[orc.qwen_timestep_embedding(float(t)) for t in cases.timesteps_digest()]), GOLD["timestep_digest"])


def test_library_host_timestep_embedding_equals_the_reference():
    """mxk_qwen_timestep_embedding_host is plain host code: it runs without a GPU."""
    import ctypes as C
    from miroxen_b200 import _lib, build
    if not _lib.lib_path().exists():
        build.build()
    f = _lib.lib().mxk_qwen_timestep_embedding_host

    def emb(t):
        out = np.empty((2, 256), np.float32)
        assert f(C.c_float(t), out.ctypes.data) == 0
        return out
    assert same_bits(np.stack([emb(float(t)) for t in cases.TIMESTEPS_FULL]), GOLD["timestep_full"])
    assert np.array_equal(digest(*[emb(float(t)) for t in cases.timesteps_digest()]), GOLD["timestep_digest"])


def test_oracle_h3_time_basis_equals_the_reference():
    table, ts, small = cases.h3_basis_inputs()
    assert same_bits(orc.h3_time_basis(ts, table), GOLD["h3_basis"])
    assert same_bits(orc.h3_time_basis(ts, small), GOLD["h3_basis_small"])


def test_oracle_h3_rope_table_equals_the_reference():
    invf = cases.h3_inv_freq()
    for name, pos in cases.h3_rope_positions():
        cos, sin = orc.h3_rope_table(pos, invf)
        assert np.array_equal(digest(cos, sin), GOLD[f"h3_rope_{name}_digest"]), name
        if pos.shape[0] <= 64:
            assert same_bits(cos, GOLD[f"h3_rope_{name}_cos"]) and same_bits(sin, GOLD[f"h3_rope_{name}_sin"])


@pytest.mark.skipif(not orc.have_ref_builders(), reason="oracle/_ref/libmx_ref_builders.so not built (needs the reference tree)")
def test_oracle_against_the_reference_statements_on_random_cases():
    g = np.random.default_rng(2024)
    for _ in range(25):
        H, W = 2 * int(g.integers(1, 20)), 2 * int(g.integers(1, 20))
        conds, cur = [], 0
        for _ in range(int(g.integers(0, 3))):
            h, w = 2 * int(g.integers(1, 8)), 2 * int(g.integers(1, 8))
            slot0 = cur + int(g.integers(0, 9))
            conds.append((slot0, h, w))
            cur = slot0 + h * w // 4
        T = cur + int(g.integers(0, 40))
        rc, rs = orc.ref_qwen_rope_table(T, H, W, conds)
        oc, os_ = orc.qwen_rope_table(orc.qwen_segs(T, H, W, conds))
        assert same_bits(rc, oc) and same_bits(rs, os_), (T, H, W, conds)
    for t in g.random(300, dtype=np.float32):
        assert same_bits(orc.ref_qwen_timestep_embedding(float(t)), orc.qwen_timestep_embedding(float(t))), t
    for _ in range(10):
        grid, basis = int(g.integers(2, 2000)), int(g.integers(1, 12))
        table = g.standard_normal((grid, basis)).astype(np.float32)
        ts = (g.random(64, dtype=np.float32) * np.float32(1.4) - np.float32(0.2)).astype(np.float32)
        assert same_bits(orc.ref_h3_time_basis(ts, table), orc.h3_time_basis(ts, table))
    for _ in range(10):
        S, nf = int(g.integers(1, 300)), int(g.integers(1, 24))
        pos = (g.random((S, 3), dtype=np.float32) * np.float32(60.0)).astype(np.float32)
        invf = (1.0 / np.power(np.float32(10000.0), g.random(nf, dtype=np.float32))).astype(np.float32)
        rc, rs = orc.ref_h3_rope_table(pos, invf)
        oc, os_ = orc.h3_rope_table(pos, invf)
        assert same_bits(rc, oc) and same_bits(rs, os_)


def test_the_reference_rejects_a_condition_image_that_overruns_the_text():
    if not orc.have_ref_builders():
        pytest.skip("oracle/_ref/libmx_ref_builders.so not built")
    with pytest.raises(RuntimeError):
        orc.ref_qwen_rope_table(10, 4, 4, [(8, 4, 4)])
