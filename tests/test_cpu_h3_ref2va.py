"""Rotary positions of the reference-conditioned MiniMax-H3 layout: the CPU oracle and the library's host-side
plan (per-axis position lists + run descriptors) against positions produced by the REFERENCE's own host code
(tests/golden/h3_ref2va_positions.npz, generator tests/golden/make_h3_ref2va_positions.py)."""
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import binding as orc

GOLD = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLD))
from make_h3_ref2va_positions import CASES  # noqa: E402


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_positions_match_reference_fixture(name):
    gold = np.load(GOLD / "h3_ref2va_positions.npz")[name]
    assert same_bits(orc.h3_ref2va_positions(*CASES[name]), gold)


@pytest.mark.skipif(not orc.have_ref_layout(), reason="oracle/_ref/libmx_ref_layout.so not built (needs the reference tree)")
def test_oracle_positions_match_reference_code_on_random_requests():
    g = np.random.default_rng(12)
    for _ in range(40):
        refs = []
        for _ in range(int(g.integers(0, 5))):
            kind = ["image", "video", "audio"][int(g.integers(0, 3))]
            r = dict(kind=kind, h=2 * int(g.integers(1, 9)), w=2 * int(g.integers(1, 9)), frames=int(g.integers(1, 14)),
                     audio=int(g.integers(1, 30)) if kind == "audio" else int(g.integers(0, 30)))
            refs.append(r)
        args = (int(g.integers(0, 40)), refs, int(g.integers(1, 12)), 2 * int(g.integers(1, 9)), 2 * int(g.integers(1, 9)),
                int(g.integers(1, 25)))
        assert same_bits(orc.h3_ref2va_positions(*args), orc.h3_ref2va_positions(*args, use_reference=True))


@pytest.mark.parametrize("name", sorted(CASES))
def test_library_plan_describes_the_same_positions(name):
    """Host-only: the plan's lists come from libmxk's host builders; no kernel runs."""
    from miroxen_b200 import rope_tables
    gold = np.load(GOLD / "h3_ref2va_positions.npz")[name]
    t_list, h_list, w_list, runs, S = rope_tables.h3_ref2va_plan(*CASES[name])
    assert S == gold.shape[0]
    covered = np.zeros(S, np.int32)
    for r in runs:
        covered[r.row0:r.row0 + r.n0 * r.n1 * r.n2] += 1
    assert (covered == 1).all(), "runs must tile the rows exactly once"
    assert same_bits(rope_tables.positions_from_plan(t_list, h_list, w_list, runs, S), gold)


def test_library_plan_rejects_bad_requests():
    from miroxen_b200 import rope_tables
    with pytest.raises(ValueError):
        rope_tables.h3_ref2va_plan(4, [], 2, 5, 6, 1)
    with pytest.raises(ValueError):
        rope_tables.h3_ref2va_plan(4, [dict(kind="audio", audio=0)], 2, 4, 6, 1)
    with pytest.raises(ValueError):
        rope_tables.h3_ref2va_plan(4, [dict(kind="image", h=3, w=4)], 2, 4, 6, 1)
    with pytest.raises(ValueError):
        rope_tables.h3_ref2va_plan(4, [dict(kind="clip", h=4, w=4)], 2, 4, 6, 1)
