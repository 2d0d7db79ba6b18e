"""The CPU oracle's block-scale quantiser: pinned against byte outputs of the REFERENCE's kernel
(tests/golden/ref_blockscale_sm100a.npz: src/kernels/blockscale.cu built unmodified for sm_100a and run
on a B200 over tests/golden/ref_blockscale_cases.py), plus the properties the reference's own test
checks on decoded values (tests/blockscale_test.cpp:83-105)."""
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import binding as orc

GOLD = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLD))
import ref_blockscale_cases  # noqa: E402

CASES = ref_blockscale_cases.cases()
GOLDEN = GOLD / "ref_blockscale_sm100a.npz"
# relative RMS error bounds of the reference's test (tests/blockscale_test.cpp:99-100)
ELEM_ERR = {1: 0.04, 2: 0.12}


def bits_to_f32(b):
    return (np.asarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def rel_rms(got, want):
    num = np.sqrt(np.mean((got.astype(np.float64) - want.astype(np.float64)) ** 2))
    den = np.sqrt(np.mean(want.astype(np.float64) ** 2))
    return num / den if den > 0 else num


def test_e4m3_codes_round_trip_and_order():
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8)
    vals = orc.e4m3_to_f32(codes)
    back = orc.f32_to_e4m3(vals)
    assert np.array_equal(back, codes)
    pos = orc.e4m3_to_f32(np.arange(0, 0x7F, dtype=np.uint8))
    assert np.all(np.diff(pos) > 0) and pos[-1] == 448.0 and pos[1] == 2.0 ** -9 and pos[8] == 2.0 ** -6


def test_e4m3_rounds_to_nearest_even_and_saturates():
    pos = orc.e4m3_to_f32(np.arange(0, 0x7F, dtype=np.uint8)).astype(np.float64)
    mid = (pos[:-1] + pos[1:]) / 2  # exact in fp32
    got = orc.f32_to_e4m3(mid.astype(np.float32))
    want = np.array([c if c % 2 == 0 else c + 1 for c in range(0x7E)], np.uint8)
    assert np.array_equal(got, want)
    below = np.nextafter(mid.astype(np.float32), np.float32(0))
    above = np.nextafter(mid.astype(np.float32), np.float32(1e9))
    assert np.array_equal(orc.f32_to_e4m3(below), np.arange(0x7E, dtype=np.uint8))
    assert np.array_equal(orc.f32_to_e4m3(above), np.arange(1, 0x7F, dtype=np.uint8))
    edge = np.array([448.0, 463.9, 464.0, 1e6, 3e38, np.inf, -500.0, -np.inf, -0.0, 2.0 ** -11, 2.0 ** -10 * 1.01], np.float32)
    assert list(orc.f32_to_e4m3(edge)) == [0x7E, 0x7E, 0x7E, 0x7E, 0x7E, 0x7E, 0xFE, 0xFE, 0x80, 0x00, 0x01]


@pytest.mark.parametrize("mode", [1, 2])
def test_scale_layout_is_a_padded_permutation(mode):
    V = 32 if mode == 1 else 16
    for rows, K in ((1, 32), (130, 384), (300, 160), (128, 4 * V), (129, 5 * V)):
        nb = K // V
        nkb_pad = (nb + 3) // 4 * 4
        total = orc.qscale_bytes(mode, rows, K)
        assert total == (rows + 127) // 128 * 128 * nkb_pad
        offs = np.array([[orc.sf_offset(r, kb, nkb_pad) for kb in range(nb)] for r in range(rows)])
        assert offs.min() >= 0 and offs.max() < total and np.unique(offs).size == offs.size
        # one 128 x 4 tile is 512 contiguous bytes: row r, column c at (r % 32) * 16 + (r / 32) * 4 + c
        assert orc.sf_offset(0, 0, nkb_pad) == 0 and orc.sf_offset(1, 0, nkb_pad) == 16
        assert orc.sf_offset(32 % rows if rows > 32 else 0, 0, nkb_pad) in (0, 4)


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_quantiser_properties(name):
    c = CASES[name]
    mode, K = c["mode"], c["K"]
    rows = c["x"].shape[0]
    q, sf, amax = orc.quantize_blockscaled(mode, c["x"], K)
    x = bits_to_f32(c["x"][:, :K])
    V = 32 if mode == 1 else 16
    nkb_pad = (K // V + 3) // 4 * 4
    used = np.zeros(sf.size, bool)
    for r in range(rows):
        for kb in range(K // V):
            used[orc.sf_offset(r, kb, nkb_pad)] = True
    assert not sf[~used].any(), "padding of the scale buffer must be cleared"
    if mode == 2:
        assert amax == np.abs(x).max()
    if name in ("mx_every_bf16", "mx_every_bf16_shuffled"):
        return  # decoded values reach 2^128
    d = orc.dequantize_blockscaled(mode, q, sf, amax, rows, K)
    if name.endswith("_wide") or name.endswith("tiny") or name.endswith("huge"):
        assert rel_rms(d, x) < ELEM_ERR[mode]
        return
    assert rel_rms(d, x) < ELEM_ERR[mode]
    if mode == 1:  # per element: within half an e4m3 step of the block scale, or saturating nothing
        scale = np.repeat(np.abs(x).reshape(rows, K // 32, 32).max(-1), 32, axis=1).reshape(rows, K)
        assert np.all(np.abs(d - x) <= scale * 2.0 ** -4 + 1e-30)


def test_oracle_quantiser_matches_reference_test_bounds_on_activation_like_input():
    """The reference's own test input shape and distribution (tests/blockscale_test.cpp:60-71: M = 200
    rows, K = 192, values around +-2 with a few outliers), seeded here."""
    g = np.random.default_rng(7)
    a = g.uniform(-2.0, 2.0, (200, 192)).astype(np.float32)
    a[g.uniform(size=a.shape) < 0.01] *= 8.0
    bits = orc.f32_to_bf16_bits(a)
    x = bits_to_f32(bits)
    for mode in (1, 2):
        q, sf, amax = orc.quantize_blockscaled(mode, bits)
        d = orc.dequantize_blockscaled(mode, q, sf, amax, 200, 192)
        assert rel_rms(d, x) < ELEM_ERR[mode]


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_reference_kernel_bytes(name):
    gold = np.load(GOLDEN)
    c = CASES[name]
    q, sf, amax = orc.quantize_blockscaled(c["mode"], c["x"], c["K"])
    assert np.array_equal(sf, gold[name + ".sf"]), f"{name}: scale bytes differ"
    assert np.array_equal(q, gold[name + ".q"]), f"{name}: {(q != gold[name + '.q']).sum()} data bytes differ"
    if c["mode"] == 2:
        assert np.float32(amax) == gold[name + ".amax"][0]
