"""Pins the CPU oracle: against fixtures generated from the reference's own code (tests/golden/),
against the reference's host code directly where oracle/_ref is built, and against independent
float64 numpy statements of each formula."""
from pathlib import Path

import numpy as np
import pytest

import helpers as H
from oracle import binding as orc

GOLD = Path(__file__).resolve().parent / "golden"


def f64(bits):
    return orc.bf16_bits_to_f32(bits).astype(np.float64)


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.005859375, 1.01171875, -1.00390625, 3.0e38, 1e-40, 0.0, -0.0], np.float32)
    b = orc.f32_to_bf16(x)
    # 1 + 2^-8 is a tie -> even (1.0); 1 + 3*2^-9 rounds up; 1 + 3*2^-8 is a tie -> even (1 + 2^-6)
    assert list(b[:5]) == [0x3F80, 0x3F80, 0x3F81, 0x3F82, 0xBF80]
    assert np.array_equal(orc.f32_to_bf16_bits(x), b)
    back = orc.bf16_to_f32(b)
    assert back[0] == 1.0 and back[7] == 0.0


def test_h3_positions_match_reference_fixture():
    z = np.load(GOLD / "h3_positions.npz")
    n = len([k for k in z.files if k.endswith("_args")])
    assert n >= 5
    for i in range(n):
        args = z[f"case{i}_args"]
        T, F, Hh, W, A = (int(v) for v in args[:5])
        anchors = ["first" if v == 0 else "last" for v in args[5:]]
        pos = orc.h3_positions(T, F, Hh, W, A, anchors)
        assert np.array_equal(pos.view(np.uint32), z[f"case{i}_pos"].view(np.uint32)), f"case {i}"


@pytest.mark.skipif(not orc.have_ref_layout(), reason="oracle/_ref/libmx_ref_layout.so not built (needs the reference tree)")
def test_h3_positions_match_reference_code():
    for T, F, Hh, W, A, anchors in [(64, 9, 36, 64, 40, ["first", "last"]), (300, 21, 60, 104, 0, []), (1, 3, 8, 8, 1, ["first"])]:
        a = orc.h3_positions(T, F, Hh, W, A, anchors)
        b = orc.h3_positions(T, F, Hh, W, A, anchors, use_reference=True)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("rows,dim", [(4, 3072), (3, 100), (2, 5376)])
def test_norms_against_float64(rows, dim):
    g = H.rng(dim)
    x = H.normal_f32(g, (rows, dim), 1.0, 0.5)
    w = H.normal_f32(g, dim, 0.1, 1.0)
    sc_t, sc_p, sh = H.normal_f32(g, dim, 0.3), H.normal_f32(g, dim, 0.3), H.normal_f32(g, dim, 0.3)
    plen = 1
    xd = x.astype(np.float64)
    scale = np.where(np.arange(rows)[:, None] < plen, sc_p, sc_t).astype(np.float64)
    ln = (xd - xd.mean(1, keepdims=True)) / np.sqrt(xd.var(1, keepdims=True) + 1e-6) * (1 + scale) + sh
    got = orc.layernorm_mod(x, 1e-6, orc.mod(sc_t, sc_p, plen), orc.mod(sh))
    H.assert_bf16_close(got, orc.f32_to_bf16_bits(ln.astype(np.float32)), "layernorm_mod vs float64")
    rms = xd / np.sqrt((xd * xd).mean(1, keepdims=True) + 1e-5) * w * (1 + scale) + sh
    got = orc.rmsnorm_mod(x, 1e-5, w, orc.mod(sc_t, sc_p, plen), orc.mod(sh))
    H.assert_bf16_close(got, orc.f32_to_bf16_bits(rms.astype(np.float32)), "rmsnorm_mod vs float64")
    xb = orc.f32_to_bf16_bits(x)
    xbd = f64(xb)
    rms2 = xbd / np.sqrt((xbd * xbd).mean(1, keepdims=True) + 1e-6) * w
    H.assert_bf16_close(orc.rmsnorm_bf16(xb, 1e-6, w), orc.f32_to_bf16_bits(rms2.astype(np.float32)), "rmsnorm_bf16")


@pytest.mark.parametrize("mode,rot,D", [(1, 128, 128), (2, 128, 128), (2, 96, 128), (2, 72, 72), (0, 0, 64)])
def test_head_norm_rope_against_float64(mode, rot, D):
    g = H.rng(mode + rot)
    S, Hh = 5, 3
    inp = H.normal_bf16(g, (S, Hh * D + 16))
    w = H.normal_f32(g, D, 0.05, 1.0)
    half = max(rot // 2, 1)
    ang = g.uniform(-3, 3, (S, half))
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    got = orc.head_norm_rope(inp, S, Hh * D + 16, 16, Hh, D, w, 1e-6, cos, sin, rot, mode)
    v = f64(inp)[:, 16:].reshape(S, Hh, D)
    v = v / np.sqrt((v * v).mean(-1, keepdims=True) + 1e-6) * w
    out = v.copy()
    c, s = cos.astype(np.float64)[:, None, :], sin.astype(np.float64)[:, None, :]
    if mode == 1:
        a, b = v[..., 0:rot:2], v[..., 1:rot:2]
        out[..., 0:rot:2], out[..., 1:rot:2] = a * c - b * s, a * s + b * c
    elif mode == 2:
        h = rot // 2
        a, b = v[..., :h], v[..., h:rot]
        out[..., :h], out[..., h:rot] = a * c - b * s, a * s + b * c
    H.assert_bf16_close(got, orc.f32_to_bf16_bits(out.astype(np.float32)), "head_norm_rope vs float64")
    with pytest.raises(ValueError):
        orc.head_norm_rope(inp, S, Hh * D + 16, 0, Hh, 7, None, 1e-6, cos, sin, 2, 1)


def test_residual_and_activations_against_float64():
    g = H.rng(1)
    rows, dim, F = 6, 256, 384
    x, y = H.normal_f32(g, (rows, dim)), H.normal_bf16(g, (rows, dim))
    gt, gp = H.normal_f32(g, dim), H.normal_f32(g, dim)
    gate = np.where(np.arange(rows)[:, None] < 2, gp, gt).astype(np.float64)
    H.assert_f32_close(orc.gated_residual(x.copy(), y, orc.mod(gt, gp, 2), 1), x + np.tanh(gate) * f64(y), "tanh gate")
    H.assert_f32_close(orc.gated_residual(x.copy(), y, orc.mod(gt, gp, 2), 0), x + gate * f64(y), "plain gate")
    H.assert_f32_close(orc.gated_residual(x.copy(), y), x + f64(y), "no gate")
    gu = H.normal_bf16(g, (rows, 2 * F), 2.0)
    gd = f64(gu)
    ref = gd[:, :F] / (1 + np.exp(-gd[:, :F])) * gd[:, F:]
    H.assert_bf16_close(orc.silu_mul(gu, F), orc.f32_to_bf16_bits(ref.astype(np.float32)), "silu_mul")
    v = H.normal_bf16(g, 5000, 2.0)
    vd = f64(v)
    ref = 0.5 * vd * (1 + np.tanh(0.7978845608 * (vd + 0.044715 * vd ** 3)))
    H.assert_bf16_close(orc.gelu_tanh_inplace(v.copy()), orc.f32_to_bf16_bits(ref.astype(np.float32)), "gelu_tanh")
    from math import erf
    ref = np.array([0.5 * t * (1 + erf(t / np.sqrt(2))) for t in vd])
    H.assert_bf16_close(orc.gelu_erf_inplace(v.copy()), orc.f32_to_bf16_bits(ref.astype(np.float32)), "gelu_erf")


def _libm():
    import ctypes
    m = ctypes.CDLL("libm.so.6")
    for f in (m.cosf, m.sinf):
        f.argtypes, f.restype = [ctypes.c_float], ctypes.c_float
    return (lambda v: np.float32(m.cosf(float(np.float32(v))))), (lambda v: np.float32(m.sinf(float(np.float32(v)))))


def test_qwen_rope_table_layout():
    """Closed-form spot checks of the MSRoPE layout rules (src/models/qwen_image/dit.cpp:151-185),
    with libm's own cosf / sinf as the yardstick (numpy's float32 routines are a different algorithm)."""
    cosf, sinf = _libm()
    segs = [("text", 5), ("image", 4, 6), ("text", 2), ("image", 8, 8)]
    cos, sin = orc.qwen_rope_table(segs)
    assert cos.shape == (5 + 24 + 2 + 64, 64)
    # pair 0 of every axis has frequency 1: the angle is the position itself
    for k in range(5):  # text rows: all three axes at position k
        for p in (0, 8, 36):
            assert cos[k, p] == cosf(k) and sin[k, p] == sinf(k)
    # first image: frame axis at position 5; h = r - 2, w = col - 3
    r, c = 3, 1
    row = 5 + r * 6 + c
    assert cos[row, 0] == cosf(5) and cos[row, 8] == cosf(r - 2) and sin[row, 36] == sinf(c - 3)
    # the image advances the position by max(4, 6): the next text row sits at 11
    assert cos[29, 0] == cosf(11) and cos[30, 36] == cosf(12)
    # target image at frame 13, centred: row 0 has h = -4, w = -4
    assert cos[31, 0] == cosf(13) and sin[31, 8] == sinf(-4)
    # a higher pair uses invf = 1 / 10000^(2j/axis) evaluated in fp32
    invf = 1.0 / (10000.0 ** (2 * 3 / 56.0))
    assert abs(float(cos[31, 8 + 3]) - np.cos(-4 * invf)) < 1e-6


def test_timestep_embedding_and_time_basis():
    e = orc.qwen_timestep_embedding(0.5)
    assert e.shape == (2, 256)
    assert np.all(e[1, :128] == 1.0) and np.all(e[1, 128:] == 0.0)  # t = 0 row: cos 0, sin 0
    ts = np.float32(500.0)  # bf16(0.5) * 1000
    cosf, _ = _libm()
    assert e[0, 0] == orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(np.array([cosf(ts)], np.float32)))[0]
    assert np.array_equal(orc.f32_to_bf16_bits(e), orc.f32_to_bf16_bits(orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(e))))
    table = np.arange(1025 * 8, dtype=np.float32).reshape(1025, 8)
    out = orc.h3_time_basis(np.array([0.0, 1.0, 0.5, 2.0, -1.0], np.float32), table)
    assert np.array_equal(out[0], table[0]) and np.array_equal(out[1], table[1024]) and np.array_equal(out[2], table[512])
    assert np.array_equal(out[3], table[1024]) and np.array_equal(out[4], table[0])


def test_oracle_threads_do_not_change_results():
    g = H.rng(4)
    x = H.normal_f32(g, (37, 3072))
    sc = H.normal_f32(g, 3072, 0.3)
    orc.set_threads(1)
    a = orc.layernorm_mod(x, 1e-6, orc.mod(sc), orc.NONE)
    orc.set_threads(4)
    b = orc.layernorm_mod(x, 1e-6, orc.mod(sc), orc.NONE)
    orc.set_threads(1)
    assert np.array_equal(a, b)
