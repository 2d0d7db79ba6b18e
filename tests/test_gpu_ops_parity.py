"""GPU parity: every libmxk op, called through the C ABI (ctypes), against the CPU oracle on the
same seeded inputs.  Shapes cover the benchmark configurations' widths (3072, 4096, 5120, 5376),
the vision tower's D = 72, ragged sizes that leave the vector paths, unaligned base pointers,
the prefix/target modulation switch and poisoned guard bands around every output."""
import numpy as np
import pytest

import helpers as H
from oracle import binding as orc

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["bulk_copy", "registers", "bulk_copy_wide_heads", "tile_heads"])
def mx(request):
    """Every test runs four times: with the bulk-copy (TMA) pipelined row / head kernels, which are the
    default; with the register-prefetch kernels that serve the shapes the bulk copies cannot; with the
    head pipeline's sixteen-channels-per-lane mapping (D = 128 shapes; the others fall to the default); and with
    the head kernel that reads straight from global memory, one group of tokens per CTA (D = 128 shapes)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import miroxen_b200 as m
    m.lib()  # raises if libmxk.so is missing - there is no fallback
    path = 2 if request.param == "registers" else 1
    m.set_tuning("norm_path", path)
    m.set_tuning("rope_path", 3 if request.param == "tile_heads" else path)
    m.set_tuning("rope_wide", 1 if request.param == "bulk_copy_wide_heads" else 0)
    yield m
    torch.cuda.synchronize()
    assert m.device_error() == 0, "a kernel's bounded wait ran out"
    m.set_tuning("norm_path", 0)
    m.set_tuning("rope_path", 0)
    m.set_tuning("rope_wide", 0)


def dev_mod(mx, keep, target=None, prefix=None, prefix_len=0):
    t = H.to_dev(torch, target) if target is not None else None
    p = H.to_dev(torch, prefix) if prefix is not None else None
    keep.extend([t, p])
    return mx.row_mod(t, p, prefix_len)


NORM_SHAPES = [(8, 3072), (129, 4096), (17, 5120), (33, 5376), (5, 1152), (3, 72), (7, 100), (7, 99), (1, 3072),
               (700, 3072), (2, 8192), (2, 9216)]


@pytest.mark.parametrize("rows,dim", NORM_SHAPES)
@pytest.mark.parametrize("variant", ["scale_shift_prefix", "scale_only", "plain"])
def test_layernorm_mod(mx, rows, dim, variant):
    g = H.rng(rows * 131 + dim)
    x = H.normal_f32(g, (rows, dim), std=1.0, mean=0.3)
    sc_t, sc_p = H.normal_f32(g, dim, 0.3), H.normal_f32(g, dim, 0.3)
    sh_t, sh_p = H.normal_f32(g, dim, 0.3), H.normal_f32(g, dim, 0.3)
    plen = rows // 3
    keep = []
    if variant == "scale_shift_prefix":
        o_sc, o_sh = orc.mod(sc_t, sc_p, plen), orc.mod(sh_t, sh_p, plen)
        d_sc, d_sh = dev_mod(mx, keep, sc_t, sc_p, plen), dev_mod(mx, keep, sh_t, sh_p, plen)
    elif variant == "scale_only":
        o_sc, o_sh = orc.mod(sc_t), orc.NONE
        d_sc, d_sh = dev_mod(mx, keep, sc_t), None
    else:
        o_sc = o_sh = orc.NONE
        d_sc = d_sh = None
    ref = orc.layernorm_mod(x, 1e-6, o_sc, o_sh)
    xd = H.to_dev(torch, x)
    out = H.Guarded(torch, (rows, dim), torch.bfloat16)
    mx.layernorm_mod(xd, rows, dim, 1e-6, d_sc, d_sh, out.t)
    torch.cuda.synchronize()
    out.check("layernorm_mod")
    H.assert_bf16_close(H.bits(out.t), ref, f"layernorm_mod {rows}x{dim} {variant}")


@pytest.mark.parametrize("rows,dim", [(8, 3072), (65, 5120), (33, 5376), (4, 1152), (7, 99), (300, 4096)])
@pytest.mark.parametrize("has_w,has_sc,has_sh", [(1, 1, 1), (1, 0, 0), (0, 1, 0), (0, 0, 0), (1, 1, 0)])
def test_rmsnorm_mod(mx, rows, dim, has_w, has_sc, has_sh):
    g = H.rng(rows * 7 + dim + has_w * 3 + has_sc * 5 + has_sh * 11)
    x = H.normal_f32(g, (rows, dim), std=2.0)
    w = H.normal_f32(g, dim, 0.1, 1.0) if has_w else None
    sc_t, sc_p = H.normal_f32(g, dim, 0.3), H.normal_f32(g, dim, 0.3)
    sh_t = H.normal_f32(g, dim, 0.3)
    plen = rows // 2
    keep = []
    o_sc = orc.mod(sc_t, sc_p, plen) if has_sc else orc.NONE
    o_sh = orc.mod(sh_t) if has_sh else orc.NONE
    d_sc = dev_mod(mx, keep, sc_t, sc_p, plen) if has_sc else None
    d_sh = dev_mod(mx, keep, sh_t) if has_sh else None
    ref = orc.rmsnorm_mod(x, 1e-5, w, o_sc, o_sh)
    out = H.Guarded(torch, (rows, dim), torch.bfloat16)
    wd = H.to_dev(torch, w) if has_w else None
    mx.rmsnorm_mod(H.to_dev(torch, x), rows, dim, 1e-5, wd, d_sc, d_sh, out.t)
    torch.cuda.synchronize()
    out.check("rmsnorm_mod")
    H.assert_bf16_close(H.bits(out.t), ref, f"rmsnorm_mod {rows}x{dim}")


@pytest.mark.parametrize("rows,dim", [(16, 3584), (5, 1152), (9, 77), (64, 4096)])
def test_rmsnorm_bf16(mx, rows, dim):
    g = H.rng(rows + dim)
    x = H.normal_bf16(g, (rows, dim), 1.5)
    w = H.normal_f32(g, dim, 0.1, 1.0)
    ref = orc.rmsnorm_bf16(x, 1e-6, w)
    out = H.Guarded(torch, (rows, dim), torch.bfloat16)
    mx.rmsnorm_bf16(H.to_dev(torch, x), rows, dim, 1e-6, H.to_dev(torch, w), out.t)
    torch.cuda.synchronize()
    out.check("rmsnorm_bf16")
    H.assert_bf16_close(H.bits(out.t), ref, "rmsnorm_bf16")


def test_norm_unaligned_pointers(mx):
    """Base pointers offset by one element (only element alignment is guaranteed by the callers)."""
    g = H.rng(5)
    rows, dim = 9, 3072
    x = H.normal_f32(g, (rows, dim))
    sc = H.normal_f32(g, dim, 0.3)
    ref = orc.layernorm_mod(x, 1e-6, orc.mod(sc), orc.NONE)
    xbuf = torch.zeros(rows * dim + 1, dtype=torch.float32, device="cuda")
    xbuf[1:].copy_(torch.from_numpy(x).reshape(-1))
    obuf = torch.zeros(rows * dim + 1, dtype=torch.bfloat16, device="cuda")
    scd = H.to_dev(torch, sc)
    mx.layernorm_mod(xbuf[1:], rows, dim, 1e-6, mx.row_mod(scd), None, obuf[1:])
    torch.cuda.synchronize()
    H.assert_bf16_close(H.bits(obuf[1:]), ref, "unaligned layernorm_mod")
    assert float(obuf[0]) == 0.0


def _offset_view(flat, off, n):
    """`n` elements of a flat device tensor starting `off` elements in (an offset pointer, as the
    reference's callers pass: src/models/minimax_h3/dit_sp.cpp:91,153-163)."""
    return flat[off:off + n]


@pytest.mark.parametrize("off", [4, 8, 12])
def test_rmsnorm_bf16_input_offset_by_eight_bytes(mx, off):
    """A bf16 x that starts 4 (or 12) elements into its buffer is 8- but not 16-byte aligned: it must
    leave the bulk-copy kernel (whose copies need 16) and still match the oracle."""
    g = H.rng(40 + off)
    rows, dim = 37, 3584
    x = H.normal_bf16(g, (rows, dim), 1.5)
    w = H.normal_f32(g, dim, 0.1, 1.0)
    ref = orc.rmsnorm_bf16(x, 1e-6, w)
    xbuf = torch.zeros(rows * dim + 16, dtype=torch.bfloat16, device="cuda")
    xv = _offset_view(xbuf, off, rows * dim)
    xv.copy_(H.to_dev(torch, x).reshape(-1))
    out = H.Guarded(torch, (rows, dim), torch.bfloat16)
    wd = H.to_dev(torch, w)
    path = mx.norm_path_probe(2, xv, None, out.t, wd, rows, dim)
    assert xv.data_ptr() % 16 == (off * 2) % 16
    if xv.data_ptr() % 16:
        assert path == mx.NORM_PATH_VECTOR
    mx.rmsnorm_bf16(xv, rows, dim, 1e-6, wd, out.t)
    torch.cuda.synchronize()
    out.check("rmsnorm_bf16 offset x")
    H.assert_bf16_close(H.bits(out.t), ref, f"rmsnorm_bf16 x offset {off}")


@pytest.mark.parametrize("norm_mode", [0, 1])
@pytest.mark.parametrize("off", [4, 8])
def test_gated_residual_norm_residual_row_offset_by_eight_bytes(mx, norm_mode, off):
    """The fused residual + norm with y starting 4 elements into its buffer: the register kernel's
    64-bit loads take it; the result equals the oracle and x equals the two-call form bit for bit."""
    g = H.rng(50 + off + norm_mode)
    rows, dim = 41, 3072
    x = H.normal_f32(g, (rows, dim))
    y = H.normal_bf16(g, (rows, dim))
    gate = H.normal_f32(g, dim, 0.7)
    sc, sh = H.normal_f32(g, dim, 0.3), H.normal_f32(g, dim, 0.3)
    w = H.normal_f32(g, dim, 0.1, 1.0) if norm_mode == 1 else None
    xr = orc.gated_residual(x.copy(), y, orc.mod(gate), 1)
    ref = (orc.layernorm_mod(xr, 1e-6, orc.mod(sc), orc.mod(sh)) if norm_mode == 0
           else orc.rmsnorm_mod(xr, 1e-6, w, orc.mod(sc), orc.mod(sh)))
    keep = []
    dg, dsc, dsh = dev_mod(mx, keep, gate), dev_mod(mx, keep, sc), dev_mod(mx, keep, sh)
    wd = H.to_dev(torch, w) if w is not None else None
    ybuf = torch.zeros(rows * dim + 16, dtype=torch.bfloat16, device="cuda")
    yv = _offset_view(ybuf, off, rows * dim)
    yv.copy_(H.to_dev(torch, y).reshape(-1))
    xf = H.Guarded(torch, (rows, dim), torch.float32, fill=torch.from_numpy(x))
    of = H.Guarded(torch, (rows, dim), torch.bfloat16)
    path = mx.norm_path_probe(3 + norm_mode, xf.t, yv, of.t, wd, rows, dim, dsc, dsh, dg)
    if yv.data_ptr() % 16:
        assert path == mx.NORM_PATH_VECTOR
    mx.gated_residual_norm(xf.t, yv, rows, dim, dg, 1, norm_mode, 1e-6, wd, dsc, dsh, of.t)
    x2 = H.to_dev(torch, x)
    mx.gated_residual(x2, yv, rows, dim, dg, 1)
    torch.cuda.synchronize()
    xf.check("fused x"), of.check("fused out")
    H.assert_f32_close(xf.t.cpu().numpy(), xr, "fused residual x, offset y")
    H.assert_bf16_close(H.bits(of.t), ref, "fused norm out, offset y")
    assert torch.equal(xf.t, x2)


def test_gated_residual_norm_quant_refuses_a_residual_row_offset_by_eight_bytes(mx):
    """The one-pass MXFP8 form exists for the bulk-copy kernel only: an 8-byte aligned y is refused
    with a status (the caller then makes the two calls), nothing is launched."""
    rows, dim = 16, 3072
    x = torch.zeros((rows, dim), dtype=torch.float32, device="cuda")
    ybuf = torch.zeros(rows * dim + 16, dtype=torch.bfloat16, device="cuda")
    launches = mx.launch_count()
    with pytest.raises(mx.MxkError, match="outside the one-pass kernel"):
        mx.gated_residual_norm_quant_mxfp8(x, _offset_view(ybuf, 4, rows * dim), rows, dim, None, 0, 0, 1e-6, None, None, None)
    assert mx.launch_count() == launches
    # the same call with y offset by a multiple of 16 bytes runs
    mx.gated_residual_norm_quant_mxfp8(x, _offset_view(ybuf, 8, rows * dim), rows, dim, None, 0, 0, 1e-6, None, None, None)
    torch.cuda.synchronize()


@pytest.mark.parametrize("rows,dim", [(8, 3072), (37, 5376), (19, 100), (7, 99), (1, 4096), (260, 3072)])
@pytest.mark.parametrize("mode", ["tanh_prefix", "identity", "none"])
def test_gated_residual(mx, rows, dim, mode):
    g = H.rng(rows * 3 + dim)
    x = H.normal_f32(g, (rows, dim))
    y = H.normal_bf16(g, (rows, dim))
    gt, gp = H.normal_f32(g, dim, 0.7), H.normal_f32(g, dim, 0.7)
    plen = rows // 2 + 1
    keep = []
    if mode == "tanh_prefix":
        og, dg, tanh = orc.mod(gt, gp, plen), dev_mod(mx, keep, gt, gp, plen), 1
    elif mode == "identity":
        og, dg, tanh = orc.mod(gt), dev_mod(mx, keep, gt), 0
    else:
        og, dg, tanh = orc.NONE, None, 0
    ref = orc.gated_residual(x.copy(), y, og, tanh)
    xd = H.Guarded(torch, (rows, dim), torch.float32, fill=torch.from_numpy(x))
    mx.gated_residual(xd.t, H.to_dev(torch, y), rows, dim, dg, tanh)
    torch.cuda.synchronize()
    xd.check("gated_residual")
    H.assert_f32_close(xd.t.cpu().numpy(), ref, f"gated_residual {rows}x{dim} {mode}")


@pytest.mark.parametrize("rows,dim,norm_mode", [(40, 3072, 0), (33, 5376, 1), (9, 5120, 1), (7, 99, 0), (130, 4096, 0)])
def test_gated_residual_norm_equals_two_calls(mx, rows, dim, norm_mode):
    """The fused extension against the oracle's gated_residual followed by its norm, and against
    libmxk's own two calls (x must match bit for bit, out within tolerance)."""
    g = H.rng(rows + dim + norm_mode)
    x = H.normal_f32(g, (rows, dim))
    y = H.normal_bf16(g, (rows, dim))
    gate_t, gate_p = H.normal_f32(g, dim, 0.7), H.normal_f32(g, dim, 0.7)
    sc, sh = H.normal_f32(g, dim, 0.3), H.normal_f32(g, dim, 0.3)
    w = H.normal_f32(g, dim, 0.1, 1.0) if norm_mode == 1 else None
    plen = rows // 2
    tanh = 1 if norm_mode == 0 else 0
    xr = orc.gated_residual(x.copy(), y, orc.mod(gate_t, gate_p, plen), tanh)
    if norm_mode == 0:
        ref = orc.layernorm_mod(xr, 1e-6, orc.mod(sc), orc.mod(sh))
    else:
        ref = orc.rmsnorm_mod(xr, 1e-6, w, orc.mod(sc), orc.mod(sh))
    keep = []
    dg = dev_mod(mx, keep, gate_t, gate_p, plen)
    dsc, dsh = dev_mod(mx, keep, sc), dev_mod(mx, keep, sh)
    wd = H.to_dev(torch, w) if w is not None else None
    yd = H.to_dev(torch, y)
    xf = H.Guarded(torch, (rows, dim), torch.float32, fill=torch.from_numpy(x))
    of = H.Guarded(torch, (rows, dim), torch.bfloat16)
    mx.gated_residual_norm(xf.t, yd, rows, dim, dg, tanh, norm_mode, 1e-6, wd, dsc, dsh, of.t)
    x2 = H.to_dev(torch, x)
    o2 = torch.empty((rows, dim), dtype=torch.bfloat16, device="cuda")
    mx.gated_residual(x2, yd, rows, dim, dg, tanh)
    if norm_mode == 0:
        mx.layernorm_mod(x2, rows, dim, 1e-6, dsc, dsh, o2)
    else:
        mx.rmsnorm_mod(x2, rows, dim, 1e-6, wd, dsc, dsh, o2)
    torch.cuda.synchronize()
    xf.check("fused x"), of.check("fused out")
    H.assert_f32_close(xf.t.cpu().numpy(), xr, "fused residual x")
    H.assert_bf16_close(H.bits(of.t), ref, "fused norm out")
    assert torch.equal(xf.t, x2), "fused and two-call residual streams differ"
    H.assert_bf16_close(H.bits(of.t), H.bits(o2), "fused vs two calls")


ROPE_CASES = [
    # S, H, D, rot, mode, in_stride(None=H*D), col0, has_norm
    (37, 24, 128, 128, 1, None, 0, True),      # Qwen-Image q/k
    (19, 40, 128, 128, 2, 3 * 5120, 5120, True),  # H3-shaped packed qkv, k slot
    (21, 56, 128, 96, 2, 3 * 7168, 0, True),   # true H3: only 96 of 128 channels rotate
    (11, 32, 128, 128, 1, None, 0, False),     # rope without norm
    (13, 8, 64, 64, 2, None, 0, True),         # text-encoder style heads
    (9, 16, 72, 72, 2, None, 0, True),         # vision tower D = 72 (generic kernel)
    (9, 16, 72, 0, 0, None, 0, True),          # norm only
    (23, 40, 128, 0, 0, 3 * 5120, 10240, False),  # v: strided copy
    (5, 7, 128, 64, 1, None, 0, True),         # prime head count, partial rotation
    (6, 3, 256, 256, 2, None, 0, True),
    (6, 5, 32, 32, 1, None, 0, True),
    (4, 2, 10, 6, 1, None, 0, True),           # tiny generic shape
    (1, 24, 128, 128, 1, None, 0, True),
]


@pytest.mark.parametrize("S,Hh,D,rot,mode,stride,col0,has_norm", ROPE_CASES)
def test_head_norm_rope(mx, S, Hh, D, rot, mode, stride, col0, has_norm):
    g = H.rng(S * 17 + Hh + D + rot + mode)
    stride = stride or Hh * D
    inp = H.normal_bf16(g, (S, stride), 1.3)
    w = H.normal_f32(g, D, 0.05, 1.0) if has_norm else None
    half = max(rot // 2, 1)
    ang = g.uniform(-3.1, 3.1, (S, half)).astype(np.float32)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    ref = orc.head_norm_rope(inp, S, stride, col0, Hh, D, w, 1e-6, cos, sin, rot, mode)
    out = H.Guarded(torch, (S, Hh, D), torch.bfloat16)
    mx.head_norm_rope(H.to_dev(torch, inp), S, stride, col0, Hh, D, H.to_dev(torch, w) if has_norm else None, 1e-6,
                      H.to_dev(torch, cos), H.to_dev(torch, sin), rot, mode, out.t)
    torch.cuda.synchronize()
    out.check("head_norm_rope")
    H.assert_bf16_close(H.bits(out.t), ref, f"head_norm_rope S{S} H{Hh} D{D} rot{rot} mode{mode}")


def test_head_norm_rope_copy_is_exact(mx):
    g = H.rng(3)
    S, Hh, D, I = 50, 40, 128, 5120
    inp = H.normal_bf16(g, (S, 3 * I))
    out = torch.zeros((S, Hh, D), dtype=torch.bfloat16, device="cuda")
    mx.head_norm_rope(H.to_dev(torch, inp), S, 3 * I, 2 * I, Hh, D, None, 0.0, None, None, 0, mx.ROPE_NONE, out)
    torch.cuda.synchronize()
    assert np.array_equal(H.bits(out).reshape(S, I), inp[:, 2 * I:3 * I])


@pytest.mark.parametrize("S,Hh,rot,mode", [(33, 40, 128, 2), (20, 24, 128, 1), (17, 56, 96, 2)])
def test_qkv_norm_rope_equals_three_calls(mx, S, Hh, rot, mode):
    g = H.rng(S + Hh)
    D, I = 128, Hh * 128
    qkv = H.to_dev(torch, H.normal_bf16(g, (S, 3 * I)))
    wq, wk = H.to_dev(torch, H.normal_f32(g, D, 0.05, 1.0)), H.to_dev(torch, H.normal_f32(g, D, 0.05, 1.0))
    ang = g.uniform(-3, 3, (S, rot // 2)).astype(np.float32)
    cos, sin = H.to_dev(torch, np.cos(ang)), H.to_dev(torch, np.sin(ang))
    one = [torch.zeros((S, Hh, D), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    sep = [torch.zeros((S, Hh, D), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    mx.qkv_norm_rope([mx.HeadSpec(qkv, 3 * I, 0, wq, one[0], rot, mode), mx.HeadSpec(qkv, 3 * I, I, wk, one[1], rot, mode),
                      mx.HeadSpec(qkv, 3 * I, 2 * I, None, one[2], 0, mx.ROPE_NONE)], S, Hh, D, 1e-5, cos, sin)
    mx.head_norm_rope(qkv, S, 3 * I, 0, Hh, D, wq, 1e-5, cos, sin, rot, mode, sep[0])
    mx.head_norm_rope(qkv, S, 3 * I, I, Hh, D, wk, 1e-5, cos, sin, rot, mode, sep[1])
    mx.head_norm_rope(qkv, S, 3 * I, 2 * I, Hh, D, None, 0.0, None, None, 0, mx.ROPE_NONE, sep[2])
    torch.cuda.synchronize()
    for a, b in zip(one, sep):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))


ACT_PATHS = [0, 1, 2]  # the default (one tile per CTA), the bulk-copy pipeline, the register kernels on one resident wave


@pytest.mark.parametrize("act_path", ACT_PATHS)
@pytest.mark.parametrize("rows,F", [(9, 12288), (33, 13824), (5, 100), (3, 99), (130, 14336), (300, 1736)])
def test_silu_mul(mx, rows, F, act_path):
    g = H.rng(rows + F)
    gu = H.normal_bf16(g, (rows, 2 * F), 2.0)
    ref = orc.silu_mul(gu, F)
    out = H.Guarded(torch, (rows, F), torch.bfloat16)
    mx.set_tuning("act_path", act_path)
    try:
        mx.silu_mul(H.to_dev(torch, gu), rows, F, out.t)
        torch.cuda.synchronize()
    finally:
        mx.set_tuning("act_path", 0)
    out.check("silu_mul")
    H.assert_bf16_close(H.bits(out.t), ref, "silu_mul")


def _all_bf16_values():
    bits_ = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    v = orc.bf16_bits_to_f32(bits_)
    return bits_[np.isfinite(v)]


@pytest.mark.parametrize("act_path", ACT_PATHS)
@pytest.mark.parametrize("kind", ["tanh", "erf"])
def test_gelu_every_bf16_value(mx, kind, act_path):
    """Both GELUs on every finite bf16 input (the whole domain), plus a ragged random length."""
    g = H.rng(11)
    for x in (_all_bf16_values(), H.normal_bf16(g, 1000003, 2.5)):
        ref = (orc.gelu_tanh_inplace if kind == "tanh" else orc.gelu_erf_inplace)(x.copy())
        xd = H.Guarded(torch, (x.size,), torch.bfloat16, fill=H.to_dev(torch, x))
        mx.set_tuning("act_path", act_path)
        try:
            (mx.gelu_tanh_inplace if kind == "tanh" else mx.gelu_erf_inplace)(xd.t, x.size)
            torch.cuda.synchronize()
        finally:
            mx.set_tuning("act_path", 0)
        xd.check("gelu")
        H.assert_bf16_close(H.bits(xd.t), ref, f"gelu_{kind}")


def test_silu_inplace_f32(mx):
    g = H.rng(2)
    x = H.normal_f32(g, 2 * 3072 + 3, 3.0)
    ref = orc.silu_inplace_f32(x.copy())
    xd = H.Guarded(torch, (x.size,), torch.float32, fill=torch.from_numpy(x))
    mx.silu_inplace_f32(xd.t, x.size)
    torch.cuda.synchronize()
    xd.check("silu_f32")
    H.assert_f32_close(xd.t.cpu().numpy(), ref, "silu_inplace_f32", rel=2.0 ** -18)


@pytest.mark.parametrize("rows,dim", [(33, 3072), (7, 99), (5, 15360), (1, 8)])
def test_add_bias(mx, rows, dim):
    g = H.rng(rows + dim)
    bias = H.normal_f32(g, dim)
    yb = H.normal_bf16(g, (rows, dim))
    yf = H.normal_f32(g, (rows, dim))
    rb, rf = orc.add_bias_bf16(yb.copy(), bias), orc.add_bias_f32(yf.copy(), bias)
    bd = H.to_dev(torch, bias)
    db = H.Guarded(torch, (rows, dim), torch.bfloat16, fill=H.to_dev(torch, yb))
    df = H.Guarded(torch, (rows, dim), torch.float32, fill=torch.from_numpy(yf))
    mx.add_bias_bf16(db.t, bd, rows, dim)
    mx.add_bias_f32(df.t, bd, rows, dim)
    torch.cuda.synchronize()
    db.check("add_bias_bf16"), df.check("add_bias_f32")
    assert np.array_equal(H.bits(db.t), rb)
    assert np.array_equal(df.t.cpu().numpy(), rf)


@pytest.mark.parametrize("n", [1, 7, 8, 4099, 64 * 4096 + 5])
def test_casts_axpy_add(mx, n):
    g = H.rng(n)
    x, y = H.normal_f32(g, n), H.normal_f32(g, n)
    xb, yb = H.normal_bf16(g, n), H.normal_bf16(g, n)
    # casts are exact
    ob = H.Guarded(torch, (n,), torch.bfloat16)
    mx.f32_to_bf16(H.to_dev(torch, x), ob.t, n)
    of = H.Guarded(torch, (n,), torch.float32)
    mx.bf16_to_f32(H.to_dev(torch, xb), of.t, n)
    ab = H.Guarded(torch, (n,), torch.bfloat16, fill=H.to_dev(torch, xb))
    mx.add_inplace_bf16(ab.t, H.to_dev(torch, yb), n)
    ax = H.Guarded(torch, (n,), torch.float32, fill=torch.from_numpy(x))
    mx.axpy_f32(ax.t, H.to_dev(torch, y), 0.37, n)
    ay = H.Guarded(torch, (n,), torch.float32, fill=torch.from_numpy(x))
    mx.axpby_f32(ay.t, H.to_dev(torch, y), 1.7, -0.6, n)
    torch.cuda.synchronize()
    for b in (ob, of, ab, ax, ay):
        b.check("elementwise")
    assert np.array_equal(H.bits(ob.t), orc.f32_to_bf16(x))
    assert np.array_equal(of.t.cpu().numpy(), orc.bf16_to_f32(xb))
    assert np.array_equal(H.bits(ab.t), orc.add_inplace_bf16(xb.copy(), yb))
    H.assert_f32_close(ax.t.cpu().numpy(), orc.axpy_f32(x.copy(), y, 0.37), "axpy", rel=2.0 ** -22)
    H.assert_f32_close(ay.t.cpu().numpy(), orc.axpby_f32(x.copy(), y, 1.7, -0.6), "axpby", rel=2.0 ** -22)


@pytest.mark.parametrize("dim,add", [(2048, 0), (2048, 1), (99, 1)])
def test_scatter_rows(mx, dim, add):
    g = H.rng(dim + add)
    total, n = 50, 13
    x = H.normal_f32(g, (total, dim))
    rows = g.permutation(total)[:n].astype(np.int32)
    src = H.normal_bf16(g, (n, dim))
    ref = orc.scatter_rows(x.copy(), rows, src, add)
    xd = H.Guarded(torch, (total, dim), torch.float32, fill=torch.from_numpy(x))
    mx.scatter_rows(xd.t, dim, torch.from_numpy(rows).cuda(), H.to_dev(torch, src), n, add)
    torch.cuda.synchronize()
    xd.check("scatter_rows")
    assert np.array_equal(xd.t.cpu().numpy(), ref)


def test_zero_rows_are_noops(mx):
    mx.layernorm_mod(None, 0, 3072, 1e-6, None, None, None)
    mx.rmsnorm_mod(None, -1, 3072, 1e-6, None, None, None, None)
    mx.gated_residual(None, None, 0, 3072, None, 1)
    mx.head_norm_rope(None, 0, 3072, 0, 24, 128, None, 1e-6, None, None, 128, 1, None)
    mx.gelu_tanh_inplace(None, 0)
    mx.silu_mul(None, 0, 12288, None)


def test_two_shards_equal_one(mx):
    """Row ops are independent, so two half-launches with the prefix boundary shifted the way the
    reference shifts it (src/kernels/ops.cu:183-184) must reproduce the single launch bit for bit."""
    g = H.rng(77)
    rows, dim, plen = 301, 3072, 120
    x = H.to_dev(torch, H.normal_f32(g, (rows, dim)))
    sc_t, sc_p = H.to_dev(torch, H.normal_f32(g, dim, 0.3)), H.to_dev(torch, H.normal_f32(g, dim, 0.3))
    one = torch.empty((rows, dim), dtype=torch.bfloat16, device="cuda")
    two = torch.empty((rows, dim), dtype=torch.bfloat16, device="cuda")
    mx.layernorm_mod(x, rows, dim, 1e-6, mx.row_mod(sc_t, sc_p, plen), None, one)
    r0 = 150
    mx.layernorm_mod(x, r0, dim, 1e-6, mx.row_mod(sc_t, sc_p, plen), None, two)
    mx.layernorm_mod(x[r0:], rows - r0, dim, 1e-6, mx.row_mod(sc_t, sc_p, plen - r0), None, two[r0:])
    torch.cuda.synchronize()
    assert torch.equal(one.view(torch.int16), two.view(torch.int16))


@pytest.mark.parametrize("op", ["layernorm", "rmsnorm", "fused", "residual"])
@pytest.mark.parametrize("stages", [2, 3])
def test_row_pipeline_many_trips(mx, op, stages):
    """Enough rows per CTA that every shared-memory stage of the bulk-copy pipeline is refilled many
    times (one CTA per SM, 2-3 stages, thousands of rows), with the prefix switch in the middle."""
    rows, dim, plen = 4001, 3072, 1777
    g = H.rng(stages * 10 + len(op))
    x = H.normal_f32(g, (rows, dim), 1.0, 0.2)
    y = H.normal_bf16(g, (rows, dim))
    sc_t, sc_p, sh = H.normal_f32(g, dim, 0.3), H.normal_f32(g, dim, 0.3), H.normal_f32(g, dim, 0.3)
    gt, gp = H.normal_f32(g, dim, 0.7), H.normal_f32(g, dim, 0.7)
    w = H.normal_f32(g, dim, 0.1, 1.0)
    keep = []
    dsc, dsh, dg = dev_mod(mx, keep, sc_t, sc_p, plen), dev_mod(mx, keep, sh), dev_mod(mx, keep, gt, gp, plen)
    osc, osh, og = orc.mod(sc_t, sc_p, plen), orc.mod(sh), orc.mod(gt, gp, plen)
    orc.set_threads(8)
    mx.set_tuning("norm_stages", stages)
    mx.set_tuning("norm_ctas_per_sm", 1)
    try:
        xd = H.Guarded(torch, (rows, dim), torch.float32, fill=torch.from_numpy(x))
        out = H.Guarded(torch, (rows, dim), torch.bfloat16)
        if op == "layernorm":
            ref = orc.layernorm_mod(x, 1e-6, osc, osh)
            mx.layernorm_mod(xd.t, rows, dim, 1e-6, dsc, dsh, out.t)
        elif op == "rmsnorm":
            ref = orc.rmsnorm_mod(x, 1e-6, w, osc, osh)
            mx.rmsnorm_mod(xd.t, rows, dim, 1e-6, H.to_dev(torch, w), dsc, dsh, out.t)
        elif op == "fused":
            xr = orc.gated_residual(x.copy(), y, og, 1)
            ref = orc.layernorm_mod(xr, 1e-6, osc, osh)
            mx.gated_residual_norm(xd.t, H.to_dev(torch, y), rows, dim, dg, 1, 0, 1e-6, None, dsc, dsh, out.t)
        else:
            xr = orc.gated_residual(x.copy(), y, og, 1)
            mx.gated_residual(xd.t, H.to_dev(torch, y), rows, dim, dg, 1)
        torch.cuda.synchronize()
        xd.check(op), out.check(op)
        if op != "residual":
            H.assert_bf16_close(H.bits(out.t), ref, op)
        if op in ("fused", "residual"):
            H.assert_f32_close(xd.t.cpu().numpy(), xr, op + " x")
    finally:
        orc.set_threads(1)
        mx.set_tuning("norm_stages", 0)
        mx.set_tuning("norm_ctas_per_sm", 0)


@pytest.mark.parametrize("tokens,stages,threads", [(1, 2, 128), (3, 2, 512), (2, 4, 192)])
@pytest.mark.parametrize("layout", ["dense_qk", "packed_qkv"])
def test_head_pipeline_many_trips(mx, tokens, stages, threads, layout):
    """The head pipeline with every stage refilled many times, one and several tokens per stage,
    one and several passes over the heads, separate and packed projections."""
    S, Hh, D = 2999, 24, 128
    I = Hh * D
    g = H.rng(tokens * 100 + stages * 10 + threads)
    ang = g.uniform(-3, 3, (S, D // 2)).astype(np.float32)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    wq, wk = H.normal_f32(g, D, 0.05, 1.0), H.normal_f32(g, D, 0.05, 1.0)
    orc.set_threads(8)
    mx.set_tuning("rope_stages", stages)
    mx.set_tuning("rope_tokens", tokens)
    mx.set_tuning("rope_threads", threads)
    mx.set_tuning("rope_ctas_per_sm", 1)
    try:
        cd, sd = H.to_dev(torch, cos), H.to_dev(torch, sin)
        wqd, wkd = H.to_dev(torch, wq), H.to_dev(torch, wk)
        outs = [H.Guarded(torch, (S, Hh, D), torch.bfloat16) for _ in range(3)]
        if layout == "dense_qk":
            q, k = H.normal_bf16(g, (S, I)), H.normal_bf16(g, (S, I))
            refs = [orc.head_norm_rope(q, S, I, 0, Hh, D, wq, 1e-6, cos, sin, D, 1),
                    orc.head_norm_rope(k, S, I, 0, Hh, D, wk, 1e-6, cos, sin, D, 1)]
            qd, kd = H.to_dev(torch, q), H.to_dev(torch, k)
            mx.head_norm_rope(qd, S, I, 0, Hh, D, wqd, 1e-6, cd, sd, D, 1, outs[0].t)
            mx.qkv_norm_rope([mx.HeadSpec(qd, I, 0, wqd, outs[2].t, D, 1), mx.HeadSpec(kd, I, 0, wkd, outs[1].t, D, 1)],
                             S, Hh, D, 1e-6, cd, sd)
            refs.append(refs[0])
        else:
            qkv = H.normal_bf16(g, (S, 3 * I))
            refs = [orc.head_norm_rope(qkv, S, 3 * I, 0, Hh, D, wq, 1e-6, cos, sin, D, 2),
                    orc.head_norm_rope(qkv, S, 3 * I, I, Hh, D, wk, 1e-6, cos, sin, D, 2),
                    orc.head_norm_rope(qkv, S, 3 * I, 2 * I, Hh, D, None, 0.0, None, None, 0, 0)]
            d = H.to_dev(torch, qkv)
            mx.qkv_norm_rope([mx.HeadSpec(d, 3 * I, 0, wqd, outs[0].t, D, 2), mx.HeadSpec(d, 3 * I, I, wkd, outs[1].t, D, 2),
                              mx.HeadSpec(d, 3 * I, 2 * I, None, outs[2].t, 0, 0)], S, Hh, D, 1e-6, cd, sd)
        torch.cuda.synchronize()
        for o, r in zip(outs, refs):
            o.check("head pipeline")
            H.assert_bf16_close(H.bits(o.t), r, f"head pipeline {layout}")
    finally:
        orc.set_threads(1)
        for k in ("rope_stages", "rope_tokens", "rope_threads", "rope_ctas_per_sm"):
            mx.set_tuning(k, 0)


@pytest.mark.parametrize("stages,warps,chunk_kb", [(2, 4, 8), (3, 8, 16), (4, 2, 4)])
def test_stream_pipeline_many_trips(mx, stages, warps, chunk_kb):
    """GELU and SiLU-mul through the streaming pipeline with every stage refilled many times
    (one CTA per SM), ragged array length and a ragged last chunk per row."""
    g = H.rng(stages + warps)
    orc.set_threads(8)
    for k, v in (("stream_stages", stages), ("stream_warps", warps), ("stream_chunk_kb", chunk_kb), ("stream_ctas_per_sm", 1),
                 ("act_path", 1)):
        mx.set_tuning(k, v)
    try:
        n = 12 * 1000 * 1000 + 5
        x = H.normal_bf16(g, n, 2.0)
        ref = orc.gelu_tanh_inplace(x.copy())
        xd = H.Guarded(torch, (n,), torch.bfloat16, fill=H.to_dev(torch, x))
        mx.gelu_tanh_inplace(xd.t, n)
        rows, F = 700, 13824
        gu = H.normal_bf16(g, (rows, 2 * F), 2.0)
        rs = orc.silu_mul(gu, F)
        out = H.Guarded(torch, (rows, F), torch.bfloat16)
        mx.silu_mul(H.to_dev(torch, gu), rows, F, out.t)
        torch.cuda.synchronize()
        xd.check("gelu pipeline"), out.check("silu pipeline")
        H.assert_bf16_close(H.bits(xd.t), ref, "gelu pipeline")
        H.assert_bf16_close(H.bits(out.t), rs, "silu pipeline")
    finally:
        orc.set_threads(1)
        for k in ("stream_stages", "stream_warps", "stream_chunk_kb", "stream_ctas_per_sm", "act_path"):
            mx.set_tuning(k, 0)
