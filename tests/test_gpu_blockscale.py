"""libmxk's block-scale quantiser through the C ABI: byte-exact against the CPU oracle, against the
golden outputs of the REFERENCE's kernel, and - where oracle/_ref/libmx_ref_blockscale.so travelled with
the tree - against that kernel run side by side on the same device buffers."""
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
import ref_blockscale_cases  # noqa: E402
from make_ref_blockscale_golden import run_reference  # noqa: E402
from test_cpu_blockscale import ELEM_ERR, GOLDEN, bits_to_f32, rel_rms  # noqa: E402

CASES = ref_blockscale_cases.cases()


@pytest.fixture(scope="module", params=["bulk_copy", "registers", "block_per_thread"])
def mx(request):
    """Every test runs with the bulk-copy streaming pipeline, with the register kernels and with the kernels that give
    a thread a whole MXFP8 scale block (or a pair of NVFP4 blocks) and a CTA one row."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import miroxen_b200 as m
    m.lib()
    m.set_tuning("quant_path", {"bulk_copy": 1, "registers": 2, "block_per_thread": 3}[request.param])
    yield m
    torch.cuda.synchronize()
    assert m.device_error() == 0, "a kernel's bounded wait ran out"
    m.set_tuning("quant_path", 0)


def mxk_quant(mx, mode, x_bits, K, guard=True):
    """Runs mxk_quantize_blockscaled; outputs sit between poisoned guard bands."""
    rows, ldx = x_bits.shape
    x = torch.from_numpy(np.ascontiguousarray(x_bits)).cuda()
    q = H.Guarded(torch, (mx.ops.qdata_bytes(mode, rows, K),), torch.uint8)
    sf = H.Guarded(torch, (mx.ops.qscale_bytes(mode, rows, K),), torch.uint8)
    sf.t.fill_(0x5A)
    amax = torch.full((1,), -1.0, dtype=torch.float32, device="cuda") if mode == 2 else None
    mx.ops.quantize_blockscaled(mode, x, ldx, rows, K, mx.ops.QMat(q.t, sf.t, amax))
    torch.cuda.synchronize()
    q.check("q")
    sf.check("sf")
    return q.t.cpu().numpy(), sf.t.cpu().numpy(), (float(amax.item()) if mode == 2 else 0.0)


def assert_same(name, got, want):
    (q, sf, amax), (rq, rsf, ramax) = got, want
    assert np.array_equal(sf, rsf), f"{name}: {(sf != rsf).sum()} scale bytes differ"
    assert np.array_equal(q, rq), f"{name}: {(q != rq).sum()} of {q.size} data bytes differ"
    assert np.float32(amax) == np.float32(ramax), name


@pytest.mark.parametrize("name", sorted(CASES))
def test_cases_match_oracle_and_golden(mx, name):
    c = CASES[name]
    got = mxk_quant(mx, c["mode"], c["x"], c["K"])
    assert_same(name, got, orc.quantize_blockscaled(c["mode"], c["x"], c["K"]))
    gold = np.load(GOLDEN)
    assert_same(name + " (reference kernel bytes)", got,
                (gold[name + ".q"], gold[name + ".sf"], gold[name + ".amax"][0] if c["mode"] == 2 else 0.0))


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("rows,K,ldx", [(1, 32, 32), (3, 64, 72), (127, 96, 96), (128, 128, 128), (129, 160, 168),
                                         (257, 2048, 2048), (40, 2080, 2088), (33, 4096 + 32, 4096 + 32),
                                         (1000, 3072, 3072), (515, 12288, 12288)])
def test_shapes_match_oracle(mx, mode, rows, K, ldx):
    g = H.rng(rows * 7 + K + mode)
    a = H.normal_f32(g, (rows, ldx), 1.5)
    a[:, ::53] *= 30.0
    bits = orc.f32_to_bf16_bits(a)
    assert_same(f"{rows}x{K}", mxk_quant(mx, mode, bits, K), orc.quantize_blockscaled(mode, bits, K))


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("knob,value", [("quant_rows_per_cta", 1), ("quant_rows_per_cta", 3), ("quant_rows_per_cta", 64),
                                        ("stream_chunk_kb", 1), ("stream_chunk_kb", 2), ("stream_stages", 2),
                                        ("stream_warps", 3), ("stream_ctas_per_sm", 1)])
def test_work_split_does_not_change_bytes(mx, mode, knob, value):
    """Row strips, row pieces (1 KB chunks cut the 2112-byte rows in three), pipeline depth and a grid
    of one CTA per SM, where every CTA wraps its ring of stages many times."""
    g = H.rng(90 + value)
    bits = H.normal_bf16(g, (1777, 1056), 2.0)
    want = orc.quantize_blockscaled(mode, bits)
    mx.ops.set_tuning(knob, value)
    try:
        assert_same(f"{knob}={value}", mxk_quant(mx, mode, bits, 1056), want)
    finally:
        mx.ops.set_tuning(knob, 0)


@pytest.mark.parametrize("mode", [1, 2])
def test_block_size_workload_matches_oracle_and_error_bound(mx, mode):
    """One image-stream activation of the benchmark's block: 8704 rows of 3072 (> L2 with its outputs)."""
    g = H.rng(5)
    rows, K = 8704, 3072
    a = H.normal_f32(g, (rows, K), 1.0)
    a[:, ::211] *= 25.0
    bits = orc.f32_to_bf16_bits(a)
    orc.set_threads(8)
    try:
        want = orc.quantize_blockscaled(mode, bits)
    finally:
        orc.set_threads(1)
    got = mxk_quant(mx, mode, bits, K)
    assert_same("8704x3072", got, want)
    d = orc.dequantize_blockscaled(mode, got[0], got[1], got[2], rows, K)
    assert rel_rms(d, bits_to_f32(bits)) < ELEM_ERR[mode]


def test_second_call_reuses_buffers_and_clears_padding(mx):
    g = H.rng(11)
    big, small = H.normal_bf16(g, (100, 160), 3.0), H.normal_bf16(g, (100, 160), 0.01)
    for mode in (1, 2):
        x = torch.from_numpy(big).cuda()
        out = mx.ops.quantize_blockscaled(mode, x, 160, 100, 160)
        x.copy_(torch.from_numpy(small))
        mx.ops.quantize_blockscaled(mode, x, 160, 100, 160, out)
        torch.cuda.synchronize()
        want = orc.quantize_blockscaled(mode, small)
        assert_same("second call", (out.q.cpu().numpy(), out.sf.cpu().numpy(), float(out.amax.item()) if mode == 2 else 0.0), want)


def test_argument_errors(mx):
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda")
    out = mx.ops.quantize_blockscaled(1, x, 64, 4, 64)
    for bad in (dict(mode=0), dict(K=48), dict(ldx=60), dict(ldx=32), dict(mode=3)):
        kw = dict(mode=1, ldx=64, K=64)
        kw.update(bad)
        with pytest.raises(mx.MxkError):
            mx.ops.quantize_blockscaled(kw["mode"], x, kw["ldx"], 4, kw["K"], out)
    with pytest.raises(mx.MxkError):  # NVFP4 needs the amax slot
        mx.ops.quantize_blockscaled(2, x, 64, 4, 64, mx.ops.QMat(out.q, out.sf, None))
    with pytest.raises(mx.MxkError):  # misaligned input
        mx.ops.quantize_blockscaled(1, x.view(-1)[1:].data_ptr(), 64, 3, 64, out)
    mx.ops.quantize_blockscaled(1, x, 64, 0, 64, out)  # no rows: nothing to do
    torch.cuda.synchronize()


@pytest.mark.skipif(not orc.have_ref_blockscale(), reason="oracle/_ref/libmx_ref_blockscale.so not built")
@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("rows,K,ldx", [(130, 384, 384), (37, 160, 168), (2049, 3072, 3072), (300, 12288, 12288)])
def test_side_by_side_with_reference_kernel(mx, mode, rows, K, ldx):
    g = H.rng(rows + K)
    a = H.normal_f32(g, (rows, ldx), 1.2)
    a[:, ::101] *= 17.0
    bits = orc.f32_to_bf16_bits(a)
    rq, rsf, ramax = run_reference(orc.ref_blockscale(), mode, bits, K)
    assert_same("reference kernel", mxk_quant(mx, mode, bits, K), (rq, rsf, float(ramax[0]) if mode == 2 else 0.0))


# ---- activation + MXFP8 quantisation in one pass ----

def two_calls(mx, act_mode, x_bits, rows, F):
    """The activation kernel of this library followed by its quantiser."""
    x = H.to_dev(torch, x_bits)
    if act_mode == mx.ops.ACT_SILU_MUL:
        act = torch.empty(rows, F, dtype=torch.bfloat16, device="cuda")
        mx.ops.silu_mul(x, rows, F, act)
    else:
        act = x.clone()
        (mx.ops.gelu_tanh_inplace if act_mode == mx.ops.ACT_GELU_TANH else mx.ops.gelu_erf_inplace)(act, rows * F)
    out = mx.ops.quantize_blockscaled(mx.ops.Q_MXFP8, act, F, rows, F)
    torch.cuda.synchronize()
    return out.q.cpu().numpy(), out.sf.cpu().numpy(), H.bits(act)


def one_call(mx, act_mode, x_bits, rows, F):
    x = H.to_dev(torch, x_bits)
    q = H.Guarded(torch, (mx.ops.qdata_bytes(1, rows, F),), torch.uint8)
    sf = H.Guarded(torch, (mx.ops.qscale_bytes(1, rows, F),), torch.uint8)
    sf.t.fill_(0x5A)
    before = x.clone()
    mx.ops.act_quantize_mxfp8(act_mode, x, rows, F, mx.ops.QMat(q.t, sf.t))
    torch.cuda.synchronize()
    q.check("q")
    sf.check("sf")
    assert torch.equal(x.view(torch.uint16), before.view(torch.uint16)), "the input must not be written"
    return q.t.cpu().numpy(), sf.t.cpu().numpy()


@pytest.mark.parametrize("act_mode", [0, 1, 2])
@pytest.mark.parametrize("rows,F", [(1, 32), (5, 96), (129, 160), (64, 4096), (37, 4128), (300, 12288), (2049, 3072)])
def test_act_quantize_equals_two_calls_and_oracle_bound(mx, act_mode, rows, F):
    g = H.rng(rows + F + act_mode)
    cols = 2 * F if act_mode == 1 else F
    bits = H.normal_bf16(g, (rows, cols), 2.0)
    q2, sf2, act_bits = two_calls(mx, act_mode, bits, rows, F)
    q1, sf1 = one_call(mx, act_mode, bits, rows, F)
    assert np.array_equal(sf1, sf2), f"{(sf1 != sf2).sum()} scale bytes differ"
    assert np.array_equal(q1, q2), f"{(q1 != q2).sum()} of {q1.size} data bytes differ"
    # and the decoded values are the oracle's activation within the format's error bound
    if act_mode == 1:
        ref = orc.silu_mul(bits, F)
    else:
        ref = (orc.gelu_tanh_inplace if act_mode == 0 else orc.gelu_erf_inplace)(bits.copy())
    d = orc.dequantize_blockscaled(1, q1, sf1, 0.0, rows, F)
    assert rel_rms(d, bits_to_f32(ref).reshape(rows, F)) < ELEM_ERR[1]


@pytest.mark.parametrize("knob,value", [("stream_chunk_kb", 1), ("stream_chunk_kb", 2), ("stream_stages", 2),
                                        ("stream_warps", 3), ("stream_ctas_per_sm", 1)])
@pytest.mark.parametrize("act_mode", [0, 1])
def test_act_quantize_work_split(mx, act_mode, knob, value):
    g = H.rng(17 + value)
    rows, F = 1500, 1056
    bits = H.normal_bf16(g, (rows, 2 * F if act_mode == 1 else F), 1.5)
    q2, sf2, _ = two_calls(mx, act_mode, bits, rows, F)
    mx.ops.set_tuning(knob, value)
    try:
        q1, sf1 = one_call(mx, act_mode, bits, rows, F)
    finally:
        mx.ops.set_tuning(knob, 0)
    assert np.array_equal(sf1, sf2) and np.array_equal(q1, q2)


def test_act_quantize_argument_errors(mx):
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda")
    out = mx.ops.act_quantize_mxfp8(0, x, 4, 64)
    for kw in (dict(act_mode=3), dict(F=48), dict(act_mode=-1)):
        a = dict(act_mode=0, F=64)
        a.update(kw)
        with pytest.raises(mx.MxkError):
            mx.ops.act_quantize_mxfp8(a["act_mode"], x, 4, a["F"], out)
    with pytest.raises(mx.MxkError):
        mx.ops.act_quantize_mxfp8(0, x.view(-1)[1:].data_ptr(), 3, 64, out)
    mx.ops.act_quantize_mxfp8(0, x, 0, 64, out)
    torch.cuda.synchronize()


# ---- norm + modulation + MXFP8 quantisation in one pass ----

@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm", "rmsnorm_now"])
@pytest.mark.parametrize("rows,dim,plen", [(1, 32, 0), (7, 96, 3), (130, 3072, 41), (300, 5120, 0), (2049, 1152, 2049),
                                           (33, 4128, 5), (1200, 3072, 256), (64, 8192, 64)])
def test_norm_quantize_equals_two_calls_and_oracle_bound(mx, kind, rows, dim, plen):
    g = H.rng(rows * 3 + dim)
    x = H.normal_f32(g, (rows, dim), 1.3, 0.2)
    vecs = [H.normal_f32(g, dim, 0.3) for _ in range(4)]
    w = None if kind != "rmsnorm" else H.normal_f32(g, dim, 0.1, 1.0)
    xd, wd = H.to_dev(torch, x), (H.to_dev(torch, w) if w is not None else None)
    vd = [H.to_dev(torch, v) for v in vecs]
    sc, sh = mx.row_mod(vd[0], vd[1], plen), mx.row_mod(vd[2], vd[3], plen)
    eps = 1e-6
    bf = torch.empty(rows, dim, dtype=torch.bfloat16, device="cuda")
    q = H.Guarded(torch, (rows * dim,), torch.uint8)
    sf = H.Guarded(torch, (mx.ops.qscale_bytes(1, rows, dim),), torch.uint8)
    sf.t.fill_(0x5A)
    if kind == "layernorm":
        mx.ops.layernorm_mod(xd, rows, dim, eps, sc, sh, bf)
        mx.ops.layernorm_mod_quant_mxfp8(xd, rows, dim, eps, sc, sh, mx.ops.QMat(q.t, sf.t))
        ref = orc.layernorm_mod(x, eps, orc.mod(vecs[0], vecs[1], plen), orc.mod(vecs[2], vecs[3], plen))
    else:
        mx.ops.rmsnorm_mod(xd, rows, dim, eps, wd, sc, sh, bf)
        mx.ops.rmsnorm_mod_quant_mxfp8(xd, rows, dim, eps, wd, sc, sh, mx.ops.QMat(q.t, sf.t))
        ref = orc.rmsnorm_mod(x, eps, w, orc.mod(vecs[0], vecs[1], plen), orc.mod(vecs[2], vecs[3], plen))
    two = mx.ops.quantize_blockscaled(1, bf, dim, rows, dim)
    torch.cuda.synchronize()
    q.check("q")
    sf.check("sf")
    q1, sf1 = q.t.cpu().numpy(), sf.t.cpu().numpy()
    assert np.array_equal(sf1, two.sf.cpu().numpy()), "scale bytes differ from the two calls"
    assert np.array_equal(q1, two.q.cpu().numpy()), "data bytes differ from the two calls"
    d = orc.dequantize_blockscaled(1, q1, sf1, 0.0, rows, dim)
    assert rel_rms(d, bits_to_f32(ref).reshape(rows, dim)) < ELEM_ERR[1]


def test_norm_quantize_many_trips_per_cta(mx):
    """One CTA per SM, so every CTA wraps its ring of stages many times."""
    g = H.rng(3)
    rows, dim = 3000, 1024
    x = H.to_dev(torch, H.normal_f32(g, (rows, dim), 2.0))
    bf = torch.empty(rows, dim, dtype=torch.bfloat16, device="cuda")
    none = mx.row_mod()
    mx.ops.set_tuning("norm_ctas_per_sm", 1)
    try:
        mx.ops.layernorm_mod(x, rows, dim, 1e-6, none, none, bf)
        one = mx.ops.layernorm_mod_quant_mxfp8(x, rows, dim, 1e-6, none, none)
    finally:
        mx.ops.set_tuning("norm_ctas_per_sm", 0)
    two = mx.ops.quantize_blockscaled(1, bf, dim, rows, dim)
    torch.cuda.synchronize()
    assert torch.equal(one.q, two.q) and torch.equal(one.sf, two.sf)


def test_norm_quantize_argument_errors(mx):
    x = torch.zeros(4, 64, dtype=torch.float32, device="cuda")
    none = mx.row_mod()
    out = mx.ops.layernorm_mod_quant_mxfp8(x, 4, 64, 1e-6, none, none)
    with pytest.raises(mx.MxkError):  # dim not a multiple of 32
        mx.ops.layernorm_mod_quant_mxfp8(x, 4, 48, 1e-6, none, none, out)
    with pytest.raises(mx.MxkError):  # unaligned row
        mx.ops.layernorm_mod_quant_mxfp8(x.view(-1)[1:].data_ptr(), 3, 64, 1e-6, none, none, out)
    with pytest.raises(mx.MxkError):
        mx.ops.rmsnorm_mod_quant_mxfp8(x, 4, 64, 1e-6, None, none, none, mx.ops.QMat(out.q, None))
    mx.ops.rmsnorm_mod_quant_mxfp8(x, 0, 64, 1e-6, None, none, none, out)
    torch.cuda.synchronize()


@pytest.mark.parametrize("norm_mode", [0, 1])
@pytest.mark.parametrize("rows,dim,plen,tanh", [(1, 32, 0, 1), (7, 96, 3, 0), (130, 3072, 41, 1), (300, 5120, 0, 0), (1200, 3072, 256, 1),
                                                (64, 8192, 64, 0)])
def test_residual_norm_quantize_equals_the_two_calls(mx, norm_mode, rows, dim, plen, tanh):
    g = H.rng(rows * 5 + dim + norm_mode)
    x, ybits = H.normal_f32(g, (rows, dim), 1.3), H.normal_bf16(g, (rows, dim), 1.0)
    vecs = [H.to_dev(torch, H.normal_f32(g, dim, 0.3)) for _ in range(6)]
    w = H.to_dev(torch, H.normal_f32(g, dim, 0.1, 1.0)) if norm_mode == 1 else None
    gate, sc, sh = mx.row_mod(vecs[0], vecs[1], plen), mx.row_mod(vecs[2], vecs[3], plen), mx.row_mod(vecs[4], vecs[5], plen)
    x2, y = H.to_dev(torch, x), H.to_dev(torch, ybits)
    bf = torch.empty(rows, dim, dtype=torch.bfloat16, device="cuda")
    mx.ops.gated_residual_norm(x2, y, rows, dim, gate, tanh, norm_mode, 1e-6, w, sc, sh, bf)
    two = mx.ops.quantize_blockscaled(1, bf, dim, rows, dim)
    x1 = H.to_dev(torch, x)
    q = H.Guarded(torch, (rows * dim,), torch.uint8)
    sf = H.Guarded(torch, (mx.ops.qscale_bytes(1, rows, dim),), torch.uint8)
    sf.t.fill_(0x5A)
    mx.ops.gated_residual_norm_quant_mxfp8(x1, y, rows, dim, gate, tanh, norm_mode, 1e-6, w, sc, sh, mx.ops.QMat(q.t, sf.t))
    torch.cuda.synchronize()
    q.check("q")
    sf.check("sf")
    assert torch.equal(x1, x2), "residual stream differs from the two calls"
    assert torch.equal(sf.t, two.sf) and torch.equal(q.t, two.q)


@pytest.mark.parametrize("act_mode", [0, 1])
@pytest.mark.parametrize("rows,F", [(5, 96), (129, 160), (37, 4128), (300, 12288)])
def test_bias_act_quantize_equals_three_calls(mx, act_mode, rows, F):
    g = H.rng(rows + F + 7 * act_mode)
    cols = 2 * F if act_mode == 1 else F
    bits, bias = H.normal_bf16(g, (rows, cols), 2.0), H.normal_f32(g, cols, 0.5)
    bd = H.to_dev(torch, bias)
    x = H.to_dev(torch, bits)
    one = mx.ops.act_quantize_mxfp8(act_mode, x, rows, F, bias=bd)
    mx.ops.add_bias_bf16(x, bd, rows, cols)
    if act_mode == 1:
        act = torch.empty(rows, F, dtype=torch.bfloat16, device="cuda")
        mx.ops.silu_mul(x, rows, F, act)
    else:
        act = x
        mx.ops.gelu_tanh_inplace(act, rows * F)
    three = mx.ops.quantize_blockscaled(1, act, F, rows, F)
    torch.cuda.synchronize()
    assert torch.equal(one.sf, three.sf) and torch.equal(one.q, three.q)


def test_mxfp8_row_shards_on_tile_boundaries_equal_the_whole(mx):
    """Rows are independent and a scale tile holds 128 rows, so shards cut at multiples of 128 rows write
    disjoint parts of the same (q, sf): what a row-sharded run does with one shard per GPU."""
    g = H.rng(77)
    rows, K = 640, 1056
    bits = H.normal_bf16(g, (rows, K), 1.5)
    x = H.to_dev(torch, bits)
    whole = mx.ops.quantize_blockscaled(1, x, K, rows, K)
    q = torch.zeros_like(whole.q)
    sf = torch.zeros_like(whole.sf)
    tile = mx.ops.qscale_bytes(1, 128, K)
    for r0, n in ((0, 256), (256, 128), (384, 256)):
        part = mx.ops.QMat(q[r0 * K:(r0 + n) * K], sf[r0 // 128 * tile:(r0 + n) // 128 * tile])
        mx.ops.quantize_blockscaled(1, x[r0:r0 + n], K, n, K, part)
    torch.cuda.synchronize()
    assert torch.equal(q, whole.q) and torch.equal(sf, whole.sf)
