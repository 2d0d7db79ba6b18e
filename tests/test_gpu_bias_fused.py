"""The bias-folding entry points: byte-identical to mxk_add_bias_bf16 followed by the plain op of this library,
and within the usual tolerance of the CPU oracle's composition of the reference ops (src/kernels/ops.cu:249-262
add_bias_bf16, then :220-226 / :121-128 / :73-84)."""
import numpy as np
import pytest

import helpers as H
from oracle import binding as orc

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mx():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import miroxen_b200 as m
    m.lib()
    yield m
    torch.cuda.synchronize()
    assert m.device_error() == 0


SHAPES = [(1, 8), (5, 96), (129, 160), (64, 4096), (37, 4136), (300, 12288), (2049, 3072)]


@pytest.mark.parametrize("rows,F", SHAPES)
def test_bias_gelu_equals_two_calls_and_oracle(mx, rows, F):
    g = H.rng(rows + F)
    bits, bias = H.normal_bf16(g, (rows, F), 2.0), H.normal_f32(g, F, 0.5)
    bd = H.to_dev(torch, bias)
    two = H.to_dev(torch, bits)
    mx.ops.add_bias_bf16(two, bd, rows, F)
    mx.ops.gelu_tanh_inplace(two, rows * F)
    one = H.to_dev(torch, bits)
    mx.ops.bias_gelu_tanh_inplace(one, bd, rows, F)
    torch.cuda.synchronize()
    assert np.array_equal(H.bits(one), H.bits(two))
    ref = orc.gelu_tanh_inplace(orc.add_bias_bf16(bits.copy(), bias))
    H.assert_bf16_close(H.bits(one), ref, "bias + gelu")


@pytest.mark.parametrize("rows,F", SHAPES)
def test_bias_silu_mul_equals_two_calls_and_oracle(mx, rows, F):
    g = H.rng(rows * 2 + F)
    bits, bias = H.normal_bf16(g, (rows, 2 * F), 2.0), H.normal_f32(g, 2 * F, 0.5)
    bd = H.to_dev(torch, bias)
    gu = H.to_dev(torch, bits)
    before = gu.clone()
    one = H.Guarded(torch, (rows, F), torch.bfloat16)
    mx.ops.bias_silu_mul(gu, bd, rows, F, one.t)
    torch.cuda.synchronize()
    one.check("out")
    assert torch.equal(gu.view(torch.uint16), before.view(torch.uint16)), "the input must not be written"
    mx.ops.add_bias_bf16(gu, bd, rows, 2 * F)
    two = torch.empty(rows, F, dtype=torch.bfloat16, device="cuda")
    mx.ops.silu_mul(gu, rows, F, two)
    torch.cuda.synchronize()
    assert np.array_equal(H.bits(one.t), H.bits(two))
    ref = orc.silu_mul(orc.add_bias_bf16(bits.copy(), bias), F)
    H.assert_bf16_close(H.bits(one.t), ref, "bias + silu_mul")


@pytest.mark.parametrize("rows,dim,plen,tanh", [(1, 8, 0, 1), (7, 96, 3, 0), (130, 3072, 41, 1), (300, 5120, 0, 0),
                                                (2049, 1152, 2049, 1), (33, 4136, 5, 1), (64, 8192, 64, 0)])
def test_gated_residual_bias_equals_two_calls_and_oracle(mx, rows, dim, plen, tanh):
    g = H.rng(rows + dim)
    x, ybits, bias = H.normal_f32(g, (rows, dim)), H.normal_bf16(g, (rows, dim), 1.5), H.normal_f32(g, dim, 0.5)
    gt, gp = H.normal_f32(g, dim, 0.7), H.normal_f32(g, dim, 0.7)
    gtd, gpd, bd = H.to_dev(torch, gt), H.to_dev(torch, gp), H.to_dev(torch, bias)
    gate = mx.row_mod(gtd, gpd, plen)
    x2, y2 = H.to_dev(torch, x), H.to_dev(torch, ybits)
    mx.ops.add_bias_bf16(y2, bd, rows, dim)
    mx.ops.gated_residual(x2, y2, rows, dim, gate, tanh)
    x1, y1 = H.to_dev(torch, x), H.to_dev(torch, ybits)
    mx.ops.gated_residual_bias(x1, y1, bd, rows, dim, gate, tanh)
    torch.cuda.synchronize()
    assert torch.equal(y1.view(torch.uint16), H.to_dev(torch, ybits).view(torch.uint16)), "y must not be written"
    assert torch.equal(x1, x2)
    ref = orc.gated_residual(x.copy(), orc.add_bias_bf16(ybits.copy(), bias), orc.mod(gt, gp, plen), tanh)
    H.assert_f32_close(x1.cpu().numpy(), ref, "bias + gated_residual")


def test_null_bias_is_the_plain_op_and_bad_shapes_are_refused(mx):
    g = H.rng(1)
    bits = H.normal_bf16(g, (16, 64), 1.0)
    a, b = H.to_dev(torch, bits), H.to_dev(torch, bits)
    mx.ops.bias_gelu_tanh_inplace(a, None, 16, 64)
    mx.ops.gelu_tanh_inplace(b, 16 * 64)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.uint16), b.view(torch.uint16))
    bias = torch.zeros(64, device="cuda")
    with pytest.raises(mx.MxkError):  # F not a multiple of 8
        mx.ops.bias_gelu_tanh_inplace(a, bias, 16, 60)
    with pytest.raises(mx.MxkError):  # unaligned
        mx.ops.bias_gelu_tanh_inplace(a.view(-1)[1:].data_ptr(), bias, 15, 64)
    x = torch.zeros(4, 12, device="cuda")
    y = torch.zeros(4, 12, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(mx.MxkError):  # dim not a multiple of 8
        mx.ops.gated_residual_bias(x, y, bias, 4, 12, mx.row_mod(), 0)


@pytest.mark.parametrize("knob,value", [("stream_chunk_kb", 1), ("stream_stages", 2), ("stream_warps", 3), ("stream_ctas_per_sm", 1)])
def test_bias_act_work_split(mx, knob, value):
    g = H.rng(5 + value)
    rows, F = 1500, 1056
    bits, bias = H.normal_bf16(g, (rows, 2 * F), 1.5), H.normal_f32(g, 2 * F, 0.3)
    bd = H.to_dev(torch, bias)
    want_g = orc.gelu_tanh_inplace(orc.add_bias_bf16(bits[:, :F].copy(), bias[:F]))
    want_s = orc.silu_mul(orc.add_bias_bf16(bits.copy(), bias), F)
    mx.ops.set_tuning(knob, value)
    try:
        xg = H.to_dev(torch, np.ascontiguousarray(bits[:, :F]))
        mx.ops.bias_gelu_tanh_inplace(xg, bd, rows, F)
        out = torch.empty(rows, F, dtype=torch.bfloat16, device="cuda")
        mx.ops.bias_silu_mul(H.to_dev(torch, bits), bd, rows, F, out)
        torch.cuda.synchronize()
    finally:
        mx.ops.set_tuning(knob, 0)
    H.assert_bf16_close(H.bits(xg), want_g, "bias + gelu")
    H.assert_bf16_close(H.bits(out), want_s, "bias + silu_mul")
