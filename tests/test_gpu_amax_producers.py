"""NVFP4 without the extra read pass: the ops that produce a tensor also leave its maximum on the
device (mxk_*_amax), and mxk_quantize_nvfp4_known_amax quantises from it in one pass.  The outputs
of the producing op must equal the plain op's bit for bit, the maximum must equal max |out| exactly,
and codes, scales and maximum must equal the two-pass mxk_quantize_blockscaled(NVFP4) byte for byte
(which tests/test_gpu_blockscale.py holds to the reference kernel's bytes)."""
import numpy as np
import pytest

import helpers as H

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["bulk_copy", "registers"])
def mx(request):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import miroxen_b200 as m
    m.lib()
    path = 1 if request.param == "bulk_copy" else 2
    m.set_tuning("norm_path", path)
    m.set_tuning("quant_path", path)
    yield m
    torch.cuda.synchronize()
    assert m.device_error() == 0
    m.set_tuning("norm_path", 0)
    m.set_tuning("quant_path", 0)


def true_amax(t):
    return float(t.float().abs().max().item())


def check_quant(mx, t, rows, K, amax):
    """One-pass NVFP4 from the producer's maximum against the two-pass quantiser."""
    two = mx.ops.quantize_blockscaled(mx.ops.Q_NVFP4, t, K, rows, K)
    one = mx.ops.quantize_nvfp4_known_amax(t, K, rows, K, amax)
    torch.cuda.synchronize()
    assert float(amax.item()) == float(two.amax.item()) == true_amax(t)
    assert torch.equal(one.q, two.q) and torch.equal(one.sf, two.sf)


def mods(mx, g, dim, plen):
    sc_t, sc_p, sh_t, sh_p = (H.to_dev(torch, H.normal_f32(g, dim, 0.3)) for _ in range(4))
    return mx.row_mod(sc_t, sc_p, plen), mx.row_mod(sh_t, sh_p, plen), (sc_t, sc_p, sh_t, sh_p)


@pytest.mark.parametrize("rows,dim,norm_mode", [(300, 3072, 0), (129, 5120, 1), (65, 4096, 0), (33, 5376, 1), (7, 96, 0), (1, 3072, 1)])
def test_norm_with_amax(mx, rows, dim, norm_mode):
    g = H.rng(rows + dim)
    x = H.to_dev(torch, H.normal_f32(g, (rows, dim), 3.0))
    w = H.to_dev(torch, H.normal_f32(g, dim, 0.1, 1.0)) if norm_mode == 1 else None
    sc, sh, keep = mods(mx, g, dim, rows // 3)
    plain = torch.empty((rows, dim), dtype=torch.bfloat16, device="cuda")
    out = H.Guarded(torch, (rows, dim), torch.bfloat16)
    amax = torch.full((1,), 123.0, dtype=torch.float32, device="cuda")   # stale content must not survive
    if norm_mode == 0:
        mx.layernorm_mod(x, rows, dim, 1e-6, sc, sh, plain)
        mx.layernorm_mod_amax(x, rows, dim, 1e-6, sc, sh, out.t, amax)
    else:
        mx.rmsnorm_mod(x, rows, dim, 1e-6, w, sc, sh, plain)
        mx.rmsnorm_mod_amax(x, rows, dim, 1e-6, w, sc, sh, out.t, amax)
    torch.cuda.synchronize()
    out.check("norm amax out")
    assert torch.equal(out.t, plain)
    assert float(amax.item()) == true_amax(plain)
    if dim % 32 == 0:
        check_quant(mx, out.t, rows, dim, amax)


@pytest.mark.parametrize("rows,dim,norm_mode", [(200, 3072, 0), (77, 5120, 1)])
def test_gated_residual_norm_with_amax(mx, rows, dim, norm_mode):
    g = H.rng(rows * 2 + dim)
    x0 = H.normal_f32(g, (rows, dim))
    y = H.to_dev(torch, H.normal_bf16(g, (rows, dim)))
    gate = H.to_dev(torch, H.normal_f32(g, dim, 0.7))
    w = H.to_dev(torch, H.normal_f32(g, dim, 0.1, 1.0)) if norm_mode == 1 else None
    sc, sh, keep = mods(mx, g, dim, rows // 2)
    xa, xb = H.to_dev(torch, x0), H.to_dev(torch, x0)
    oa = torch.empty((rows, dim), dtype=torch.bfloat16, device="cuda")
    ob = torch.empty((rows, dim), dtype=torch.bfloat16, device="cuda")
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    mx.gated_residual_norm(xa, y, rows, dim, mx.row_mod(gate), 1, norm_mode, 1e-6, w, sc, sh, oa)
    mx.gated_residual_norm_amax(xb, y, rows, dim, mx.row_mod(gate), 1, norm_mode, 1e-6, w, sc, sh, ob, amax)
    torch.cuda.synchronize()
    assert torch.equal(xa, xb) and torch.equal(oa, ob)
    assert float(amax.item()) == true_amax(oa)
    check_quant(mx, ob, rows, dim, amax)


@pytest.mark.parametrize("act_mode,rows,F,with_bias", [(0, 130, 12288, False), (0, 33, 3072, True), (1, 65, 13824, False),
                                                       (1, 40, 4096, True), (2, 20, 2048, False)])
def test_activation_with_amax(mx, act_mode, rows, F, with_bias):
    g = H.rng(rows + F + act_mode)
    width = 2 * F if act_mode == 1 else F
    src = H.to_dev(torch, H.normal_bf16(g, (rows, width), 2.0))
    bias = H.to_dev(torch, H.normal_f32(g, width, 0.2)) if with_bias else None
    plain = torch.empty((rows, F), dtype=torch.bfloat16, device="cuda")
    if act_mode == 1:
        if bias is not None:
            mx.bias_silu_mul(src, bias, rows, F, plain)
        else:
            mx.silu_mul(src, rows, F, plain)
    else:
        plain.copy_(src)
        if bias is not None:
            mx.add_bias_bf16(plain, bias, rows, F)
        (mx.gelu_tanh_inplace if act_mode == 0 else mx.gelu_erf_inplace)(plain, rows * F)
    amax = torch.full((1,), 7.0, dtype=torch.float32, device="cuda")
    if act_mode == 1:
        out = H.Guarded(torch, (rows, F), torch.bfloat16)
        mx.act_amax(act_mode, src, rows, F, out.t, amax, bias=bias)
    else:
        out = H.Guarded(torch, (rows, F), torch.bfloat16, fill=src)
        mx.act_amax(act_mode, out.t, rows, F, out.t, amax, bias=bias)   # in place
    torch.cuda.synchronize()
    out.check("act amax out")
    assert torch.equal(out.t, plain)
    assert float(amax.item()) == true_amax(plain)
    check_quant(mx, out.t, rows, F, amax)


def test_amax_argument_checks(mx):
    L = mx.lib()
    from miroxen_b200._lib import RowMod
    none = RowMod(None, None, 0)
    assert L.mxk_layernorm_mod_amax(256, 4, 64, 1e-6, none, none, 256, None, None) == -1
    assert L.mxk_act_amax(0, 256, None, 4, 64, 256, None, None) == -1
    assert L.mxk_act_amax(5, 256, None, 4, 64, 256, 256, None) == -1
    a = torch.full((1,), 5.0, dtype=torch.float32, device="cuda")
    assert L.mxk_act_amax(0, None, None, 0, 64, None, a.data_ptr(), None) == 0   # no rows: the maximum of nothing is 0
    torch.cuda.synchronize()
    assert float(a.item()) == 0.0
