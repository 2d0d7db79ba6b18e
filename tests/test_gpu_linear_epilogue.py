"""The tensor-core linear layer with the following op in its epilogue (mxk_linear_bf16,
mxk_linear_gated_residual) against the calls it replaces: the library GEMM (torch.matmul on bf16,
i.e. cuBLAS, which is what the reference's linear() calls, src/core/weights.cpp:159-177), then
mxk_add_bias_bf16, then mxk_gated_residual.  The GEMMs accumulate in different orders, so a bf16
output may differ by one unit in the last place (tolerance of tests/helpers.py, stated there); the
residual stream may then differ by |act(gate)| times that."""
import numpy as np
import pytest

import helpers as H

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["cta_pair", "single_cta"])
def mx(request):
    """Every test runs with the two-CTA form (a cluster of two CTAs per 256 x 256 tile, the default for M > 128) and
    with the single-CTA form (128 x 256 tiles)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import miroxen_b200 as m
    m.lib()
    m.set_tuning("linear_ctas", 2 if request.param == "cta_pair" else 1)
    yield m
    torch.cuda.synchronize()
    m.set_tuning("linear_ctas", 0)
    assert m.device_error() == 0, "a bounded wait of the GEMM ran out"


def operands(M, N, K, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    A = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn((N, K), generator=g, device="cuda") / (K ** 0.5)).to(torch.bfloat16)
    bias = torch.randn(N, generator=g, device="cuda") * 0.1
    return A, W, bias


SHAPES = [(128, 256, 64), (256, 512, 128), (1000, 3072, 3072), (5, 320, 200), (129, 32, 8), (2176, 3072, 12288), (300, 5120, 1024)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_linear_bf16_equals_the_fp32_product(mx, M, N, K, with_bias):
    A, W, bias = operands(M, N, K, M + N + K)
    y = H.Guarded(torch, (M, N), torch.bfloat16)
    mx.linear_bf16(A, W, bias if with_bias else None, M, N, K, y.t)
    torch.cuda.synchronize()
    y.check("linear y")
    prod = (A.float() @ W.float().T).to(torch.bfloat16)     # fp32 accumulate, rounded as the GEMM output is
    lib_prod = A @ W.T                                      # the library GEMM the reference calls
    if not with_bias:
        H.assert_bf16_close(H.bits(y.t), H.bits(prod), f"linear {M}x{N}x{K}")
        H.assert_bf16_close(H.bits(y.t), H.bits(lib_prod), f"linear vs cuBLAS {M}x{N}x{K}")
        return
    # with a bias the product is rounded to bf16 BEFORE the bias is added (add_bias_bf16 reads the stored bf16):
    # two GEMMs that round one product a unit apart then differ by that unit whatever the sum is, so the bound
    # is one bf16 unit of the product plus one of the sum
    for name, p_ in (("fp32 product", prod), ("cuBLAS", lib_prod)):
        ref = (p_.float() + bias).to(torch.bfloat16)
        err = (y.t.float() - ref.float()).abs()
        # one bf16 unit in the last place is at most 2^-7 of the value
        tol = 2.0 ** -7 * (torch.clamp(p_.float().abs(), min=H.BF16_FLOOR) + torch.clamp(ref.float().abs(), min=H.BF16_FLOOR))
        assert bool((err <= tol).all()), f"linear + bias vs {name} {M}x{N}x{K}: {int((err > tol).sum())} beyond tolerance"
        assert float((y.t != ref).float().mean()) < 0.02


@pytest.mark.parametrize("group_m", [1, 3, 5])
def test_tile_order_does_not_change_a_result(mx, group_m):
    """The persistent loop numbers its tiles in bands of `linear_group_m` row tiles; every band height (a last band
    lower than the others included: 1000 rows are 4 pair tiles or 8 single tiles) gives the same bits, because a tile's
    arithmetic does not depend on who computes it when."""
    M, N, K = 1000, 3072, 512
    A, W, bias = operands(M, N, K, 77)
    want = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    mx.linear_bf16(A, W, bias, M, N, K, want)
    mx.set_tuning("linear_group_m", group_m)
    try:
        y = H.Guarded(torch, (M, N), torch.bfloat16)
        mx.linear_bf16(A, W, bias, M, N, K, y.t)
        torch.cuda.synchronize()
    finally:
        mx.set_tuning("linear_group_m", 0)
    y.check("linear y")
    assert torch.equal(y.t, want)


@pytest.mark.parametrize("M,N,K", [(1000, 3072, 3072), (272, 3072, 12288), (130, 5120, 512), (5, 320, 200)])
@pytest.mark.parametrize("mode", ["tanh_prefix_bias", "identity", "none"])
def test_linear_gated_residual_equals_the_separate_calls(mx, M, N, K, mode):
    A, W, bias = operands(M, N, K, M + K)
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    x0 = torch.randn((M, N), generator=g, device="cuda")
    gt, gp = torch.randn(N, generator=g, device="cuda") * 0.7, torch.randn(N, generator=g, device="cuda") * 0.7
    if mode == "tanh_prefix_bias":
        gate, tanh, b = mx.row_mod(gt, gp, M // 2 + 1), 1, bias
    elif mode == "identity":
        gate, tanh, b = mx.row_mod(gt), 0, None
    else:
        gate, tanh, b = None, 0, None
    # the calls it replaces
    y = A @ W.T
    if b is not None:
        mx.add_bias_bf16(y, b, M, N)
    x_ref = x0.clone()
    mx.gated_residual(x_ref, y, M, N, gate, tanh)
    x = H.Guarded(torch, (M, N), torch.float32, fill=x0)
    mx.linear_gated_residual(A, W, b, M, N, K, x.t, gate, tanh)
    torch.cuda.synchronize()
    x.check("fused x")
    # |x - x_ref| <= |act(gate)| * (one bf16 ulp of y, or the floor of tests/helpers.py) + fp32 rounding of the update
    act = torch.ones(N, device="cuda") if gate is None else (torch.tanh(gt) if tanh else gt)
    bound_rows = act.abs().expand(M, N).clone()
    if mode == "tanh_prefix_bias":
        bound_rows[:M // 2 + 1] = torch.tanh(gp).abs()
    ulp = torch.maximum(y.float().abs(), torch.tensor(H.BF16_FLOOR, device="cuda")) * 2.0 ** -7   # one bf16 unit is at most 2^-7 of the value
    tol = bound_rows * ulp + H.F32_REL * torch.maximum(x_ref.abs(), torch.tensor(1.0, device="cuda"))
    err = (x.t - x_ref).abs()
    assert bool((err <= tol).all()), f"{int((err > tol).sum())} of {err.numel()} beyond tolerance, worst {float((err - tol).max()):.3e}"
    # the two GEMMs round nearly every element the same way: the results should agree exactly almost everywhere
    assert float((x.t != x_ref).float().mean()) < 0.02


@pytest.mark.parametrize("M,Hh,K,rot,mode,n_t,with_bias", [(300, 24, 3072, 128, 1, 2, True), (1000, 40, 1024, 128, 2, 3, False),
                                                          (130, 56, 512, 96, 2, 3, True), (5, 2, 64, 64, 1, 1, False)])
def test_linear_qkv_norm_rope_equals_the_separate_calls(mx, M, Hh, K, rot, mode, n_t, with_bias):
    """QKV projection + head_norm_rope in one kernel against the library GEMM + add_bias_bf16 + mxk_qkv_norm_rope.
    A bf16 product that the two GEMMs round a unit apart moves its whole head by a relative 2^-7 / sqrt(128) at most
    and its own element by one unit, so the outputs are compared at two bf16 units."""
    D, inner = 128, Hh * 128
    N = n_t * inner
    A, W, bias = operands(M, N, K, M + Hh + K)
    g = torch.Generator(device="cuda")
    g.manual_seed(21)
    nq = 1 + 0.05 * torch.randn(D, generator=g, device="cuda")
    nk = 1 + 0.05 * torch.randn(D, generator=g, device="cuda")
    ang = torch.rand((M, rot // 2), generator=g, device="cuda") * 6.2 - 3.1
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    norms, rots, modes = [nq, nk, None][:n_t], [rot, rot, 0][:n_t], [mode, mode, 0][:n_t]
    b = bias if with_bias else None
    # the calls it replaces
    y = A @ W.T
    if b is not None:
        mx.add_bias_bf16(y, b, M, N)
    ref = [torch.empty((M, Hh, D), dtype=torch.bfloat16, device="cuda") for _ in range(n_t)]
    mx.qkv_norm_rope([mx.HeadSpec(y, N, i * inner, norms[i], ref[i], rots[i], modes[i]) for i in range(n_t)], M, Hh, D, 1e-6, cos, sin)
    outs = [H.Guarded(torch, (M, Hh, D), torch.bfloat16) for _ in range(n_t)]
    mx.linear_qkv_norm_rope(A, W, b, M, K, Hh, D, [mx.HeadSpec(None, 0, 0, norms[i], outs[i].t, rots[i], modes[i]) for i in range(n_t)],
                            1e-6, cos, sin)
    torch.cuda.synchronize()
    for i in range(n_t):
        outs[i].check(f"tensor {i}")
        got, want = outs[i].t.float(), ref[i].float()
        err = (got - want).abs()
        # rotation mixes two channels: bound by the larger of the pair, approximated by the head's largest magnitude
        scale = torch.clamp(want.abs().amax(dim=-1, keepdim=True), min=H.BF16_FLOOR)
        tol = 2.0 ** -6 * torch.maximum(want.abs(), 0.25 * scale)
        assert bool((err <= tol).all()), f"tensor {i}: {int((err > tol).sum())} of {err.numel()} beyond tolerance, worst {float((err - tol).max()):.3e}"
        assert float((outs[i].t != ref[i]).float().mean()) < 0.05, f"tensor {i}: too many elements differ"


@pytest.mark.parametrize("M,N,K", [(1000, 3072, 512), (272, 12288, 3072), (130, 320, 200), (5, 64, 64)])
@pytest.mark.parametrize("act_mode", [0, 2])
@pytest.mark.parametrize("with_bias", [False, True])
def test_linear_act_equals_linear_then_the_activation(mx, M, N, K, act_mode, with_bias):
    """linear() + gelu in one kernel.  Against this library's own linear layer followed by the stand-alone activation
    the result is the same bits (same tiles, same accumulation order, same activation arithmetic); against the library
    GEMM + add_bias_bf16 + the activation it is within what one unit of the product and one of the biased sum can move
    the output (|gelu'| <= 1.13) plus one unit of the output."""
    A, W, bias = operands(M, N, K, M + N + K + act_mode)
    b = bias if with_bias else None
    act = mx.gelu_tanh_inplace if act_mode == 0 else mx.gelu_erf_inplace
    same = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    mx.linear_bf16(A, W, b, M, N, K, same)
    act(same, M * N)
    prod = A @ W.T
    y = prod.clone()
    if b is not None:
        mx.add_bias_bf16(y, b, M, N)
    ref = y.clone()
    act(ref, M * N)
    out = H.Guarded(torch, (M, N), torch.bfloat16)
    mx.linear_act(A, W, b, M, N, K, act_mode, out.t)
    torch.cuda.synchronize()
    out.check("linear_act y")
    assert torch.equal(out.t, same)
    floor = lambda t: torch.clamp(t.float().abs(), min=H.BF16_FLOOR)
    tol = 2.0 ** -7 * (1.2 * (floor(prod) + floor(y)) + floor(ref))
    err = (out.t.float() - ref.float()).abs()
    assert bool((err <= tol).all()), f"{int((err > tol).sum())} of {err.numel()} beyond tolerance, worst {float((err - tol).max()):.3e}"
    assert float((out.t != ref).float().mean()) < 0.03


@pytest.mark.parametrize("M,F,K", [(1000, 1536, 512), (272, 13824, 1024), (300, 12288, 3072), (130, 160, 200), (5, 32, 64), (2176, 3456, 256)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_linear_silu_mul_equals_linear_then_silu_mul(mx, M, F, K, with_bias):
    """The first MLP projection with silu_mul in its epilogue: W [2F, K] = gate rows then up rows.  Same bits as this
    library's linear layer on the whole weight followed by the stand-alone silu_mul; within the propagated rounding of
    the library GEMM + add_bias_bf16 + silu_mul (|silu'| <= 1.1, |silu(g)| <= |g|).  F = 13824, 3456 and 160 are not
    whole numbers of 128-column tiles: their last tile's gate rows run into the up rows and must be ignored."""
    A, W, bias = operands(M, 2 * F, K, M + F + K)
    b = bias if with_bias else None
    gu_same = torch.empty((M, 2 * F), dtype=torch.bfloat16, device="cuda")
    mx.linear_bf16(A, W, b, M, 2 * F, K, gu_same)
    same = torch.empty((M, F), dtype=torch.bfloat16, device="cuda")
    mx.silu_mul(gu_same, M, F, same)
    prod = A @ W.T
    gu = prod.clone()
    if b is not None:
        mx.add_bias_bf16(gu, b, M, 2 * F)
    ref = torch.empty((M, F), dtype=torch.bfloat16, device="cuda")
    mx.silu_mul(gu, M, F, ref)
    out = H.Guarded(torch, (M, F), torch.bfloat16)
    mx.linear_silu_mul(A, W, b, M, F, K, out.t)
    torch.cuda.synchronize()
    out.check("linear_silu_mul out")
    assert torch.equal(out.t, same)
    floor = lambda t: torch.clamp(t.float().abs(), min=H.BF16_FLOOR)
    g, u, pg, pu = gu[:, :F], gu[:, F:], prod[:, :F], prod[:, F:]
    tol = 2.0 ** -7 * (1.1 * floor(u) * (floor(pg) + floor(g)) + floor(g) * (floor(pu) + floor(u)) + floor(ref))
    err = (out.t.float() - ref.float()).abs()
    assert bool((err <= tol).all()), f"{int((err > tol).sum())} of {err.numel()} beyond tolerance, worst {float((err - tol).max()):.3e}"
    assert float((out.t != ref).float().mean()) < 0.05


def test_linear_argument_checks(mx):
    L = mx.lib()
    from miroxen_b200._lib import RowMod
    none = RowMod(None, None, 0)
    assert L.mxk_linear_bf16(256, 256, None, 4, 33, 64, 256, None) == -1      # N % 32
    assert L.mxk_linear_bf16(256, 256, None, 4, 64, 12, 256, None) == -1      # K % 8
    assert L.mxk_linear_bf16(258, 256, None, 4, 64, 64, 256, None) == -1      # alignment
    assert L.mxk_linear_bf16(None, None, None, 0, 64, 64, None, None) == 0    # no rows
    assert L.mxk_linear_gated_residual(256, 256, None, 4, 64, 64, None, none, 0, None) == -1
    assert L.mxk_linear_act(256, 256, None, 4, 64, 64, 1, 256, None) == -1      # silu_mul is not an in-place activation
    assert L.mxk_linear_act(256, 256, None, 4, 64, 64, 0, None, None) == -1     # null y
    assert L.mxk_linear_silu_mul(256, 256, None, 4, 48, 64, 256, None) == -1    # F % 32
    assert L.mxk_linear_silu_mul(256, 256, None, 0, 64, 64, None, None) == 0    # no rows
    from miroxen_b200.ops import HeadTensor
    arr = (HeadTensor * 1)(HeadTensor(None, 0, 0, None, 256, 0, 0))
    assert L.mxk_linear_qkv_norm_rope(256, 256, None, 4, 64, 3, 128, arr, 1, 1e-6, None, None, None) == -1   # odd head count
    assert L.mxk_linear_qkv_norm_rope(256, 256, None, 4, 64, 2, 64, arr, 1, 1e-6, None, None, None) == -1    # D != 128
