"""Parity at the row counts the benchmark times (8704, 16 896 and 33 272 rows), not only on the small
blocks of the other files: the prefix / target switch at row 8192 or 16 384, the 8192-row chunking of the
video block, grids of more than one wave with interleaved row assignment, and the row ranges an 8-way
shard launches.  Inputs are the benchmark's own seeded buffers (miroxen_b200.workloads.BlockBuffers);
the checker is the exact CPU oracle on all host threads."""
import os

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
    try:
        n = len(os.sched_getaffinity(0))
    except Exception:
        n = os.cpu_count() or 1
    orc.set_threads(n)
    yield m
    torch.cuda.synchronize()
    assert m.device_error() == 0
    orc.set_threads(1)


def host(t):
    """device tensor -> numpy (bf16 as uint16 bit patterns)."""
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).cpu().numpy()
    return t.cpu().numpy()


def oracle_block(w, b):
    """The block's op sequence on the CPU oracle from the device buffers' initial contents."""
    rows, inner, F = b.rows, w.inner, w.F
    m = b.mods
    pl = b.args.scale1.prefix_len
    mod = lambda k: orc.mod(host(m[k + "_t"]), host(m[k + "_p"]), pl)
    nq, nk = host(m["norm_q"]), host(m["norm_k"])
    cos, sin = host(b.cos), host(b.sin)
    x = host(b.x).copy()
    out = {}

    def norm(sc, sh, wt):
        if w.norm_mode == 0:
            return orc.layernorm_mod(x, w.eps, mod(sc), mod(sh))
        return orc.rmsnorm_mod(x, w.eps, host(m[wt]), mod(sc), mod(sh))

    out["h1"] = norm("scale1", "shift1", "norm1_w")
    if w.packed_qkv:
        qkv = host(b.qkv)
        out["q_out"] = orc.head_norm_rope(qkv, rows, 3 * inner, 0, w.H, w.D, nq, w.eps, cos, sin, w.rot, w.rope_mode)
        out["k_out"] = orc.head_norm_rope(qkv, rows, 3 * inner, inner, w.H, w.D, nk, w.eps, cos, sin, w.rot, w.rope_mode)
        out["v_out"] = orc.head_norm_rope(qkv, rows, 3 * inner, 2 * inner, w.H, w.D, None, 0.0, None, None, 0, 0)
        del qkv
    else:
        out["q_out"] = orc.head_norm_rope(host(b.q_in), rows, inner, 0, w.H, w.D, nq, w.eps, cos, sin, w.rot, w.rope_mode)
        out["k_out"] = orc.head_norm_rope(host(b.k_in), rows, inner, 0, w.H, w.D, nk, w.eps, cos, sin, w.rot, w.rope_mode)
    orc.gated_residual(x, host(b.attn_o), mod("gate1"), w.gate_tanh)
    out["h2"] = norm("scale2", "shift2", "norm2_w")
    out["act"] = orc.gelu_tanh_inplace(host(b.act).copy()) if w.act_mode == 0 else orc.silu_mul(host(b.act2), F)
    orc.gated_residual(x, host(b.mlp_o), mod("gate2"), w.gate_tanh)
    out["x"] = x
    return out


def buffers(w, seed):
    from miroxen_b200.workloads import BlockBuffers, make_mods, rope_tables_for
    cos, sin = rope_tables_for(w)
    return BlockBuffers(w, w.rows, w.prefix_rows, seed=seed, mods=make_mods(w, seed=1000), cos=cos, sin=sin)


def compare(w, b, ref, what):
    for k in ("h1", "q_out", "k_out", "h2", "act"):
        H.assert_bf16_close(host(getattr(b, k)), ref[k], f"{what} {k}")
    if w.packed_qkv:
        assert np.array_equal(host(b.v_out), ref["v_out"].reshape(host(b.v_out).shape)), f"{what} v_out"
    H.assert_f32_close(host(b.x), ref["x"], f"{what} x")


# (the two 33 272-row shapes take the oracle about a minute each on 16 host threads: one chain each, the drop-in one on the
# benchmark shape and the fused one on the reference's true widths; both chains run at 8704 rows)
CASES = [("qwen1024", 0), ("qwen1024", 1), ("qwen2048", 0), ("h3video", 0), ("qwen21_true", 0), ("h3_true", 1)]


@pytest.mark.parametrize("name,fused", CASES)
def test_block_chain_at_the_benchmarked_row_counts(mx, name, fused):
    from miroxen_b200.workloads import WORKLOADS
    w = WORKLOADS[name]
    b = buffers(w, seed=3)
    ref = oracle_block(w, b)  # before the launch: x and (GELU) act are updated in place
    b.args.fused = fused
    mx.dit_block_ops(b.args)
    torch.cuda.synchronize()
    compare(w, b, ref, f"{name} fused={fused}")


@pytest.mark.parametrize("name,split", [("qwen1024", "rows"), ("qwen2048", "rows"), ("h3video", "frames"), ("h3video", "rows")])
@pytest.mark.parametrize("fused", [0, 1])
def test_eight_way_shards_equal_the_single_launch_bit_for_bit(mx, name, split, fused):
    """Rows [r0, r0 + n) launched the way a rank of an 8-GPU job launches them (offset pointers, prefix
    boundary moved by r0) must give exactly the bits of the whole-sequence launch: every op is row-independent
    (the reference checks its 2-card split the same way, tests/h3_dit_parity_test.cpp:105)."""
    from miroxen_b200 import sharding
    from miroxen_b200.workloads import WORKLOADS
    w = WORKLOADS[name]
    whole, parts = buffers(w, seed=5), buffers(w, seed=5)
    whole.args.fused = fused
    mx.dit_block_ops(whole.args)
    shards = []
    for rank in range(8):
        if split == "frames":
            s = sharding.shard_frames(w.frames, w.rows_per_frame, w.rows - w.frames * w.rows_per_frame, 8, rank)
        else:
            s = sharding.shard_rows(w.rows, 8, rank)
        shards.append(s)
        a = parts.shard_args(s.row0, s.rows)
        a.fused = fused
        assert a.scale1.prefix_len == s.shift_prefix(w.prefix_rows)
        mx.dit_block_ops(a)
    assert sharding.covers(shards, w.rows)
    torch.cuda.synchronize()
    keys = ["h1", "q_out", "k_out", "h2", "act", "x"] + (["v_out"] if w.packed_qkv else [])
    for k in keys:
        assert torch.equal(getattr(whole, k), getattr(parts, k)), f"{name} {split} shards differ from the whole in {k}"
