"""GPU parity for the table builders (bit-exact against the oracle's libm evaluation) and for the
block call-pattern drivers (device chain, fused chain, host-buffer pipeline)."""
import ctypes as C

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
    return m


QWEN_LAYOUTS = [
    [("image", 32, 32), ("text", 128)],                       # benchmark config 1 ordering: image then text
    [("text", 77), ("image", 64, 64)],                        # text to image
    [("text", 20), ("image", 24, 40), ("text", 9), ("image", 17, 31), ("text", 3), ("image", 128, 128)],  # edit layout
    [("image", 1, 1)],
]


@pytest.mark.parametrize("segs", QWEN_LAYOUTS)
def test_qwen_rope_table_bit_exact(mx, segs):
    from miroxen_b200 import rope_tables
    cos, sin = rope_tables.qwen_rope_table(segs)
    rc, rs = orc.qwen_rope_table(segs)
    torch.cuda.synchronize()
    assert cos.shape == rc.shape
    assert np.array_equal(cos.cpu().numpy().view(np.uint32), rc.view(np.uint32))
    assert np.array_equal(sin.cpu().numpy().view(np.uint32), rs.view(np.uint32))


@pytest.mark.parametrize("T,F_lat,Hh,W,A,anchors", [
    (512, 21, 60, 104, 0, []),            # benchmark config 5 geometry
    (37, 7, 30, 52, 25, ["first", "last"]),
    (5, 2, 4, 6, 3, ["last"]),
])
def test_h3_rope_table_bit_exact(mx, T, F_lat, Hh, W, A, anchors):
    from miroxen_b200 import rope_tables
    inv_freq = (1.0 / (10000.0 ** (np.arange(16, dtype=np.float64) * 2 / 32))).astype(np.float32)
    cos, sin = rope_tables.h3_rope_table(T, F_lat, Hh, W, A, anchors, inv_freq)
    pos = orc.h3_positions(T, F_lat, Hh, W, A, anchors)
    rc, rs = orc.h3_rope_table(pos, inv_freq)
    torch.cuda.synchronize()
    assert cos.shape == rc.shape
    assert np.array_equal(cos.cpu().numpy().view(np.uint32), rc.view(np.uint32))
    assert np.array_equal(sin.cpu().numpy().view(np.uint32), rs.view(np.uint32))


@pytest.mark.parametrize("name", ["mixed", "video_with_track", "no_text", "h3_480p_one_image"])
def test_h3_ref2va_rope_table_bit_exact(mx, name):
    """The reference-conditioned layout (src/models/minimax_h3/layout.cpp:121-188): table gathered on the GPU from
    the host look-up tables == libm on the positions of the reference's own host code."""
    import sys
    from pathlib import Path
    from miroxen_b200 import rope_tables
    gold_dir = Path(__file__).resolve().parent / "golden"
    sys.path.insert(0, str(gold_dir))
    from make_h3_ref2va_positions import CASES
    inv_freq = (1.0 / (10000.0 ** (np.arange(16, dtype=np.float64) * 2 / 32))).astype(np.float32)
    cos, sin = rope_tables.h3_ref2va_rope_table(*CASES[name], inv_freq)
    pos = np.load(gold_dir / "h3_ref2va_positions.npz")[name]
    rc, rs = orc.h3_rope_table(pos, inv_freq)
    torch.cuda.synchronize()
    assert cos.shape == rc.shape
    assert np.array_equal(cos.cpu().numpy().view(np.uint32), rc.view(np.uint32))
    assert np.array_equal(sin.cpu().numpy().view(np.uint32), rs.view(np.uint32))


def test_qwen_timestep_embedding_bit_exact(mx):
    from miroxen_b200 import rope_tables
    ts = [0.0, 0.5, 1.0, 0.999, 0.001, 0.123456, 0.7071] + [k / 1000.0 for k in range(0, 1000, 7)]
    for t in ts:
        ref = orc.qwen_timestep_embedding(t)
        host = rope_tables.qwen_timestep_embedding(t, on_host=True).numpy()
        dev = rope_tables.qwen_timestep_embedding(t).cpu().numpy()
        assert np.array_equal(host.view(np.uint32), ref.view(np.uint32)), t
        assert np.array_equal(dev.view(np.uint32), ref.view(np.uint32)), t


def test_h3_time_basis_bit_exact(mx):
    from miroxen_b200 import rope_tables
    g = H.rng(9)
    table = H.normal_f32(g, (1025, 8))
    ts = np.concatenate([g.uniform(-0.2, 1.2, 200).astype(np.float32), np.array([0, 1, 0.5, 1023 / 1024], np.float32)])
    ref = orc.h3_time_basis(ts, table)
    out = rope_tables.h3_time_basis(torch.from_numpy(ts).cuda(), torch.from_numpy(table).cuda())
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))


def make_block(mx, g, rows, dim, Hh, D, F, norm_mode, act_mode, rot, rope_mode, packed, n_prefix, host=False):
    """Seeded inputs of one block; returns (numpy dict, tensor dict, BlockArgs)."""
    inner = Hh * D
    n = {}
    n["x"] = H.normal_f32(g, (rows, dim))
    stride = 3 * inner if packed else inner
    n["qkv"] = H.normal_bf16(g, (rows, stride)) if packed else None
    n["q_in"] = None if packed else H.normal_bf16(g, (rows, inner))
    n["k_in"] = None if packed else H.normal_bf16(g, (rows, inner))
    n["attn_o"] = H.normal_bf16(g, (rows, dim))
    n["mlp_o"] = H.normal_bf16(g, (rows, dim))
    n["act"] = H.normal_bf16(g, (rows, F))
    n["act2"] = H.normal_bf16(g, (rows, 2 * F)) if act_mode == 1 else None
    for k in ("shift1", "scale1", "gate1", "shift2", "scale2", "gate2"):
        n[k + "_t"], n[k + "_p"] = H.normal_f32(g, dim, 0.3), H.normal_f32(g, dim, 0.3)
    n["norm1_w"] = H.normal_f32(g, dim, 0.1, 1.0) if norm_mode == 1 else None
    n["norm2_w"] = H.normal_f32(g, dim, 0.1, 1.0) if norm_mode == 1 else None
    n["norm_q"], n["norm_k"] = H.normal_f32(g, D, 0.05, 1.0), H.normal_f32(g, D, 0.05, 1.0)
    ang = g.uniform(-3, 3, (rows, rot // 2)).astype(np.float32)
    n["cos"], n["sin"] = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)

    def place(a, is_data):
        if a is None:
            return None
        t = torch.from_numpy(np.ascontiguousarray(a))
        if a.dtype == np.uint16:
            t = t.view(torch.bfloat16)
        return t.pin_memory() if (host and is_data) else t.cuda()

    data_keys = {"x", "qkv", "q_in", "k_in", "attn_o", "mlp_o", "act", "act2", "cos", "sin"}
    t = {k: place(v, k in data_keys) for k, v in n.items()}
    mk = (lambda *s: torch.empty(s, dtype=torch.bfloat16).pin_memory()) if host else \
         (lambda *s: torch.empty(s, dtype=torch.bfloat16, device="cuda"))
    for k, shape in (("h1", (rows, dim)), ("h2", (rows, dim)), ("q_out", (rows, Hh, D)), ("k_out", (rows, Hh, D)),
                     ("v_out", (rows, Hh, D))):
        t[k] = mk(*shape)
    a = mx.BlockArgs()
    a.rows, a.dim, a.F, a.H, a.D = rows, dim, F, Hh, D
    a.norm_mode, a.eps, a.act_mode, a.fused, a.chunk_rows = norm_mode, 1e-6, act_mode, 0, 0
    a.norm1_w, a.norm2_w = mx.ops._p(t["norm1_w"]), mx.ops._p(t["norm2_w"])
    for k in ("shift1", "scale1", "gate1", "shift2", "scale2", "gate2"):
        setattr(a, k, mx.row_mod(t[k + "_t"], t[k + "_p"], n_prefix))
    a.gate_tanh = 1 if norm_mode == 0 else 0
    if packed:
        a.q_in = a.k_in = a.v_in = t["qkv"].data_ptr()
        a.qkv_stride, a.q_col0, a.k_col0, a.v_col0 = stride, 0, inner, 2 * inner
        a.v_out = t["v_out"].data_ptr()
    else:
        a.q_in, a.k_in, a.v_in = t["q_in"].data_ptr(), t["k_in"].data_ptr(), None
        a.qkv_stride, a.q_col0, a.k_col0, a.v_col0 = inner, 0, 0, 0
    a.norm_q, a.norm_k = t["norm_q"].data_ptr(), t["norm_k"].data_ptr()
    a.cos, a.sin, a.rot, a.rope_mode = t["cos"].data_ptr(), t["sin"].data_ptr(), rot, rope_mode
    a.q_out, a.k_out = t["q_out"].data_ptr(), t["k_out"].data_ptr()
    a.x, a.h1, a.h2 = t["x"].data_ptr(), t["h1"].data_ptr(), t["h2"].data_ptr()
    a.attn_o, a.act, a.mlp_o = t["attn_o"].data_ptr(), t["act"].data_ptr(), t["mlp_o"].data_ptr()
    a.act2 = t["act2"].data_ptr() if act_mode == 1 else None
    return n, t, a


def oracle_block(n, rows, dim, Hh, D, F, norm_mode, act_mode, rot, rope_mode, packed, n_prefix):
    """The same op sequence on the CPU oracle."""
    inner = Hh * D
    m = lambda k: orc.mod(n[k + "_t"], n[k + "_p"], n_prefix)
    tanh = 1 if norm_mode == 0 else 0
    x = n["x"].copy()
    out = {}
    if norm_mode == 0:
        out["h1"] = orc.layernorm_mod(x, 1e-6, m("scale1"), m("shift1"))
    else:
        out["h1"] = orc.rmsnorm_mod(x, 1e-6, n["norm1_w"], m("scale1"), m("shift1"))
    if packed:
        out["q_out"] = orc.head_norm_rope(n["qkv"], rows, 3 * inner, 0, Hh, D, n["norm_q"], 1e-6, n["cos"], n["sin"], rot, rope_mode)
        out["k_out"] = orc.head_norm_rope(n["qkv"], rows, 3 * inner, inner, Hh, D, n["norm_k"], 1e-6, n["cos"], n["sin"], rot, rope_mode)
        out["v_out"] = orc.head_norm_rope(n["qkv"], rows, 3 * inner, 2 * inner, Hh, D, None, 0.0, None, None, 0, 0)
    else:
        out["q_out"] = orc.head_norm_rope(n["q_in"], rows, inner, 0, Hh, D, n["norm_q"], 1e-6, n["cos"], n["sin"], rot, rope_mode)
        out["k_out"] = orc.head_norm_rope(n["k_in"], rows, inner, 0, Hh, D, n["norm_k"], 1e-6, n["cos"], n["sin"], rot, rope_mode)
    orc.gated_residual(x, n["attn_o"], m("gate1"), tanh)
    if norm_mode == 0:
        out["h2"] = orc.layernorm_mod(x, 1e-6, m("scale2"), m("shift2"))
    else:
        out["h2"] = orc.rmsnorm_mod(x, 1e-6, n["norm2_w"], m("scale2"), m("shift2"))
    out["act"] = orc.gelu_tanh_inplace(n["act"].copy()) if act_mode == 0 else orc.silu_mul(n["act2"], F)
    orc.gated_residual(x, n["mlp_o"], m("gate2"), tanh)
    out["x"] = x
    return out


BLOCKS = [
    # rows, dim, H, D, F, norm_mode, act_mode, rot, rope_mode, packed, n_prefix
    (272, 3072, 24, 128, 12288, 0, 0, 128, 1, False, 256),   # Qwen-Image-shaped (benchmark configs 1-4), image|text switch
    (200, 5120, 40, 128, 13824, 1, 1, 128, 2, True, 0),      # MiniMax-H3-shaped (config 5)
    (150, 5376, 56, 128, 14336, 1, 1, 96, 2, True, 0),       # the reference's true H3 widths
]


@pytest.mark.parametrize("cfg", BLOCKS)
@pytest.mark.parametrize("fused", [0, 1])
@pytest.mark.parametrize("chunk", [0, 64])
def test_dit_block_ops(mx, cfg, fused, chunk):
    rows = cfg[0]
    g = H.rng(rows + fused)
    n, t, a = make_block(mx, g, *cfg)
    a.fused, a.chunk_rows = fused, chunk
    ref = oracle_block(n, *cfg)
    mx.dit_block_ops(a)
    torch.cuda.synchronize()
    for k in ("h1", "q_out", "k_out", "h2", "act"):
        H.assert_bf16_close(H.bits(t[k]), ref[k], f"block {k} fused={fused}")
    if cfg[9]:
        assert np.array_equal(H.bits(t["v_out"]), ref["v_out"])
    H.assert_f32_close(t["x"].cpu().numpy(), ref["x"], "block x")


@pytest.mark.parametrize("cfg", BLOCKS[:2])
def test_host_pipeline_equals_device_chain(mx, cfg):
    rows = cfg[0]
    g1, g2 = H.rng(rows), H.rng(rows)
    nd, td, ad = make_block(mx, g1, *cfg)
    nh, th, ah = make_block(mx, g2, *cfg, host=True)
    mx.dit_block_ops(ad)
    pipe = mx.HostPipeline(48, cfg[1], cfg[4], cfg[2], cfg[3], cfg[7], with_v=cfg[9], act_mode=cfg[6])
    up, down = pipe.run(ah)
    pipe.close()
    torch.cuda.synchronize()
    assert up > 0 and down > 0
    for k in ("h1", "q_out", "k_out", "h2", "act"):
        assert np.array_equal(H.bits(td[k]), th[k].view(torch.uint16).numpy()), k
    assert np.array_equal(td["x"].cpu().numpy(), th["x"].numpy())


@pytest.mark.parametrize("cfg", BLOCKS[:2])
@pytest.mark.parametrize("fused", [0, 1])
def test_block_chain_captures_into_a_cuda_graph(mx, cfg, fused):
    """The launchers allocate nothing and never synchronise, so a block's op sequence (with its programmatic
    dependent launches and, in the quantiser, its memsets) can be captured once and replayed: the replay
    writes the same bits as the eager call."""
    rows = cfg[0]
    n1, t1, a1 = make_block(mx, H.rng(rows + 31), *cfg)
    n2, t2, a2 = make_block(mx, H.rng(rows + 31), *cfg)
    a1.fused = a2.fused = fused
    a1.chunk_rows = a2.chunk_rows = 0
    mx.dit_block_ops(a1)          # eager; also the warm-up that resolves per-device caches
    torch.cuda.synchronize()
    x0 = t2["x"].clone()
    act0 = t2["act"].clone() if cfg[6] == 0 else None
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        mx.dit_block_ops(a2)
        qm = mx.ops.quantize_blockscaled(mx.ops.Q_NVFP4, t2["h1"], cfg[1], rows, cfg[1])
    torch.cuda.synchronize()
    for _ in range(2):              # replay from the same inputs twice
        t2["x"].copy_(x0)
        if act0 is not None:
            t2["act"].copy_(act0)
        graph.replay()
        torch.cuda.synchronize()
        for k in ("h1", "q_out", "k_out", "h2", "act"):
            assert np.array_equal(H.bits(t1[k]), H.bits(t2[k])), k
        assert torch.equal(t1["x"], t2["x"])
        want = orc.quantize_blockscaled(2, H.bits(t2["h1"]))
        assert np.array_equal(qm.q.cpu().numpy(), want[0]) and np.array_equal(qm.sf.cpu().numpy(), want[1])
        assert float(qm.amax.item()) == want[2]
    assert mx.device_error() == 0


def test_bounded_wait_reports_and_context_survives(mx):
    """A wait that can never be satisfied (a barrier nothing completes) runs out of its budget, the
    kernel reports through the device error word and returns; the context keeps working."""
    from miroxen_b200 import _lib
    assert mx.device_error() == 0
    _lib.check(mx.lib().mxk_selftest_bounded_wait(None))
    torch.cuda.synchronize()
    assert mx.device_error(clear=True) == 1
    assert mx.device_error() == 0
    x = torch.ones(1024, device="cuda")
    y = torch.full((1024,), 2.0, device="cuda")
    mx.axpy_f32(x, y, 0.5, 1024)
    torch.cuda.synchronize()
    assert float(x.sum()) == 2048.0


def test_host_entry_points_report_a_timed_out_wait_as_a_status(mx):
    """The host-buffer entry points return results in host memory, so they read the device error word
    themselves: with the word set (here by the harmless bounded-wait self-test) both return
    MXK_ERR_CUDA instead of 0; after the word is cleared the same calls succeed."""
    from miroxen_b200 import _lib
    cfg = BLOCKS[0]
    _, _, a = make_block(mx, H.rng(11), *cfg, host=True)
    pipe = mx.HostPipeline(64, cfg[1], cfg[4], cfg[2], cfg[3], cfg[7], with_v=cfg[9], act_mode=cfg[6])
    try:
        assert mx.device_error() == 0
        _lib.check(mx.lib().mxk_selftest_bounded_wait(None))
        torch.cuda.synchronize()
        with pytest.raises(mx.MxkError, match="bounded wait ran out"):
            pipe.run(a)
        with pytest.raises(mx.MxkError, match="bounded wait ran out"):
            mx.dit_block_ops_host_static(a)
        assert mx.device_error(clear=True) == 1  # the entry points leave the word for the caller to clear
        up, down = pipe.run(a)
        assert up > 0 and down > 0
        mx.dit_block_ops_host_static(a)
    finally:
        pipe.close()
        mx.device_error(clear=True)


# ---- the library's builders against the reference's own statements -------------------------------
# tests/golden/ref_builders.npz holds what the reference's statements produced (generator:
# tests/golden/make_ref_builders_golden.py); full tables for small layouts, SHA-256 digests for
# benchmark-sized ones.

def _gold():
    import sys
    from pathlib import Path
    gdir = Path(__file__).resolve().parent / "golden"
    if str(gdir) not in sys.path:
        sys.path.insert(0, str(gdir))
    import ref_builder_cases as cases
    return np.load(gdir / "ref_builders.npz"), cases


def _digest(*arrays):
    import hashlib
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest(), np.uint8)


def test_library_qwen_rope_table_equals_the_reference_statements(mx):
    from miroxen_b200 import rope_tables
    gold, cases = _gold()
    for i, (T, Hh, W, conds) in enumerate(cases.QWEN_ROPE_FULL):
        cos, sin = rope_tables.qwen_rope_table(orc.qwen_segs(T, Hh, W, conds))
        assert np.array_equal(cos.cpu().numpy().view(np.uint32), gold[f"qwen_rope_full{i}_cos"].view(np.uint32)), i
        assert np.array_equal(sin.cpu().numpy().view(np.uint32), gold[f"qwen_rope_full{i}_sin"].view(np.uint32)), i
    for i, (T, Hh, W, conds) in enumerate(cases.QWEN_ROPE_DIGEST):
        cos, sin = rope_tables.qwen_rope_table(orc.qwen_segs(T, Hh, W, conds))
        assert cos.shape[0] == int(gold[f"qwen_rope_digest{i}_rows"][0])
        assert np.array_equal(_digest(cos.cpu().numpy(), sin.cpu().numpy()), gold[f"qwen_rope_digest{i}"]), i


def test_library_timestep_embedding_equals_the_reference_statements(mx):
    from miroxen_b200 import rope_tables
    gold, cases = _gold()
    for on_host in (True, False):
        got = np.stack([rope_tables.qwen_timestep_embedding(float(t), on_host=on_host).cpu().numpy() for t in cases.TIMESTEPS_FULL])
        assert np.array_equal(got.view(np.uint32), gold["timestep_full"].view(np.uint32)), on_host
    dev = [rope_tables.qwen_timestep_embedding(float(t)) for t in cases.timesteps_digest()]
    assert np.array_equal(_digest(*[d.cpu().numpy() for d in dev]), gold["timestep_digest"])


def test_library_h3_builders_equal_the_reference_statements(mx):
    from miroxen_b200 import rope_tables
    gold, cases = _gold()
    table, ts, small = cases.h3_basis_inputs()
    for tab, key in ((table, "h3_basis"), (small, "h3_basis_small")):
        out = rope_tables.h3_time_basis(H.to_dev(torch, ts), H.to_dev(torch, tab))
        assert np.array_equal(out.cpu().numpy().view(np.uint32), gold[key].view(np.uint32)), key
    invf = cases.h3_inv_freq()
    layouts = {"case0": (512, 21, 60, 104, 0, []), "case1": (37, 7, 30, 52, 25, ["first", "last"]), "case2": (5, 2, 4, 6, 3, ["last"])}
    for name, (T, F_lat, Hh, W, A, anchors) in layouts.items():
        cos, sin = rope_tables.h3_rope_table(T, F_lat, Hh, W, A, anchors, invf)
        assert np.array_equal(_digest(cos.cpu().numpy(), sin.cpu().numpy()), gold[f"h3_rope_{name}_digest"]), name
