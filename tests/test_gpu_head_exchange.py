"""Head exchange kernels (mxk_qkv_norm_rope_scatter, mxk_gather_head_groups).

On one GPU the G destination buffers are all local: the launches are exactly the ones G ranks make
(rank r: its rows, dst_row0 = its first row), so the index arithmetic is covered in full, and the
result must equal the single-launch [S, H, D] layout of mxk_qkv_norm_rope head group by head group,
bit for bit.  With two or more GPUs the same check runs as one process per GPU over peer buffers
(CUDA IPC mappings, stores and loads over NVLink), NCCL only for the barrier."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

import helpers as H

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def mx():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import miroxen_b200 as m
    m.lib()
    yield m
    torch.cuda.synchronize()
    assert m.device_error() == 0


def make_inputs(S, Hh, D, rot, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    inner = Hh * D
    qkv = torch.randn((S, 3 * inner), generator=g, device="cuda").to(torch.bfloat16)
    nq = 1 + 0.05 * torch.randn(D, generator=g, device="cuda")
    nk = 1 + 0.05 * torch.randn(D, generator=g, device="cuda")
    ang = torch.rand((S, rot // 2), generator=g, device="cuda") * 6.2 - 3.1
    return qkv, nq, nk, torch.cos(ang).contiguous(), torch.sin(ang).contiguous()


def specs_for(mx, qkv, nq, nk, inner, rot, mode, row0=0, rows=None):
    v = qkv if rows is None else qkv[row0:row0 + rows]
    return [mx.HeadSpec(v, 3 * inner, 0, nq, None, rot, mode), mx.HeadSpec(v, 3 * inner, inner, nk, None, rot, mode),
            mx.HeadSpec(v, 3 * inner, 2 * inner, None, None, 0, 0)]


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("S,Hh,D,rot,mode", [(333, 40, 128, 128, 2), (130, 24, 128, 128, 1), (77, 56, 128, 96, 2), (50, 8, 64, 32, 1)])
def test_scatter_equals_the_dense_layout_group_by_group(mx, world, S, Hh, D, rot, mode):
    import ctypes as C
    from miroxen_b200 import _lib
    from miroxen_b200.head_exchange import ExchangePlan
    from miroxen_b200.ops import HeadTensor, _p
    plan = ExchangePlan(S, Hh, D, world)
    hg, inner = plan.heads_per_group, Hh * D
    qkv, nq, nk, cos, sin = make_inputs(S, Hh, D, rot, seed=S + world)
    # the dense single-launch result
    dense = [torch.empty((S, Hh, D), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    sp = specs_for(mx, qkv, nq, nk, inner, rot, mode)
    for t, o in zip(sp, dense):
        t.out = o
    # the scatter runs on the register head kernel: the dense result of the same kernel family is its bit-exact
    # counterpart (the bulk-copy pipeline, the default for the dense call, rounds a few elements the other way)
    mx.set_tuning("rope_path", 2)
    mx.qkv_norm_rope(sp, S, Hh, D, 1e-6, cos, sin)
    mx.set_tuning("rope_path", 0)
    piped = [torch.empty((S, Hh, D), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    for t, o in zip(sp, piped):
        t.out = o
    mx.qkv_norm_rope(sp, S, Hh, D, 1e-6, cos, sin)
    torch.cuda.synchronize()
    for o, p_ in zip(dense, piped):
        H.assert_bf16_close(H.bits(o), H.bits(p_), "register vs pipeline head kernel")
    # G "ranks", every destination on this GPU
    bufs = [[H.Guarded(torch, (S, hg, D), torch.bfloat16) for _ in range(world)] for _ in range(3)]
    for r in range(world):
        sh = plan.rows(r)
        if sh.rows == 0:
            continue
        spr = specs_for(mx, qkv, nq, nk, inner, rot, mode, sh.row0, sh.rows)
        arr = (HeadTensor * 3)(*[HeadTensor(_p(t.in_), t.in_stride, t.col0, _p(t.norm_w), None, t.rot, t.mode) for t in spr])
        outs = (C.c_void_p * (3 * world))(*[bufs[i][g].t.data_ptr() for i in range(3) for g in range(world)])
        _lib.check(mx.lib().mxk_qkv_norm_rope_scatter(arr, 3, sh.rows, Hh, D, 1e-6, _p(cos[sh.row0:]), _p(sin[sh.row0:]), world, outs,
                                                      sh.row0, None))
    torch.cuda.synchronize()
    for i in range(3):
        for g in range(world):
            bufs[i][g].check(f"tensor {i} group {g}")
            assert torch.equal(bufs[i][g].t, dense[i][:, g * hg:(g + 1) * hg, :]), (i, g)
    # the way back, for every rank
    for r in range(world):
        sh = plan.rows(r)
        if sh.rows == 0:
            continue
        out = H.Guarded(torch, (sh.rows, inner), torch.bfloat16)
        srcs = (C.c_void_p * world)(*[bufs[0][g].t.data_ptr() for g in range(world)])
        _lib.check(mx.lib().mxk_gather_head_groups(srcs, world, sh.row0, sh.rows, hg, D, out.t.data_ptr(), None))
        torch.cuda.synchronize()
        out.check("gather")
        assert torch.equal(out.t.view(sh.rows, Hh, D), dense[0][sh.row0:sh.row0 + sh.rows])


def test_scatter_argument_checks(mx):
    import ctypes as C
    from miroxen_b200.ops import HeadTensor
    arr = (HeadTensor * 1)(HeadTensor(256, 128, 0, None, None, 0, 0))
    outs = (C.c_void_p * 3)(256, 256, 256)
    L = mx.lib()
    assert L.mxk_qkv_norm_rope_scatter(arr, 1, 4, 8, 16, 1e-6, None, None, 3, outs, 0, None) == -1  # 3 does not divide 8
    assert L.mxk_qkv_norm_rope_scatter(arr, 1, 4, 8, 16, 1e-6, None, None, 9, outs, 0, None) == -1
    outs2 = (C.c_void_p * 2)(256, 8)
    assert L.mxk_qkv_norm_rope_scatter(arr, 1, 4, 8, 128, 1e-6, None, None, 2, outs2, 0, None) == -1  # unaligned destination
    assert L.mxk_qkv_norm_rope_scatter(arr, 1, 0, 8, 128, 1e-6, None, None, 2, outs2, 0, None) == 0   # no rows: no-op
    assert L.mxk_gather_head_groups(outs2, 2, 0, 4, 4, 128, 256, None) == -1
    assert L.mxk_gather_head_groups(outs, 3, 0, 0, 4, 128, 256, None) == 0


def _rank_main(rank, world, port, out_dir):
    """One process per GPU: scatter this rank's rows into everybody's buffers, barrier, compare this rank's
    buffers (all rows, own heads) with the dense single-GPU result computed locally, gather back."""
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import miroxen_b200 as mx
    from miroxen_b200.head_exchange import ExchangePlan, HeadExchange
    S, Hh, D, rot, mode = 2051, 40, 128, 128, 2
    inner = Hh * D
    plan = ExchangePlan(S, Hh, D, world)
    qkv, nq, nk, cos, sin = make_inputs(S, Hh, D, rot, seed=99)  # same seed everywhere: every rank can check everything
    dense = [torch.empty((S, Hh, D), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    sp = specs_for(mx, qkv, nq, nk, inner, rot, mode)
    for t, o in zip(sp, dense):
        t.out = o
    mx.set_tuning("rope_path", 2)  # the kernel family the scatter uses: bit-exact counterpart
    mx.qkv_norm_rope(sp, S, Hh, D, 1e-6, cos, sin)
    mx.set_tuning("rope_path", 0)
    ex = HeadExchange(plan, rank)
    ok = True
    try:
        sh, hg = plan.rows(rank), plan.heads_per_group
        for rep in range(2):
            spr = specs_for(mx, qkv, nq, nk, inner, rot, mode, sh.row0, sh.rows)
            ex.scatter_qkv(spr, sh.rows, 1e-6, cos[sh.row0:], sin[sh.row0:])
            ex.barrier()
            for b in range(3):
                ok = ok and bool(torch.equal(ex.local_tensor(b), dense[b][:, rank * hg:(rank + 1) * hg, :]))
            # stand-in for the attention output: buffer 3 := this rank's q heads; gather all heads of my rows back
            ex.local_tensor(3).copy_(ex.local_tensor(0))
            ex.barrier()
            out = torch.empty((sh.rows, inner), dtype=torch.bfloat16, device="cuda")
            ex.gather_heads(out)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(out.view(sh.rows, Hh, D), dense[0][sh.row0:sh.row0 + sh.rows]))
            ex.barrier()
        ok = ok and mx.device_error() == 0
    finally:
        ex.barrier()
        ex.close()
    np.save(Path(out_dir) / f"ok{rank}.npy", np.array([ok]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_exchange_over_peer_buffers(mx, world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    port = 32500 + os.getpid() % 2000 + world
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all(bool(np.load(tmp_path / f"ok{r}.npy")[0]) for r in range(world))
