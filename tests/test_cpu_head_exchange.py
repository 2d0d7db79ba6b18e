"""Index maps of the head exchange (miroxen_b200.head_exchange.ExchangePlan) without a GPU: every
rank projects its own rows for all heads, each head group goes to the rank that attends over it
and the attention output comes back, for 1, 2, 4 and 8 ranks; the 2-rank case also runs as two gloo
processes that really exchange the tiles (the reference's split: src/models/minimax_h3/dit_sp.cpp:200-207,
heads [0, H/2) on card 0, rows [0, S/2) on card 0)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("S,H,D", [(53, 40, 16), (8, 8, 8), (33272, 56, 2)])
def test_scatter_then_gather_restores_every_ranks_rows(world, S, H, D):
    from miroxen_b200.head_exchange import ExchangePlan
    from miroxen_b200.sharding import covers
    plan = ExchangePlan(S, H, D, world)
    assert covers([plan.rows(r) for r in range(world)], S)
    assert sorted(h for r in range(world) for h in plan.head_range(r)) == list(range(H))
    g = np.random.default_rng(S + world)
    full = g.integers(0, 60000, (S, H, D)).astype(np.uint16)
    bufs = [np.zeros((S, plan.heads_per_group, D), np.uint16) for _ in range(world)]
    for r in range(world):
        sh = plan.rows(r)
        plan.scatter_numpy(r, full[sh.row0:sh.row0 + sh.rows], bufs)
    hg = plan.heads_per_group
    for r in range(world):   # what the attention of rank r sees: all rows, its own heads
        assert np.array_equal(bufs[r], full[:, r * hg:(r + 1) * hg, :])
    for r in range(world):   # and back: all heads of the rank's own rows
        sh = plan.rows(r)
        assert np.array_equal(plan.gather_numpy(r, bufs), full[sh.row0:sh.row0 + sh.rows])


def test_dst_element_agrees_with_the_layout():
    from miroxen_b200.head_exchange import ExchangePlan
    plan = ExchangePlan(101, 24, 8, 4)
    g = np.random.default_rng(3)
    for _ in range(200):
        r = int(g.integers(0, 4))
        sh = plan.rows(r)
        s, h, d = int(g.integers(0, sh.rows)), int(g.integers(0, 24)), int(g.integers(0, 8))
        dst, flat = plan.dst_element(r, s, h, d)
        assert dst == h // 6
        assert flat == ((sh.row0 + s) * 6 + h % 6) * 8 + d


def test_send_bytes_and_bad_worlds():
    from miroxen_b200.head_exchange import ExchangePlan
    plan = ExchangePlan(33272, 40, 128, 8)
    assert plan.send_bytes(0) == 3 * 4159 * 40 * 128 * 2 * 7 // 8
    assert ExchangePlan(10, 8, 4, 1).send_bytes(0) == 0
    with pytest.raises(ValueError):
        ExchangePlan(10, 24, 128, 5)


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from miroxen_b200.head_exchange import ExchangePlan
    S, H, D = 37, 8, 4
    plan = ExchangePlan(S, H, D, world)
    full = np.random.default_rng(11).integers(0, 1000, (S, H, D)).astype(np.int32)  # rows a rank does not own are never read
    sh, hg = plan.rows(rank), plan.heads_per_group
    mine = full[sh.row0:sh.row0 + sh.rows]
    # the tile for rank g is [rows(rank), H/G, D]; send it, receive everybody's tile of my head group
    tiles = [torch.from_numpy(np.ascontiguousarray(mine[:, g * hg:(g + 1) * hg, :])) for g in range(world)]
    got = [torch.empty((plan.rows(r).rows, hg, D), dtype=torch.int32) for r in range(world)]
    reqs = []
    for r in range(world):
        if r == rank:
            got[r].copy_(tiles[r])
        else:
            reqs.append(dist.isend(tiles[r], r))
            reqs.append(dist.irecv(got[r], r))
    for q in reqs:
        q.wait()
    buf = np.zeros((S, hg, D), np.int32)
    for r in range(world):
        rs = plan.rows(r)
        buf[rs.row0:rs.row0 + rs.rows] = got[r].numpy()
    ok = np.array_equal(buf, full[:, rank * hg:(rank + 1) * hg, :])
    # the way back: every rank publishes its head-sharded buffer, each gathers its own rows
    everyone = [None] * world
    dist.all_gather_object(everyone, buf)
    back = plan.gather_numpy(rank, everyone)
    ok = ok and np.array_equal(back, mine)
    np.save(Path(out_dir) / f"ok{rank}.npy", np.array([ok]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_head_exchange(tmp_path):
    import torch.multiprocessing as mp
    port = 31500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert all(bool(np.load(tmp_path / f"ok{r}.npy")[0]) for r in range(2))
