"""Host-side sharding logic, including a world_size-2 gloo run in which each rank processes its
own row range (with the CPU oracle standing in for the kernels) and the pieces tile the
single-process result bit for bit."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_shard_rows_tiles_the_range():
    from miroxen_b200.sharding import covers, shard_rows
    for rows in (0, 1, 7, 8704, 16896, 33272):
        for world in (1, 2, 4, 8):
            shards = [shard_rows(rows, world, r) for r in range(world)]
            assert covers(shards, rows)
            assert max(s.rows for s in shards) - min(s.rows for s in shards) <= 1
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def test_shard_frames_matches_the_video_split():
    from miroxen_b200.sharding import covers, shard_frames
    # 21 frames of 30 x 52 rows + 512 text rows over 8 GPUs: 3,3,3,3,3,2,2,2 frames, text on the last rank
    shards = [shard_frames(21, 1560, 512, 8, r) for r in range(8)]
    assert [s.rows // 1560 for s in shards] == [3, 3, 3, 3, 3, 2, 2, 2]
    assert shards[-1].rows == 2 * 1560 + 512
    assert covers(shards, 21 * 1560 + 512)
    assert covers([shard_frames(21, 1560, 512, 1, 0)], 33272)


def test_shift_prefix():
    from miroxen_b200.sharding import shard_rows
    s = shard_rows(100, 4, 2)
    assert s.row0 == 50 and s.shift_prefix(60) == 10 and s.shift_prefix(10) == -40


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from miroxen_b200.sharding import broadcast_modulation, shard_rows
    from oracle import binding as orc
    rows, dim, plen = 53, 256, 20
    g = np.random.default_rng(0)  # the activations are "already resident": same seed on every rank
    x = g.standard_normal((rows, dim), dtype=np.float32)
    # modulation vectors exist on rank 0 only and are broadcast once
    sc_t = torch.from_numpy(g.standard_normal(dim, dtype=np.float32)) if rank == 0 else torch.zeros(dim)
    sc_p = torch.from_numpy(g.standard_normal(dim, dtype=np.float32)) if rank == 0 else torch.zeros(dim)
    broadcast_modulation([sc_t, sc_p, None], src=0)
    sh = shard_rows(rows, world, rank)
    mine = orc.layernorm_mod(np.ascontiguousarray(x[sh.row0:sh.row0 + sh.rows]), 1e-6,
                             orc.mod(sc_t.numpy(), sc_p.numpy(), sh.shift_prefix(plen)), orc.NONE)
    np.save(Path(out_dir) / f"part{rank}.npy", mine)
    if rank == 0:
        whole = orc.layernorm_mod(x, 1e-6, orc.mod(sc_t.numpy(), sc_p.numpy(), plen), orc.NONE)
        np.save(Path(out_dir) / "whole.npy", whole)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_shards_tile_the_result(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    whole = np.load(tmp_path / "whole.npy")
    parts = np.concatenate([np.load(tmp_path / f"part{r}.npy") for r in range(2)])
    assert np.array_equal(whole, parts)
