"""Token-row sharding of the fused layer ops across the GPUs of one box.

Every op on the path is row-independent, so each rank owns a contiguous range of token rows - the
same `[r0, r0 + n)` split the reference's 2-GPU sequence-parallel path uses
(src/models/minimax_h3/dit_sp.cpp:206-207) - and no collective runs in the timed loop.  Set-up
only replicates the modulation vectors and norm weights (one broadcast) and hands each rank its
slice of the cos/sin table.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Sequence


@dataclass(frozen=True)
class RowShard:
    rank: int
    world: int
    row0: int  # first global row of this rank
    rows: int  # rows owned

    def shift_prefix(self, prefix_len: int) -> int:
        """prefix_len as seen by a launch that starts at this shard's first row; the kernels compare
        `row < prefix_len`, so the value may be negative or exceed `rows`
        (src/kernels/ops.cu:183-184 does the same for its row slabs)."""
        return prefix_len - self.row0


def shard_rows(rows: int, world: int, rank: int) -> RowShard:
    """Balanced contiguous split: the first `rows % world` ranks own one row more."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(max(rows, 0), world)
    n = base + (1 if rank < extra else 0)
    r0 = rank * base + min(rank, extra)
    return RowShard(rank, world, r0, n)


def shard_frames(frames: int, rows_per_frame: int, tail_rows: int, world: int, rank: int) -> RowShard:
    """Video layout [frames x rows_per_frame | tail_rows]: whole frames per rank (earlier ranks take the
    extra frames), the tail rows (text) go to the last rank."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(frames, world)
    f = base + (1 if rank < extra else 0)
    f0 = rank * base + min(rank, extra)
    rows = f * rows_per_frame + (tail_rows if rank == world - 1 else 0)
    return RowShard(rank, world, f0 * rows_per_frame, rows)


def covers(shards: Iterable[RowShard], rows: int) -> bool:
    """True when the shards tile [0, rows) exactly, in rank order."""
    at = 0
    for s in sorted(shards, key=lambda s: s.rank):
        if s.row0 != at or s.rows < 0:
            return False
        at += s.rows
    return at == rows


def broadcast_modulation(tensors: Sequence, src: int = 0, group=None) -> None:
    """Replicates the (tiny) modulation vectors / norm weights from `src` to every rank, in place.
    One coalesced set-up step; nothing on the timed path communicates."""
    import torch.distributed as dist
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    for t in tensors:
        if t is not None:
            dist.broadcast(t, src=src, group=group)
