"""Head exchange of the sequence-parallel attention path for G = 1 ... 8 GPUs of one box.

The reference shards token rows for the linear layers and attention heads for attention, on two
cards (src/models/minimax_h3/dit_sp.cpp:1-4, 200-207): after the QKV projection every card needs
all rows of its own heads (`sp_qkv`, :83-112: norm + rope into a send buffer, then a peer copy);
after attention every card needs all heads of its own rows (`sp_mlp`, :137-149: a peer copy back,
then two strided copies).  Here rank r owns rows `shard_rows(S, G, r)` and heads
`[r * H/G, (r + 1) * H/G)`; the norm + rope kernel stores head group g straight into rank g's
`[S, H/G, D]` buffer over NVLink (`mxk_qkv_norm_rope_scatter`), and the way back is one gather
kernel reading the peers' buffers (`mxk_gather_head_groups`).  The only collective is the barrier
that orders the attention after everybody's stores; no send buffers, no copies.

`ExchangePlan` is pure index arithmetic (testable on the CPU); `HeadExchange` owns the peer buffers.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Sequence

from .sharding import RowShard, shard_rows


@dataclass(frozen=True)
class ExchangePlan:
    S: int          # rows of the whole sequence
    H: int          # attention heads
    D: int          # channels per head
    world: int

    def __post_init__(self):
        if self.world < 1 or self.H % self.world != 0:
            raise ValueError(f"{self.world} ranks must divide {self.H} heads")

    @property
    def heads_per_group(self) -> int:
        return self.H // self.world

    def rows(self, rank: int) -> RowShard:
        """Rows rank `rank` projects (and later needs every head of)."""
        return shard_rows(self.S, self.world, rank)

    def head_range(self, rank: int) -> range:
        """Heads rank `rank` attends over (for every row)."""
        return range(rank * self.heads_per_group, (rank + 1) * self.heads_per_group)

    def owner_of_head(self, h: int) -> int:
        return h // self.heads_per_group

    def dst_element(self, src_rank: int, s_local: int, h: int, d: int):
        """Where element (local row s_local, head h, channel d) of src_rank's projection lands:
        (destination rank, flat element index inside that rank's [S, H/G, D] buffer)."""
        g = self.owner_of_head(h)
        row = self.rows(src_rank).row0 + s_local
        return g, (row * self.heads_per_group + (h - g * self.heads_per_group)) * self.D + d

    def send_bytes(self, rank: int, tensors: int = 3) -> int:
        """bf16 bytes rank `rank` stores into OTHER ranks' buffers per exchange of `tensors` tensors:
        rows * H * D * 2 * (G - 1) / G each."""
        return tensors * self.rows(rank).rows * self.H * self.D * 2 * (self.world - 1) // self.world

    # numpy emulation of the two kernels, for tests of the index maps
    def scatter_numpy(self, src_rank: int, x, bufs: Sequence) -> None:
        """x: [rows(src_rank), H, D] -> writes bufs[g][row0 + s, :, :] for every group g."""
        sh, hg = self.rows(src_rank), self.heads_per_group
        for g in range(self.world):
            bufs[g][sh.row0:sh.row0 + sh.rows] = x[:, g * hg:(g + 1) * hg, :]

    def gather_numpy(self, rank: int, bufs: Sequence):
        """bufs[g]: [S, H/G, D] -> [rows(rank), H, D] (all heads of this rank's rows)."""
        import numpy as np
        sh = self.rows(rank)
        return np.concatenate([bufs[g][sh.row0:sh.row0 + sh.rows] for g in range(self.world)], axis=1)


class HeadExchange:
    """Peer buffers and launches of one rank.  `n_buffers` arrays of bf16 [S, H/G, D] are allocated on this
    GPU (q, k, v and the attention output by default) and every other rank's arrays are mapped here."""

    def __init__(self, plan: ExchangePlan, rank: int, n_buffers: int = 4, group=None):
        import torch
        import torch.distributed as dist
        from ._lib import check, lib
        self.plan, self.rank, self.group, self.n = plan, rank, group, n_buffers
        self._lib, self._check = lib(), check
        self.nbytes = plan.S * plan.heads_per_group * plan.D * 2
        self.local: List[int] = []
        handles = []
        for _ in range(n_buffers):
            ptr, h = C.c_void_p(), (C.c_ubyte * 64)()
            check(self._lib.mxk_peer_buffer_alloc(self.nbytes, C.byref(ptr), h))
            self.local.append(ptr.value)
            handles.append(bytes(h))
        self.ptrs = [[0] * plan.world for _ in range(n_buffers)]   # ptrs[buffer][rank]
        self._opened = []
        if plan.world == 1:
            for b in range(n_buffers):
                self.ptrs[b][0] = self.local[b]
        else:
            everyone = [None] * plan.world
            dist.all_gather_object(everyone, handles, group=group)
            for r in range(plan.world):
                for b in range(n_buffers):
                    if r == rank:
                        self.ptrs[b][r] = self.local[b]
                    else:
                        p = C.c_void_p()
                        raw = (C.c_ubyte * 64).from_buffer_copy(everyone[r][b])
                        check(self._lib.mxk_peer_buffer_open(raw, C.byref(p)))
                        self.ptrs[b][r] = p.value
                        self._opened.append(p.value)
            dist.barrier(group=group)
        self._torch = torch

    def local_tensor(self, b: int):
        """This rank's buffer b as a torch tensor [S, H/G, D] (a view of the allocation, not a copy)."""
        torch = self._torch
        p = self.plan

        class _Raw:
            pass
        holder = _Raw()
        holder.__cuda_array_interface__ = {"shape": (p.S, p.heads_per_group, p.D), "typestr": "<i2", "data": (self.local[b], False),
                                           "version": 2}
        self._keep = getattr(self, "_keep", []) + [holder]
        return torch.as_tensor(holder, device="cuda").view(torch.bfloat16)

    def scatter_qkv(self, specs, S_local, eps, cos, sin, buffers=(0, 1, 2), stream=None):
        """mxk_qkv_norm_rope_scatter on this rank's rows: specs as for ops.qkv_norm_rope (their `out` is unused);
        tensor i goes to buffer buffers[i] of every rank."""
        from .ops import HeadTensor, _p, _stream
        p = self.plan
        arr = (HeadTensor * len(specs))(*[HeadTensor(_p(t.in_), t.in_stride, t.col0, _p(t.norm_w), None, t.rot, t.mode) for t in specs])
        outs = (C.c_void_p * (len(specs) * p.world))(*[self.ptrs[buffers[i]][g] for i in range(len(specs)) for g in range(p.world)])
        self._check(self._lib.mxk_qkv_norm_rope_scatter(arr, len(specs), S_local, p.H, p.D, eps, _p(cos), _p(sin), p.world, outs,
                                                        p.rows(self.rank).row0, _stream(stream)))

    def gather_heads(self, out, buffer=3, stream=None):
        """mxk_gather_head_groups: all heads of this rank's rows from every rank's buffer -> out [rows, H * D]."""
        from .ops import _p, _stream
        p, sh = self.plan, self.plan.rows(self.rank)
        srcs = (C.c_void_p * p.world)(*self.ptrs[buffer])
        self._check(self._lib.mxk_gather_head_groups(srcs, p.world, sh.row0, sh.rows, p.heads_per_group, p.D, _p(out), _stream(stream)))

    def barrier(self):
        """Orders what follows on every rank after what every rank has queued so far (the stores of a
        scatter must have landed before the attention reads them)."""
        import torch.distributed as dist
        self._torch.cuda.current_stream().synchronize()
        if self.plan.world > 1:
            dist.barrier(group=self.group)

    def close(self):
        for p in self._opened:
            self._lib.mxk_peer_buffer_close(p)
        self._opened = []
        for p in self.local:
            self._lib.mxk_peer_buffer_free(p)
        self.local = []
