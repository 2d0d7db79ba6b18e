"""Synthetic DiT-block workloads for the benchmark and the smoke check: shapes, seeded inputs,
algorithmic byte counts.

GEMM and attention outputs are stand-ins: seeded N(0,1) bf16 tensors of the right shapes, as the
benchmark definition prescribes; modulation vectors are N(0, 0.3) stand-ins for the output of the
timestep MLP (a GEMM, outside this path), QK-norm weights are 1 + N(0, 0.05).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import torch

from .ops import BlockArgs, ROPE_HALF, ROPE_INTERLEAVED, row_mod, _p


@dataclass(frozen=True)
class Workload:
    name: str
    desc: str
    rows: int         # token rows of the whole job (all batch elements)
    dim: int          # residual width
    H: int
    D: int
    F: int
    norm_mode: int    # 0 LayerNorm, 1 RMSNorm
    act_mode: int     # 0 GELU-tanh in place, 1 SiLU-gated [rows, 2F] -> [rows, F]
    rot: int
    rope_mode: int
    packed_qkv: bool  # q/k/v read from one [rows, 3*H*D] buffer (and v copied out)
    eps: float
    gate_tanh: int
    prefix_rows: int  # rows [0, prefix_rows) use the "prefix" modulation set
    chunk_rows: int   # > 0: the sequence is issued per chunk of this many rows
    frames: int = 0   # video layouts: frames x rows_per_frame, then text rows
    rows_per_frame: int = 0

    @property
    def inner(self) -> int:
        return self.H * self.D

    def bytes_per_row(self) -> int:
        """Compulsory HBM bytes per token row of the unfused op list: two norms (4d in + 2d out),
        q and k rope (2 x 4*inner) plus the token's cos/sin row once, the v copy when packed, two
        gated residuals (4d + 2d in, 4d out) and the activation."""
        d, i = self.dim, self.inner
        b = 2 * 6 * d + 2 * 10 * d + 2 * 4 * i + 2 * (self.rot // 2) * 4
        if self.packed_qkv:
            b += 4 * i
        b += 4 * self.F if self.act_mode == 0 else 6 * self.F
        return b

    def op_bytes(self, rows: int) -> dict:
        d, i, F = self.dim, self.inner, self.F
        t = 2 * (self.rot // 2) * 4
        ops = {"norm_mod": 6 * d * rows, "head_norm_rope": 4 * i * rows, "gated_residual": 10 * d * rows,
               "gated_residual_norm": 12 * d * rows, "qkv_norm_rope": ((3 if self.packed_qkv else 2) * 4 * i + t) * rows,
               "gelu_tanh_inplace": 4 * F * rows, "silu_mul": 6 * F * rows}
        return ops


QWEN = dict(dim=3072, H=24, D=128, F=12288, norm_mode=0, act_mode=0, rot=128, rope_mode=ROPE_INTERLEAVED,
            packed_qkv=False, eps=1e-6, gate_tanh=1, chunk_rows=0)

WORKLOADS = {
    # BASELINE.json configs[1]: 1024^2 image (64 x 64 tokens) + 256 text tokens, CFG pair
    "qwen1024": Workload("qwen1024", "Qwen-Image-shaped block, 1024^2, batch 2: 2 x (4096 image + 256 text) rows",
                         rows=2 * (4096 + 256), prefix_rows=2 * 4096, **QWEN),
    # configs[0]: the CPU-sized case
    "qwen512": Workload("qwen512", "Qwen-Image-shaped block, 512^2, batch 1: 1024 image + 128 text rows",
                        rows=1024 + 128, prefix_rows=1024, **QWEN),
    # configs[3]
    "qwen2048": Workload("qwen2048", "Qwen-Image-shaped block, 2048^2, batch 1: 16384 image + 512 text rows",
                         rows=16384 + 512, prefix_rows=16384, **QWEN),
    # configs[4]
    "h3video": Workload("h3video", "MiniMax-H3-shaped video block: 21 x 30 x 52 video + 512 text rows",
                        rows=21 * 30 * 52 + 512, dim=5120, H=40, D=128, F=13824, norm_mode=1, act_mode=1, rot=128,
                        rope_mode=ROPE_HALF, packed_qkv=True, eps=1e-6, gate_tanh=0, prefix_rows=21 * 30 * 52,
                        chunk_rows=8192, frames=21, rows_per_frame=30 * 52),
    # the reference's true model widths (extra rows of the measurement matrix)
    "qwen21_true": Workload("qwen21_true", "Qwen-Image-2.1 widths: d 4096, 32 x 128 heads, SwiGLU 12288, 4096 + 256 rows",
                            rows=4096 + 256, dim=4096, H=32, D=128, F=12288, norm_mode=0, act_mode=1, rot=128,
                            rope_mode=ROPE_INTERLEAVED, packed_qkv=False, eps=1e-6, gate_tanh=1, prefix_rows=256,
                            chunk_rows=0),
    "h3_true": Workload("h3_true", "MiniMax-H3 widths: d 5376, 56 x 128 heads (rot 96), SwiGLU 14336, 33272 rows",
                        rows=21 * 30 * 52 + 512, dim=5376, H=56, D=128, F=14336, norm_mode=1, act_mode=1, rot=96,
                        rope_mode=ROPE_HALF, packed_qkv=True, eps=1e-5, gate_tanh=0, prefix_rows=0, chunk_rows=8192,
                        frames=21, rows_per_frame=30 * 52),
}


# image grid (tokens), text tokens and batch of the Qwen-Image-shaped workloads; rows are ordered
# [img0 | img1 | ... | txt0 | txt1 | ...] so that one prefix boundary separates image and text modulation
QWEN_GRIDS = {"qwen1024": (64, 64, 256, 2), "qwen512": (32, 32, 128, 1), "qwen2048": (128, 128, 512, 1)}


def rope_tables_for(w: "Workload", device="cuda"):
    """(cos, sin) fp32 [w.rows, rot/2] for the workload's row order, or (None, None) when the workload has no
    closed-form layout here (BlockBuffers then draws random angles).  Qwen-shaped workloads get the MSRoPE table
    of src/models/qwen_image/dit.cpp:151-185 for [image | text], repeated per batch element."""
    grid = QWEN_GRIDS.get(w.name)
    if not grid:
        return None, None
    from . import rope_tables
    ih, iw, nt, batch = grid
    c1, s1 = rope_tables.qwen_rope_table([("image", ih, iw), ("text", nt)], device=device)
    n_img = ih * iw
    cos = torch.cat([c1[:n_img]] * batch + [c1[n_img:]] * batch).contiguous()
    sin = torch.cat([s1[:n_img]] * batch + [s1[n_img:]] * batch).contiguous()
    return cos, sin


def with_rows(w: Workload, rows: int, prefix_rows: int) -> Workload:
    return replace(w, rows=rows, prefix_rows=prefix_rows)


class BlockBuffers:
    """Device (or pinned host) tensors of one block plus the BlockArgs that point at them."""

    def __init__(self, w: Workload, rows: int, prefix_rows: int, seed: int = 0, device="cuda", host: bool = False,
                 cos=None, sin=None, mods=None):
        self.w, self.rows = w, rows
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        dev = torch.device(device)

        def data(shape, dtype):
            t = torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(dtype)
            if host:
                p = torch.empty(shape, dtype=dtype, pin_memory=True)
                p.copy_(t)
                return p
            return t

        def out(shape):
            return torch.empty(shape, dtype=torch.bfloat16, pin_memory=True) if host else \
                torch.empty(shape, dtype=torch.bfloat16, device=dev)

        inner, d, F = w.inner, w.dim, w.F
        self.x = data((rows, d), torch.float32)
        if w.packed_qkv:
            self.qkv = data((rows, 3 * inner), torch.bfloat16)
            self.v_out = out((rows, w.H, w.D))
        else:
            self.q_in, self.k_in = data((rows, inner), torch.bfloat16), data((rows, inner), torch.bfloat16)
        self.attn_o, self.mlp_o = data((rows, d), torch.bfloat16), data((rows, d), torch.bfloat16)
        if w.act_mode == 0:
            self.act = data((rows, F), torch.bfloat16)
            self.act2 = None
        else:
            self.act2 = data((rows, 2 * F), torch.bfloat16)
            self.act = out((rows, F))
        self.h1, self.h2 = out((rows, d)), out((rows, d))
        self.q_out, self.k_out = out((rows, w.H, w.D)), out((rows, w.H, w.D))
        half = max(w.rot // 2, 1)
        if cos is None:
            ang = (torch.rand((rows, half), generator=g, device=dev) * 6.2 - 3.1)
            cos, sin = torch.cos(ang), torch.sin(ang)
        if host:
            hc, hs = torch.empty(cos.shape, pin_memory=True), torch.empty(sin.shape, pin_memory=True)
            hc.copy_(cos), hs.copy_(sin)
            cos, sin = hc, hs
        self.cos, self.sin = cos.contiguous(), sin.contiguous()
        # modulation / weights: always on the device, shared across buffer sets when given
        self.mods = mods if mods is not None else make_mods(w, seed=1000 + seed, device=device)
        a = BlockArgs()
        a.rows, a.dim, a.F, a.H, a.D = rows, d, F, w.H, w.D
        a.norm_mode, a.eps, a.act_mode, a.fused, a.chunk_rows = w.norm_mode, w.eps, w.act_mode, 0, w.chunk_rows
        m = self.mods
        a.norm1_w, a.norm2_w = _p(m.get("norm1_w")), _p(m.get("norm2_w"))
        for k in ("shift1", "scale1", "gate1", "shift2", "scale2", "gate2"):
            setattr(a, k, row_mod(m[k + "_t"], m[k + "_p"], prefix_rows))
        a.gate_tanh = w.gate_tanh
        if w.packed_qkv:
            a.q_in = a.k_in = a.v_in = self.qkv.data_ptr()
            a.qkv_stride, a.q_col0, a.k_col0, a.v_col0 = 3 * inner, 0, inner, 2 * inner
            a.v_out = self.v_out.data_ptr()
        else:
            a.q_in, a.k_in, a.v_in = self.q_in.data_ptr(), self.k_in.data_ptr(), None
            a.qkv_stride, a.q_col0, a.k_col0, a.v_col0 = inner, 0, 0, 0
        a.norm_q, a.norm_k = _p(m["norm_q"]), _p(m["norm_k"])
        a.cos, a.sin, a.rot, a.rope_mode = self.cos.data_ptr(), self.sin.data_ptr(), w.rot, w.rope_mode
        a.q_out, a.k_out = self.q_out.data_ptr(), self.k_out.data_ptr()
        a.x, a.h1, a.h2 = self.x.data_ptr(), self.h1.data_ptr(), self.h2.data_ptr()
        a.attn_o, a.act, a.mlp_o = self.attn_o.data_ptr(), self.act.data_ptr(), self.mlp_o.data_ptr()
        a.act2 = self.act2.data_ptr() if self.act2 is not None else None
        self.args = a

    def shard_args(self, row0: int, rows: int) -> BlockArgs:
        """BlockArgs for rows [row0, row0 + rows) of these buffers: every pointer is offset to the range's first row
        and each prefix boundary is moved by row0, which is what a rank that owns the range launches
        (the reference hands its two cards `x + r0*D` and friends the same way, src/models/minimax_h3/dit_sp.cpp:91-110)."""
        a, w = self.args, self.w
        b = BlockArgs()
        for name, _ in BlockArgs._fields_:
            setattr(b, name, getattr(a, name))
        b.rows = rows
        inner, half = w.inner, w.rot // 2
        per_row = {"x": 4 * w.dim, "h1": 2 * w.dim, "h2": 2 * w.dim, "attn_o": 2 * w.dim, "mlp_o": 2 * w.dim,
                   "act": 2 * w.F, "act2": 4 * w.F, "q_out": 2 * inner, "k_out": 2 * inner, "v_out": 2 * inner,
                   "q_in": 2 * a.qkv_stride, "k_in": 2 * a.qkv_stride, "v_in": 2 * a.qkv_stride,
                   "cos": 4 * half, "sin": 4 * half}
        for name, nbytes in per_row.items():
            base = getattr(a, name)
            if base:
                setattr(b, name, base + row0 * nbytes)
        for k in ("shift1", "scale1", "gate1", "shift2", "scale2", "gate2"):
            m = getattr(a, k)
            setattr(b, k, type(m)(m.target, m.prefix, m.prefix_len - row0))
        return b

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in vars(self).values() if isinstance(t, torch.Tensor))


def make_mods(w: Workload, seed: int, device="cuda") -> dict:
    """Two modulation sets (prefix / target) of shift, scale, gate x 2, QK-norm weights, and the
    RMSNorm weights when the block uses RMSNorm."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    m = {}
    for k in ("shift1", "scale1", "gate1", "shift2", "scale2", "gate2"):
        for s in ("_t", "_p"):
            m[k + s] = torch.randn(w.dim, generator=g, device=device) * 0.3
    m["norm_q"] = 1.0 + 0.05 * torch.randn(w.D, generator=g, device=device)
    m["norm_k"] = 1.0 + 0.05 * torch.randn(w.D, generator=g, device=device)
    if w.norm_mode == 1:
        m["norm1_w"] = 1.0 + 0.1 * torch.randn(w.dim, generator=g, device=device)
        m["norm2_w"] = 1.0 + 0.1 * torch.randn(w.dim, generator=g, device=device)
    return m
