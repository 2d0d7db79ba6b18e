"""RoPE cos/sin tables, built the way the reference's `prepare()` functions lay them out
(src/models/qwen_image/dit.cpp:151-185; src/models/minimax_h3/dit.cpp:254-262 with the positions of
src/models/minimax_h3/layout.cpp:68-118), but with the O(S) part on the GPU.

libm (through libmxk's host builders) is evaluated only on each axis' distinct positions; the
kernel behind mxk_rope_table_expand gathers those per-axis look-up tables into cos/sin [S, rot/2].
The table values are therefore libm's own, bit for bit.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np
import torch

from ._lib import RopeRun, check, lib
from .ops import _p, _stream


def _i32(vals):
    return (C.c_int32 * len(vals))(*vals)


def _expand(luts_cos, luts_sin, pairs, runs, S, device, stream):
    """luts_*: one fp32 [n_a, pairs_a] numpy array per axis; runs: list of RopeRun."""
    half = int(sum(pairs))
    off, col0, o, c = [], [], 0, 0
    for lc, p in zip(luts_cos, pairs):
        off.append(o), col0.append(c)
        o += lc.size
        c += p
    flat_c = torch.from_numpy(np.concatenate([a.ravel() for a in luts_cos])).to(device)
    flat_s = torch.from_numpy(np.concatenate([a.ravel() for a in luts_sin])).to(device)
    cos = torch.empty((S, half), dtype=torch.float32, device=device)
    sin = torch.empty((S, half), dtype=torch.float32, device=device)
    arr = (RopeRun * len(runs))(*runs)
    check(lib().mxk_rope_table_expand(_p(flat_c), _p(flat_s), (C.c_int64 * len(off))(*off), _i32(pairs), _i32(col0),
                                      len(pairs), arr, len(runs), S, half, _p(cos), _p(sin), _stream(stream)))
    # the look-up tables must outlive the asynchronous launch
    cos._mxk_keepalive = (flat_c, flat_s)
    return cos, sin


def msrope_inv_freq(axes: Sequence[int], theta: float = 10000.0) -> np.ndarray:
    out = np.empty(sum(a // 2 for a in axes), dtype=np.float32)
    check(lib().mxk_msrope_inv_freq_host(_i32(list(axes)), len(axes), theta, out.ctypes.data))
    return out


def qwen_rope_table(segs, axes=(16, 56, 56), theta: float = 10000.0, device="cuda", stream=None):
    """segs: [("text", len) | ("image", ih, iw), ...] in sequence order, the target image last.

    Text rows advance all three axes together; an image sits at the current frame position with
    h/w centred on zero and then advances the position by max(ih, iw).  Returns (cos, sin) fp32
    [S, sum(axes)/2] on `device`.
    """
    invf = msrope_inv_freq(axes, theta)
    pairs = [a // 2 for a in axes]
    # walk the sequence once to find each axis' position range
    lo, hi = [0, 0, 0], [0, 0, 0]
    position, S = 0, 0
    walked = []
    for seg in segs:
        if seg[0] == "text":
            n = int(seg[1])
            if n > 0:
                for a in range(3):
                    lo[a], hi[a] = min(lo[a], position), max(hi[a], position + n - 1)
            walked.append(("text", S, n, position))
            position += n
            S += n
        else:
            ih, iw = int(seg[1]), int(seg[2])
            h0, w0 = -(ih - ih // 2), -(iw - iw // 2)
            lo[0], hi[0] = min(lo[0], position), max(hi[0], position)
            lo[1], hi[1] = min(lo[1], h0), max(hi[1], h0 + ih - 1)
            lo[2], hi[2] = min(lo[2], w0), max(hi[2], w0 + iw - 1)
            walked.append(("image", S, ih, iw, position, h0, w0))
            position += max(ih, iw)
            S += ih * iw
    luts_c, luts_s, k = [], [], 0
    for a in range(3):
        n = hi[a] - lo[a] + 1
        lc = np.empty((n, pairs[a]), dtype=np.float32)
        ls = np.empty((n, pairs[a]), dtype=np.float32)
        f = np.ascontiguousarray(invf[k:k + pairs[a]])
        check(lib().mxk_rope_lut_int_host(lo[a], hi[a], f.ctypes.data, pairs[a], lc.ctypes.data, ls.ctypes.data))
        luts_c.append(lc), luts_s.append(ls)
        k += pairs[a]
    runs = []
    for w in walked:
        if w[0] == "text":
            _, row0, n, pos = w
            if n > 0:
                runs.append(RopeRun(row0, n, 1, 1, _i32([pos - lo[0], pos - lo[1], pos - lo[2]]), _i32([1, 1, 1]),
                                    _i32([0, 0, 0]), _i32([0, 0, 0])))
        else:
            _, row0, ih, iw, pos, h0, w0 = w
            runs.append(RopeRun(row0, ih, iw, 1, _i32([pos - lo[0], h0 - lo[1], w0 - lo[2]]), _i32([0, 1, 0]),
                                _i32([0, 0, 1]), _i32([0, 0, 0])))
    return _expand(luts_c, luts_s, pairs, runs, S, device, stream)


def h3_rope_table(T, F_lat, H, W, A, anchors: Sequence[str], inv_freq, device="cuda", stream=None):
    """First/last-frame layout: T text rows | one frame per anchor | 2A audio rows | F_lat video frames.

    inv_freq: fp32 [nf] (the checkpoint's rope.inv_freq); each of the three axes uses all nf
    frequencies, so rot/2 = 3 nf.  Returns (cos, sin) fp32 [S, 3 nf].
    """
    inv_freq = np.ascontiguousarray(inv_freq, dtype=np.float32)
    nf = inv_freq.size
    hh, ww = H // 2, W // 2
    rpf = hh * ww
    hg = np.empty(hh, dtype=np.float32)
    wg = np.empty(ww, dtype=np.float32)
    check(lib().mxk_h3_spatial_grid_host(H, H, W, hg.ctypes.data))
    check(lib().mxk_h3_spatial_grid_host(W, H, W, wg.ctypes.data))
    ft = np.empty(F_lat, dtype=np.float32)
    check(lib().mxk_h3_frame_times_host(T, F_lat, ft.ctypes.data))
    per = (1, 4, 4, 4, 4)
    total = 0.0
    for f in range(F_lat):
        total += (5.0 / 3.0) * per[f % 5]
    anchor_t = [np.float32(float(T)) if a == "first" else np.float32(float(T) + total - 5.0 / 3.0) for a in anchors]
    for a in anchors:
        if a not in ("first", "last"):
            raise ValueError("anchor must be 'first' or 'last'")
    na = len(anchors)
    t_list = np.concatenate([np.arange(T, dtype=np.float64).astype(np.float32), np.asarray(anchor_t, dtype=np.float32),
                             (float(T) + np.arange(A, dtype=np.float64)).astype(np.float32), ft]).astype(np.float32)
    h_list = np.concatenate([np.zeros(1, np.float32), hg])
    w_list = np.concatenate([np.zeros(1, np.float32), wg])
    luts_c, luts_s = [], []
    for pos in (t_list, h_list, w_list):
        pos = np.ascontiguousarray(pos)
        lc = np.empty((pos.size, nf), dtype=np.float32)
        ls = np.empty((pos.size, nf), dtype=np.float32)
        check(lib().mxk_rope_lut_f32_host(pos.ctypes.data, pos.size, inv_freq.ctypes.data, nf, lc.ctypes.data,
                                          ls.ctypes.data))
        luts_c.append(lc), luts_s.append(ls)
    runs = []
    if T > 0:
        runs.append(RopeRun(0, T, 1, 1, _i32([0, 0, 0]), _i32([1, 0, 0]), _i32([0, 0, 0]), _i32([0, 0, 0])))
    for i in range(na):
        runs.append(RopeRun(T + i * rpf, 1, hh, ww, _i32([T + i, 1, 1]), _i32([0, 0, 0]), _i32([0, 1, 0]), _i32([0, 0, 1])))
    audio0 = T + na * rpf
    if A > 0:
        runs.append(RopeRun(audio0, 2, A, 1, _i32([T + na, 0, 1]), _i32([0, 0, ww - 1]), _i32([1, 0, 0]), _i32([0, 0, 0])))
    video0 = audio0 + 2 * A
    if F_lat > 0:
        runs.append(RopeRun(video0, F_lat, hh, ww, _i32([T + na + A, 1, 1]), _i32([1, 0, 0]), _i32([0, 1, 0]),
                            _i32([0, 0, 1])))
    S = video0 + F_lat * rpf
    return _expand(luts_c, luts_s, [nf, nf, nf], runs, S, device, stream)


def _spatial_grid(dim, H, W):
    g = np.empty(dim // 2, dtype=np.float32)
    check(lib().mxk_h3_spatial_grid_host(dim, H, W, g.ctypes.data))
    return g


_PER_LATENT = (1, 4, 4, 4, 4)
_RESCALE = 5.0 / 3.0


def h3_ref2va_plan(T, refs, F_lat, H, W, A):
    """Per-axis position lists and run descriptors of the reference-conditioned layout
    (src/models/minimax_h3/layout.cpp:121-188): T text rows | one block per reference in request order
    (a video's sound track before its frames) | 2A target audio rows | F_lat target video frames.

    refs: dicts {kind: "image" | "video" | "audio", frames, h, w, audio} (latent geometry; audio =
    latents per channel).  Times run on one clock that starts at T: an image takes one unit, an audio
    reference its length, a video the longer of its track and its frame spans; all in double, as the
    reference, and rounded to fp32 once.  Returns (t_list, h_list, w_list, runs, S); runs index the
    lists as MxkRopeRun does.
    """
    if H % 2 or W % 2:
        raise ValueError("latent extents must be even")
    t_list = [float(i) for i in range(T)]
    h_list, w_list = [np.zeros(1, np.float32)], [np.zeros(1, np.float32)]
    grids = {}

    def grid(gh, gw):
        """(index of the grid's first h entry, first w entry, rows per frame, columns per row)"""
        if (gh, gw) not in grids:
            h0 = sum(a.size for a in h_list)
            w0 = sum(a.size for a in w_list)
            h_list.append(_spatial_grid(gh, gh, gw)), w_list.append(_spatial_grid(gw, gh, gw))
            grids[(gh, gw)] = (h0, w0, gh // 2, gw // 2)
        return grids[(gh, gw)]

    runs = []
    row = [T]
    if T > 0:
        runs.append(RopeRun(0, T, 1, 1, _i32([0, 0, 0]), _i32([1, 0, 0]), _i32([0, 0, 0]), _i32([0, 0, 0])))

    def audio_rows(n, t0, g):
        h0, w0, hh, ww = g
        base_t = len(t_list)
        t_list.extend(t0 + float(a) for a in range(n))
        runs.append(RopeRun(row[0], 2, n, 1, _i32([base_t, 0, w0]), _i32([0, 0, ww - 1]), _i32([1, 0, 0]), _i32([0, 0, 0])))
        row[0] += 2 * n

    def video_rows(g, frames, t0, image):
        h0, w0, hh, ww = g
        base_t = len(t_list)
        t = t0
        for f in range(frames):
            t_list.append(t)
            if not image:
                t += _RESCALE * _PER_LATENT[f % 5]
        runs.append(RopeRun(row[0], frames, hh, ww, _i32([base_t, h0, w0]), _i32([1, 0, 0]), _i32([0, 1, 0]), _i32([0, 0, 1])))
        row[0] += frames * hh * ww

    target = grid(H, W)
    clock = float(T)
    for r in refs:
        kind = r["kind"]
        if kind == "audio":
            if r.get("audio", 0) <= 0:
                raise ValueError("an audio reference needs audio > 0")
            audio_rows(r["audio"], clock, target)
            clock += float(r["audio"])
            continue
        if r["h"] % 2 or r["w"] % 2:
            raise ValueError("latent extents must be even")
        g = grid(r["h"], r["w"])
        if kind == "image":
            video_rows(g, 1, clock, True)
            clock += 1.0
            continue
        if kind != "video":
            raise ValueError(f"unknown reference kind {kind!r}")
        if r.get("audio", 0) > 0:
            audio_rows(r["audio"], clock, g)
        video_rows(g, r["frames"], clock, False)
        span = 0.0
        for f in range(r["frames"]):
            span += _RESCALE * _PER_LATENT[f % 5]
        clock += max(float(r.get("audio", 0)), span)
    if A > 0:
        audio_rows(A, clock, target)
    if F_lat > 0:
        video_rows(target, F_lat, clock, False)
    return (np.asarray(t_list, dtype=np.float64).astype(np.float32), np.concatenate(h_list), np.concatenate(w_list), runs,
            row[0])


def positions_from_plan(t_list, h_list, w_list, runs, S) -> np.ndarray:
    """fp32 [S, 3] positions the runs describe (host side; what mxk_rope_table_expand gathers from)."""
    pos = np.zeros((S, 3), np.float32)
    for r in runs:
        i0, i1, i2 = np.meshgrid(np.arange(r.n0), np.arange(r.n1), np.arange(r.n2), indexing="ij")
        rows = r.row0 + (i0 * r.n1 + i1) * r.n2 + i2
        for a, lst in enumerate((t_list, h_list, w_list)):
            idx = r.base[a] + i0 * r.step0[a] + i1 * r.step1[a] + i2 * r.step2[a]
            pos[rows.ravel(), a] = lst[idx.ravel()]
    return pos


def h3_ref2va_rope_table(T, refs, F_lat, H, W, A, inv_freq, device="cuda", stream=None):
    """cos/sin fp32 [S, 3 nf] of the reference-conditioned layout (h3_ref2va_plan)."""
    inv_freq = np.ascontiguousarray(inv_freq, dtype=np.float32)
    nf = inv_freq.size
    t_list, h_list, w_list, runs, S = h3_ref2va_plan(T, refs, F_lat, H, W, A)
    luts_c, luts_s = [], []
    for pos in (t_list, h_list, w_list):
        pos = np.ascontiguousarray(pos)
        lc = np.empty((pos.size, nf), dtype=np.float32)
        ls = np.empty((pos.size, nf), dtype=np.float32)
        check(lib().mxk_rope_lut_f32_host(pos.ctypes.data, pos.size, inv_freq.ctypes.data, nf, lc.ctypes.data,
                                          ls.ctypes.data))
        luts_c.append(lc), luts_s.append(ls)
    return _expand(luts_c, luts_s, [nf, nf, nf], runs, S, device, stream)


def qwen_timestep_embedding(t: float, device="cuda", stream=None, on_host: bool = False):
    """fp32 [2, 256]: rows for t and for 0 (src/models/qwen_image/dit.cpp:220-230)."""
    if on_host:
        out = np.empty((2, 256), dtype=np.float32)
        check(lib().mxk_qwen_timestep_embedding_host(t, out.ctypes.data))
        return torch.from_numpy(out)
    out = torch.empty((2, 256), dtype=torch.float32, device=device)
    check(lib().mxk_qwen_timestep_embedding(t, _p(out), _stream(stream)))
    return out


def h3_time_basis(ts, table, stream=None):
    """ts fp32 [nt], table fp32 [grid, basis] on the GPU -> fp32 [nt, basis]."""
    nt, (grid, basis) = ts.numel(), table.shape
    out = torch.empty((nt, basis), dtype=torch.float32, device=ts.device)
    check(lib().mxk_h3_time_basis(_p(ts), nt, _p(table), grid, basis, _p(out), _stream(stream)))
    return out
