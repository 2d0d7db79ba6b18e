#!/usr/bin/env python
"""Benchmark of the fused DiT layer-op chain (one "step" = the ops of one DiT block over one batch
of synthetic token rows).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload qwen1024] [--chain dropin|fused]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...     (N > 1)
    python bench.py --impl reference ...      the CPU restatement of the reference on the host cores

Prints ONE JSON line (rank 0).  `value` is whole-job GB/s of algorithmic bytes (the per-row byte
count of the unfused op list x rows / device time) with inputs resident in HBM; `e2e` is the same
block through mxk_dit_block_ops_host with pinned HOST buffers, copies inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "fused-layer HBM GB/s"
UNIT = "GB/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="mxk", choices=["mxk", "reference", "reference-cuda"])
    ap.add_argument("--workload", default="qwen1024")
    ap.add_argument("--chain", default="dropin", choices=["dropin", "fused"],
                    help="dropin: one launch per reference call; fused: gated_residual+norm and q/k(/v) rope fused")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every rank runs the whole workload's rows; strong: the rows are sharded")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the second chain and the per-op pass")
    ap.add_argument("--graph", action="store_true",
                    help="capture each buffer set's block chain into a CUDA graph once and time replays (small shapes)")
    ap.add_argument("--shard", choices=["frames", "rows"], default="frames",
                    help="strong scaling of a video workload: whole frames per rank (the reference's split) or equal row ranges")
    ap.add_argument("--e2e-chunk-rows", type=int, default=1024, help="rows per staged chunk of the end-to-end leg")
    ap.add_argument("--quant-only", action="store_true",
                    help="time only the block-scale quantiser on the block's activations (profiling aid; prints its own line)")
    ap.add_argument("--tune", action="append", default=[], metavar="KNOB=VALUE",
                    help="override a launch-shape knob of libmxk (see miroxen_b200/csrc/tuning.h); repeatable")
    ap.add_argument("--cpu-rows", type=int, default=0, help="rows of the CPU sample (default: chosen for ~10-30 s)")
    return ap.parse_args()


# ---- clocks -------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self.power = [], set(), None, []
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            try:  # CUDA ordinals follow CUDA_VISIBLE_DEVICES, NVML's do not: go through the UUID
                uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            except Exception:
                pass
            self._stop.wait(0.002)

    def __enter__(self):
        if self.nv:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t:
            self._t.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples),
                "power_w_max": round(max(self.power), 1) if self.power else None}


# ---- CPU arm ------------------------------------------------------------------------------------

def cpu_block(w, rows, prefix_rows, threads, reps, seed=0):
    """Times the oracle's fast build (CPU restatement of the reference kernels) on `rows` rows of the
    workload, all ops of the block in the reference's order.  Returns seconds per pass."""
    import numpy as np
    from oracle import binding as orc
    orc.build(ref=False)
    orc.set_threads(threads, fast=True)
    g = np.random.default_rng(seed)
    d, inner, F, Hh, D = w.dim, w.inner, w.F, w.H, w.D

    def nbf(shape):
        return orc.f32_to_bf16_bits(g.standard_normal(shape, dtype=np.float32))

    x = g.standard_normal((rows, d), dtype=np.float32)
    stride = 3 * inner if w.packed_qkv else inner
    qin = nbf((rows, stride))
    kin = qin if w.packed_qkv else nbf((rows, inner))
    attn_o, mlp_o = nbf((rows, d)), nbf((rows, d))
    act = nbf((rows, 2 * F if w.act_mode == 1 else F))
    vec = lambda s=0.3, m=0.0: (g.standard_normal(d, dtype=np.float32) * np.float32(s) + np.float32(m))
    mods = {k: orc.mod(vec(), vec(), prefix_rows) for k in ("sc1", "sh1", "g1", "sc2", "sh2", "g2")}
    w1 = vec(0.1, 1.0) if w.norm_mode == 1 else None
    w2 = vec(0.1, 1.0) if w.norm_mode == 1 else None
    nq = (1 + 0.05 * g.standard_normal(D)).astype(np.float32)
    nk = (1 + 0.05 * g.standard_normal(D)).astype(np.float32)
    ang = g.uniform(-3.1, 3.1, (rows, max(w.rot // 2, 1))).astype(np.float32)
    cos, sin = np.cos(ang), np.sin(ang)

    def one_pass():
        if w.norm_mode == 0:
            orc.layernorm_mod(x, w.eps, mods["sc1"], mods["sh1"], fast=True)
        else:
            orc.rmsnorm_mod(x, w.eps, w1, mods["sc1"], mods["sh1"], fast=True)
        orc.head_norm_rope(qin, rows, stride, 0, Hh, D, nq, w.eps, cos, sin, w.rot, w.rope_mode, fast=True)
        orc.head_norm_rope(kin, rows, stride, inner if w.packed_qkv else 0, Hh, D, nk, w.eps, cos, sin, w.rot,
                           w.rope_mode, fast=True)
        if w.packed_qkv:
            orc.head_norm_rope(qin, rows, stride, 2 * inner, Hh, D, None, 0.0, None, None, 0, 0, fast=True)
        orc.gated_residual(x, attn_o, mods["g1"], w.gate_tanh, fast=True)
        if w.norm_mode == 0:
            orc.layernorm_mod(x, w.eps, mods["sc2"], mods["sh2"], fast=True)
        else:
            orc.rmsnorm_mod(x, w.eps, w2, mods["sc2"], mods["sh2"], fast=True)
        if w.act_mode == 0:
            orc.gelu_tanh_inplace(act, fast=True)
        else:
            orc.silu_mul(act, F, fast=True)
        orc.gated_residual(x, mlp_o, mods["g2"], w.gate_tanh, fast=True)

    one_pass()  # page in, warm caches
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
    return statistics.median(times)


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_reference_cpu(args, W):
    """--impl reference: the reference has no CPU implementation of these ops (its kernels are CUDA
    only), so the timed CPU arm is the oracle port on all host threads, on a bounded row sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = W[args.workload]
    threads = host_threads()
    rows = args.cpu_rows or min(w.rows, 1088)
    prefix = min(w.prefix_rows, rows * w.prefix_rows // max(w.rows, 1))
    for _ in range(max(args.warmup - 1, 0)):
        pass  # cpu_block warms itself with one untimed pass
    sec = cpu_block(w, rows, prefix, threads, max(args.steps, 1))
    gbs = w.bytes_per_row() * rows / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3 * w.rows / rows, 3),
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "desc": w.desc, "rows": w.rows, "chain": "dropin",
                   "note": "ms_per_step is the sample's time scaled to the workload's rows"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{rows} of {w.rows} rows, every op of the block, median of {max(args.steps, 1)} passes"},
        "e2e": {"value": round(gbs, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- reference CUDA kernels (extra arm) ----------------------------------------------------------

def ref_cuda_chain(w, buf, stream_ptr):
    """One block pass with the REFERENCE's kernels (src/kernels/ops.cu rebuilt for sm_100a)."""
    import ctypes as C
    from oracle import binding as orc
    L = orc.ref_ops()
    RM = orc.RowMod  # same layout as the reference's RowMod

    a = buf.args
    conv = lambda m: RM(m.target, m.prefix, m.prefix_len)
    P, I64, I, F = C.c_void_p, C.c_int64, C.c_int, C.c_float
    L.ref_layernorm_mod.argtypes = [P, I64, I64, F, RM, RM, P, P]
    L.ref_rmsnorm_mod.argtypes = [P, I64, I64, F, P, RM, RM, P, P]
    L.ref_head_norm_rope.argtypes = [P, I64, I64, I64, I, I, P, F, P, P, I, I, P, P]
    L.ref_gated_residual.argtypes = [P, P, I64, I64, RM, I, P]
    L.ref_gelu_tanh_inplace.argtypes = [P, I64, P]
    L.ref_silu_mul.argtypes = [P, I64, I64, P, P]
    rows, d, Fd = a.rows, a.dim, a.F

    def norm(sc, sh, wgt, out):
        if w.norm_mode == 0:
            return L.ref_layernorm_mod(a.x, rows, d, a.eps, conv(sc), conv(sh), out, stream_ptr)
        return L.ref_rmsnorm_mod(a.x, rows, d, a.eps, wgt, conv(sc), conv(sh), out, stream_ptr)

    def go():
        rc = norm(a.scale1, a.shift1, a.norm1_w, a.h1)
        rc |= L.ref_head_norm_rope(a.q_in, rows, a.qkv_stride, a.q_col0, a.H, a.D, a.norm_q, a.eps, a.cos, a.sin, a.rot,
                                   a.rope_mode, a.q_out, stream_ptr)
        rc |= L.ref_head_norm_rope(a.k_in, rows, a.qkv_stride, a.k_col0, a.H, a.D, a.norm_k, a.eps, a.cos, a.sin, a.rot,
                                   a.rope_mode, a.k_out, stream_ptr)
        if w.packed_qkv:
            rc |= L.ref_head_norm_rope(a.v_in, rows, a.qkv_stride, a.v_col0, a.H, a.D, None, 0.0, None, None, 0, 0,
                                       a.v_out, stream_ptr)
        rc |= L.ref_gated_residual(a.x, a.attn_o, rows, d, conv(a.gate1), a.gate_tanh, stream_ptr)
        rc |= norm(a.scale2, a.shift2, a.norm2_w, a.h2)
        if w.act_mode == 0:
            rc |= L.ref_gelu_tanh_inplace(a.act, rows * Fd, stream_ptr)
        else:
            rc |= L.ref_silu_mul(a.act2, rows, Fd, a.act, stream_ptr)
        rc |= L.ref_gated_residual(a.x, a.mlp_o, rows, d, conv(a.gate2), a.gate_tanh, stream_ptr)
        if rc:
            raise RuntimeError("reference kernel launch failed: " + L.ref_last_error().decode())
    return go


# ---- GPU arm ------------------------------------------------------------------------------------

def main():
    args = parse()
    from miroxen_b200.workloads import WORKLOADS as W
    if args.workload not in W:
        raise SystemExit(f"unknown workload {args.workload}; one of {sorted(W)}")
    if args.impl == "reference":
        return run_reference_cpu(args, W)

    import torch
    import torch.distributed as dist
    import miroxen_b200 as mx
    from miroxen_b200 import rope_tables, sharding
    from miroxen_b200.workloads import BlockBuffers, make_mods

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference-cuda" and rank != 0:
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    if world > 1 and args.impl == "mxk":
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    mx.lib()
    for kv in args.tune:
        k, v = kv.split("=")
        mx.set_tuning(k, int(v))
    w = W[args.workload]
    n_gpus = world if args.impl == "mxk" else 1

    # rows of this rank
    if args.scaling == "strong" and n_gpus > 1:
        if w.frames and args.shard == "frames":
            sh = sharding.shard_frames(w.frames, w.rows_per_frame, w.rows - w.frames * w.rows_per_frame, n_gpus, rank)
        else:
            sh = sharding.shard_rows(w.rows, n_gpus, rank)
        rows, row0 = sh.rows, sh.row0
    else:
        rows, row0 = w.rows, 0
    prefix_rows = w.prefix_rows - row0
    total_rows = w.rows * (n_gpus if args.scaling == "weak" else 1)

    # modulation vectors: made on rank 0, broadcast once (set-up, untimed); no collective afterwards
    mods = make_mods(w, seed=1000, device="cuda")
    if world > 1 and args.impl == "mxk":
        sharding.broadcast_modulation(list(mods.values()), src=0)

    # rotary tables for the job's row order, sliced to this rank's rows
    cos = sin = None
    if w.name.startswith("qwen") and not w.packed_qkv:
        n_img = {"qwen1024": (64, 64, 256, 2), "qwen512": (32, 32, 128, 1), "qwen2048": (128, 128, 512, 1),
                 "qwen21_true": None}.get(w.name)
        if n_img:
            ih, iw, nt, batch = n_img
            c1, s1 = rope_tables.qwen_rope_table([("image", ih, iw), ("text", nt)])
            order = [c1[:ih * iw]] * batch + [c1[ih * iw:]] * batch
            order_s = [s1[:ih * iw]] * batch + [s1[ih * iw:]] * batch
            cos, sin = torch.cat(order)[row0:row0 + rows].contiguous(), torch.cat(order_s)[row0:row0 + rows].contiguous()

    n_sets = 2  # two buffer sets, used alternately; every step streams far more than the 126 MB L2
    sets = [BlockBuffers(w, rows, prefix_rows, seed=s, mods=mods, cos=cos, sin=sin) for s in range(n_sets)]
    for b in sets:
        b.args.fused = 1 if args.chain == "fused" else 0
    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream or None

    def barrier():
        torch.cuda.synchronize()
        if world > 1 and args.impl == "mxk":
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world > 1 and args.impl == "mxk":
            t = torch.tensor([v], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return v

    if args.impl == "reference-cuda":
        runners = [ref_cuda_chain(w, b, sp) for b in sets]
        step = lambda i: runners[i % n_sets]()
    elif args.graph:
        # one graph per buffer set, captured after an eager warm-up call (which resolves the per-device caches)
        graphs, per_replay = [], 0
        for b in sets:
            mx.dit_block_ops(b.args, stream)
        torch.cuda.synchronize()
        cap = torch.cuda.Stream()
        cap.wait_stream(stream)
        for b in sets:
            g = torch.cuda.CUDAGraph()
            mx.reset_launch_count()
            with torch.cuda.graph(g, stream=cap):
                mx.dit_block_ops(b.args)
            per_replay = mx.launch_count()
            graphs.append(g)
        torch.cuda.synchronize()
        step = lambda i: graphs[i % n_sets].replay()
    else:
        step = lambda i: mx.dit_block_ops(sets[i % n_sets].args, stream)

    def timed(step_fn, K, Wm):
        for i in range(Wm):
            step_fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        mx.reset_launch_count()
        with ClockSampler(local) as cs:
            e0.record(stream)
            for i in range(K):
                step_fn(i)
            e1.record(stream)
            barrier()
        launches = mx.launch_count() if not (args.graph and args.impl == "mxk") else per_replay * K
        return max_over_ranks(e0.elapsed_time(e1)) / K, launches, cs.summary()

    def quant_rows():
        """The step that follows these ops on the reference's fp8 / fp4 path: the activation block-scale
        quantiser, timed on this block's norm output [rows, dim] and MLP activation [rows, F]."""
        if args.impl == "reference-cuda":
            from oracle import binding as orc
            if not orc.have_ref_blockscale():
                return {"unavailable": "oracle/_ref/libmx_ref_blockscale.so not built"}
            import ctypes as C
            L = orc.ref_blockscale()
            L.ref_quantize_blockscaled.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                                   C.c_void_p, C.c_void_p, C.c_void_p]

            def quant(mode, t, cols, out):
                if L.ref_quantize_blockscaled(mode, t.data_ptr(), cols, rows, cols, out.q.data_ptr(), out.sf.data_ptr(),
                                              out.amax.data_ptr() if out.amax is not None else None, sp):
                    raise RuntimeError("reference quantize_blockscaled failed")
        else:
            def quant(mode, t, cols, out):
                mx.ops.quantize_blockscaled(mode, t, cols, rows, cols, out, stream)
        q_ops = []
        for mode, mname, per_el in ((mx.ops.Q_MXFP8, "mxfp8", 2 + 1 + 1 / 32), (mx.ops.Q_NVFP4, "nvfp4", 2 + 2 + 0.5 + 1 / 16)):
            for src_name, cols in (("h1", w.dim), ("act", w.F)):
                srcs = [getattr(b, src_name) for b in sets]
                outs = [mx.ops.QMat(torch.empty(mx.ops.qdata_bytes(mode, rows, cols), dtype=torch.uint8, device="cuda"),
                                    torch.empty(mx.ops.qscale_bytes(mode, rows, cols), dtype=torch.uint8, device="cuda"),
                                    torch.empty(1, dtype=torch.float32, device="cuda") if mode == mx.ops.Q_NVFP4 else None)
                        for _ in srcs]
                for i in range(3):
                    quant(mode, srcs[i % n_sets], cols, outs[i % n_sets])
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for i in range(K):
                    quant(mode, srcs[i % n_sets], cols, outs[i % n_sets])
                e1.record(stream)
                barrier()
                us = e0.elapsed_time(e1) / K * 1e3
                by = per_el * rows * cols
                q_ops.append({"op": f"quantize_{mname}", "input": f"{src_name} [{rows}, {cols}]", "us": round(us, 2),
                              "bytes": int(by), "gbs": round(by / us / 1e3, 1), "frac": round(by / us / 1e3 / peak_gbs, 3)})
                del outs
        res = {"quantize_blockscaled": q_ops,
               "note": "bytes = bf16 read + codes + scales; nvfp4 reads the input twice (tensor amax first)"}
        if args.impl == "mxk":
            # the MLP activation and its quantisation in one pass, against the same two calls in a row
            am = mx.ops.ACT_GELU_TANH if w.act_mode == 0 else mx.ops.ACT_SILU_MUL
            srcs = [b.act if w.act_mode == 0 else b.act2 for b in sets]
            outs = [mx.ops.act_quantize_mxfp8(am, t, rows, w.F, stream=stream) for t in srcs]
            tmp = [b.act for b in sets]

            def fused(i):
                mx.ops.act_quantize_mxfp8(am, srcs[i % n_sets], rows, w.F, outs[i % n_sets], stream)

            def separate(i):
                if w.act_mode == 0:
                    mx.ops.gelu_tanh_inplace(tmp[i % n_sets], rows * w.F, stream)
                else:
                    mx.ops.silu_mul(srcs[i % n_sets], rows, w.F, tmp[i % n_sets], stream)
                mx.ops.quantize_blockscaled(mx.ops.Q_MXFP8, tmp[i % n_sets], w.F, rows, w.F, outs[i % n_sets], stream)

            pair = {}
            for name, fn in (("one_call", fused), ("two_calls", separate)):
                for i in range(3):
                    fn(i)
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for i in range(K):
                    fn(i)
                e1.record(stream)
                barrier()
                pair[name] = round(e0.elapsed_time(e1) / K * 1e3, 2)
            by = ((2 if w.act_mode == 0 else 4) + 1 + 1 / 32) * rows * w.F
            res["act_quantize_mxfp8"] = {"act": "gelu_tanh" if w.act_mode == 0 else "silu_mul", "input": f"[{rows}, {w.F}]",
                                         "us": pair["one_call"], "us_two_calls": pair["two_calls"], "bytes": int(by),
                                         "gbs": round(by / pair["one_call"] / 1e3, 1),
                                         "frac": round(by / pair["one_call"] / 1e3 / peak_gbs, 3)}
            # the block's first norm and its quantisation in one pass, against the two calls
            bsets = sets
            nouts = [mx.ops.QMat(torch.empty(rows * w.dim, dtype=torch.uint8, device="cuda"),
                                 torch.empty(mx.ops.qscale_bytes(1, rows, w.dim), dtype=torch.uint8, device="cuda")) for _ in bsets]

            def mod(b, name):
                return mx.row_mod(b.mods[name + "_t"], b.mods[name + "_p"], min(max(prefix_rows, 0), rows))

            def norm_one(i):
                b = bsets[i % n_sets]
                if w.norm_mode == 0:
                    mx.ops.layernorm_mod_quant_mxfp8(b.x, rows, w.dim, 1e-6, mod(b, "scale1"), mod(b, "shift1"), nouts[i % n_sets], stream)
                else:
                    mx.ops.rmsnorm_mod_quant_mxfp8(b.x, rows, w.dim, 1e-6, b.mods["norm1_w"], mod(b, "scale1"), mod(b, "shift1"), nouts[i % n_sets], stream)

            def norm_two(i):
                b = bsets[i % n_sets]
                if w.norm_mode == 0:
                    mx.ops.layernorm_mod(b.x, rows, w.dim, 1e-6, mod(b, "scale1"), mod(b, "shift1"), b.h1, stream)
                else:
                    mx.ops.rmsnorm_mod(b.x, rows, w.dim, 1e-6, b.mods["norm1_w"], mod(b, "scale1"), mod(b, "shift1"), b.h1, stream)
                mx.ops.quantize_blockscaled(mx.ops.Q_MXFP8, b.h1, w.dim, rows, w.dim, nouts[i % n_sets], stream)

            pair = {}
            for name, fn in (("one_call", norm_one), ("two_calls", norm_two)):
                for i in range(3):
                    fn(i)
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for i in range(K):
                    fn(i)
                e1.record(stream)
                barrier()
                pair[name] = round(e0.elapsed_time(e1) / K * 1e3, 2)
            # bias add folded into the op that reads the GEMM output next, against add_bias_bf16 + the plain op
            bias_f = torch.randn(2 * w.F, device="cuda") * 0.1
            bias_d = torch.randn(w.dim, device="cuda") * 0.1

            def fold(one, two, bytes_one):
                t = {}
                for name, fn in (("one_call", one), ("two_calls", two)):
                    for i in range(3):
                        fn(i)
                    barrier()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    for i in range(K):
                        fn(i)
                    e1.record(stream)
                    barrier()
                    t[name] = round(e0.elapsed_time(e1) / K * 1e3, 2)
                return {"us": t["one_call"], "us_two_calls": t["two_calls"], "bytes": int(bytes_one),
                        "gbs": round(bytes_one / t["one_call"] / 1e3, 1), "frac": round(bytes_one / t["one_call"] / 1e3 / peak_gbs, 3)}

            if w.act_mode == 0:
                a_one = lambda i: mx.ops.bias_gelu_tanh_inplace(bsets[i % n_sets].act, bias_f, rows, w.F, stream)

                def a_two(i):
                    mx.ops.add_bias_bf16(bsets[i % n_sets].act, bias_f, rows, w.F, stream)
                    mx.ops.gelu_tanh_inplace(bsets[i % n_sets].act, rows * w.F, stream)
                act_bytes = 4 * rows * w.F
            else:
                a_one = lambda i: mx.ops.bias_silu_mul(bsets[i % n_sets].act2, bias_f, rows, w.F, bsets[i % n_sets].act, stream)

                def a_two(i):
                    mx.ops.add_bias_bf16(bsets[i % n_sets].act2, bias_f, rows, 2 * w.F, stream)
                    mx.ops.silu_mul(bsets[i % n_sets].act2, rows, w.F, bsets[i % n_sets].act, stream)
                act_bytes = 6 * rows * w.F
            r_one = lambda i: mx.ops.gated_residual_bias(bsets[i % n_sets].x, bsets[i % n_sets].attn_o, bias_d, rows, w.dim,
                                                         mod(bsets[i % n_sets], "gate1"), w.gate_tanh, stream)

            def r_two(i):
                b = bsets[i % n_sets]
                mx.ops.add_bias_bf16(b.attn_o, bias_d, rows, w.dim, stream)
                mx.ops.gated_residual(b.x, b.attn_o, rows, w.dim, mod(b, "gate1"), w.gate_tanh, stream)
            res["bias_folding"] = {"act": dict(op="bias + " + ("gelu_tanh" if w.act_mode == 0 else "silu_mul"), **fold(a_one, a_two, act_bytes)),
                                   "gated_residual": dict(op="bias + gated_residual", **fold(r_one, r_two, 10 * rows * w.dim))}
            by = (4 + 1 + 1 / 32) * rows * w.dim
            res["norm_mod_quant_mxfp8"] = {"norm": "layernorm" if w.norm_mode == 0 else "rmsnorm", "input": f"[{rows}, {w.dim}]",
                                           "us": pair["one_call"], "us_two_calls": pair["two_calls"], "bytes": int(by),
                                           "gbs": round(by / pair["one_call"] / 1e3, 1),
                                           "frac": round(by / pair["one_call"] / 1e3 / peak_gbs, 3)}
        return res

    K, Wm = max(args.steps, 1), max(args.warmup, 3)
    peaks = {}
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    peak_gbs, peak_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")

    if args.quant_only:
        if rank == 0:
            print(json.dumps({"impl": args.impl, "workload": w.name, "steps": K, "next_rows": quant_rows()}), flush=True)
        return

    ms, launches, clocks = timed(step, K, Wm)
    job_bytes = w.bytes_per_row() * total_rows
    value = job_bytes / (ms * 1e-3) / 1e9

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": n_gpus, "steps": K, "warmup": Wm,
        "ms_per_step": round(ms, 4), "us_per_block": round(ms * 1e3, 1), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "desc": w.desc, "rows_per_gpu": rows, "rows_total": total_rows, "dim": w.dim,
                   "heads": f"{w.H}x{w.D}", "F": w.F, "chain": args.chain, "launch": "cuda graph replay" if args.graph else "stream launches (programmatic dependent launch)", "io_dtype": "bf16 activations, fp32 residual",
                   "bytes_per_row": w.bytes_per_row(), "parallelism": (f"row-sharded x{n_gpus}" + (f" ({args.shard if w.frames else 'rows'})" if args.scaling == "strong" and n_gpus > 1 else "") + ", no collective in the loop"),
                   "l2": f"{n_sets} alternating buffer sets, {sets[0].nbytes() / 1e6:.0f} MB each (> 126 MB L2)"},
        "frac_of_hbm_peak": round(value / n_gpus / peak_gbs, 4), "hbm_peak_gbs": peak_gbs, "hbm_peak_source": peak_src,
        "clocks": clocks, "gpu_launches": int(launches),
    }
    if args.impl != "mxk":
        line["impl"] = args.impl
        line["gpu_launches"] = 7 * K if not w.packed_qkv else 8 * K
        if not args.no_extras:
            line["next_rows"] = quant_rows()
        print(json.dumps(line), flush=True)
        return

    if not args.no_extras:
        # per-op device times inside a timed pass (events between the launches), both chains
        ot = mx.OpTimes()
        per_chain = {}
        for fused in (0, 1):
            for b in sets:
                b.args.fused = fused
                keep = b.args.chunk_rows
                b.args.chunk_rows = 0
            acc = None
            for i in range(3):
                ot.run(sets[i % n_sets].args, stream)
            barrier()
            for i in range(K):
                ot.run(sets[i % n_sets].args, stream)
                t = ot.read()
                acc = t if acc is None else [a + b for a, b in zip(acc, t)]
            names = (["norm_mod", "qkv_norm_rope", "gated_residual_norm", "act", "gated_residual"] if fused else
                     ["norm_mod"] + ["head_norm_rope"] * (3 if w.packed_qkv else 2) + ["gated_residual", "norm_mod", "act", "gated_residual"])
            ob = w.op_bytes(rows)
            act_name = "gelu_tanh_inplace" if w.act_mode == 0 else "silu_mul"
            ops = []
            for nme, tot in zip(names, acc):
                key = act_name if nme == "act" else nme
                by = ob[key] if key != "head_norm_rope" else ob[key] + 2 * (w.rot // 2) * 4 * rows
                us = tot / K * 1e3
                ops.append({"op": key, "us": round(us, 2), "bytes": by, "gbs": round(by / us / 1e3, 1),
                            "frac": round(by / us / 1e3 / peak_gbs, 3)})
            per_chain["fused" if fused else "dropin"] = {"us_per_block": round(sum(o["us"] for o in ops), 1), "ops": ops}
            for b in sets:
                b.args.chunk_rows = keep
        ot.close()
        line["per_op"] = per_chain
        ops = per_chain[args.chain]["ops"]
        top = max(ops, key=lambda o: o["us"])
        line["roofline"] = {"bound": "hbm", "kernel": top["op"], "achieved": top["gbs"], "peak": peak_gbs, "unit": "GB/s",
                            "frac": round(top["gbs"] / peak_gbs, 4), "traffic": None, "peak_source": peak_src}
        tr = ROOT / "profiles" / "dram_traffic.json"
        if tr.exists():
            try:
                t = json.loads(tr.read_text()).get(w.name, {}).get(top["op"])
                if t:
                    line["roofline"]["traffic"] = int(t["bytes_per_row"] * rows)
            except Exception:
                pass
        # the other chain, clean timing
        other = "fused" if args.chain == "dropin" else "dropin"
        for b in sets:
            b.args.fused = 1 if other == "fused" else 0
        ms2, l2, _ = timed(step, K, 3)
        line["other_chain"] = {"chain": other, "ms_per_step": round(ms2, 4), "value": round(job_bytes / (ms2 * 1e-3) / 1e9, 1),
                               "gpu_launches": int(l2)}
        for b in sets:
            b.args.fused = 1 if args.chain == "fused" else 0

    if not args.no_extras and n_gpus == 1:
        line["next_rows"] = quant_rows()

    if not args.no_e2e:
        # end to end: pinned host buffers in, results back in host memory, every step
        hb = BlockBuffers(w, rows, prefix_rows, seed=7, mods=mods, cos=cos, sin=sin, host=True)
        hb.args.fused = 1 if args.chain == "fused" else 0
        pipe = mx.HostPipeline(args.e2e_chunk_rows, w.dim, w.F, w.H, w.D, w.rot, with_v=w.packed_qkv, act_mode=w.act_mode)
        up = down = 0
        for _ in range(2):
            up, down = pipe.run(hb.args)
        barrier()
        Ke = max(3, min(K, 10))
        t0 = time.perf_counter()
        for _ in range(Ke):
            pipe.run(hb.args)
        torch.cuda.synchronize()
        dt = max_over_ranks((time.perf_counter() - t0) / Ke)
        barrier()
        pipe.close()
        line["e2e"] = {"value": round(job_bytes / dt / 1e9, 2), "unit": UNIT, "ms_per_step": round(dt * 1e3, 3),
                       "h2d_bytes_per_step": int(up) * (n_gpus if args.scaling == "weak" else 1),
                       "d2h_bytes_per_step": int(down) * (n_gpus if args.scaling == "weak" else 1), "steps": Ke,
                       "api": f"mxk_dit_block_ops_host (pinned host buffers, {args.e2e_chunk_rows}-row chunks, 3 streams)"}
        del hb

    if rank == 0 and n_gpus == 1 and not args.no_cpu_baseline:
        threads = host_threads()
        crow = args.cpu_rows or min(w.rows, 2176)
        sec = cpu_block(w, crow, min(w.prefix_rows, crow * w.prefix_rows // w.rows), threads, 3)
        line["cpu_baseline"] = {"value": round(w.bytes_per_row() * crow / sec / 1e9, 3), "unit": UNIT, "cores": threads,
                                "kind": "port", "sample": f"{crow} of {w.rows} rows, every op of the block, median of 3 passes",
                                "ms_per_block_scaled": round(sec * 1e3 * w.rows / crow, 2)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
