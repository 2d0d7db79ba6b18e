#!/usr/bin/env python
"""Benchmark of the fused DiT layer-op chain (one "step" = the ops of one DiT block over one batch
of synthetic token rows).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload qwen1024] [--chain dropin|fused]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...     (N > 1)
    python bench.py --impl reference ...      the reference's own CUDA kernels (oracle/_ref) on the same buffers
    python bench.py --impl reference-cpu ...  the CPU restatement of the reference on the host cores

Prints ONE JSON line (rank 0).  `value` is whole-job GB/s of algorithmic bytes (the per-row byte
count of the unfused op list x rows / device time) with inputs resident in HBM; `e2e` is the same
block through mxk_dit_block_ops_host with pinned HOST buffers, copies inside the timed region.
With N > 1 the token rows of ONE workload are sharded over the ranks (strong scaling, no collective
in the timed loop); `--scaling weak` runs N replicas instead.
"""
from __future__ import annotations

import argparse
import json
import math
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
L2_BYTES = 126e6
MIN_TIMED_MS = 120.0  # the K-step window is repeated until this much device time has been sampled


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="mxk", choices=["mxk", "reference", "reference-cuda", "reference-cpu"])
    ap.add_argument("--workload", default="qwen1024")
    ap.add_argument("--chain", default="dropin", choices=["dropin", "fused"],
                    help="dropin: one launch per reference call; fused: gated_residual+norm and q/k(/v) rope fused")
    ap.add_argument("--scaling", default=None, choices=["weak", "strong"],
                    help="strong (default for N > 1): the workload's rows are sharded over the ranks; "
                         "weak: every rank runs the whole workload's rows")
    ap.add_argument("--repeats", type=int, default=0, help="K-step windows timed (default: >= 5, enough for ~120 ms)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the per-op pass, the second chain, the reference kernels and the extra strong-scaling records")
    ap.add_argument("--graph", action="store_true",
                    help="capture each buffer set's block chain into a CUDA graph once and time replays (small shapes)")
    ap.add_argument("--shard", choices=["frames", "rows"], default=None,
                    help="strong scaling of a video workload: whole frames per rank (the reference's split) or equal "
                         "row ranges (default: rows for the main line; the video record reports both)")
    ap.add_argument("--e2e-chunk-rows", type=int, default=1024, help="rows per staged chunk of the end-to-end leg")
    ap.add_argument("--rows", type=int, default=0, help="run only the first ROWS rows of the workload (tuning aid)")
    ap.add_argument("--ops-only", action="store_true",
                    help="time only the isolated per-op figures (profiling / tuning aid; prints its own line)")
    ap.add_argument("--linear-only", action="store_true",
                    help="time only the linear layers with the residual in the GEMM epilogue against cuBLAS + the separate ops "
                         "(prints its own line)")
    ap.add_argument("--exchange-only", action="store_true",
                    help="time only the head exchange of sequence-parallel attention over the ranks' peer buffers (N >= 1)")
    ap.add_argument("--quant-only", action="store_true",
                    help="time only the block-scale quantiser on the block's activations (profiling aid; prints its own line)")
    ap.add_argument("--no-numa-bind", action="store_true",
                    help="leave the process where the launcher put it (default: each rank moves onto the CPUs of its GPU's NUMA "
                         "node before it allocates pinned host buffers; a no-op where the host reports no node)")
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
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_mhz_min": int(min(self.samples)),
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples),
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


def cpu_baseline(w, rows, reps):
    threads = host_threads()
    sec = cpu_block(w, rows, min(w.prefix_rows, rows * w.prefix_rows // max(w.rows, 1)), threads, reps)
    return {"value": round(w.bytes_per_row() * rows / sec / 1e9, 3), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{rows} of {w.rows} rows, every op of the block, median of {reps} passes",
            "ms_per_block_scaled": round(sec * 1e3 * w.rows / rows, 2),
            "what": "CPU restatement of the reference's CUDA kernels (the reference has no CPU implementation of these ops)"}


def job_config(w, chain, n_gpus, scaling, shard):
    """The `config` object: a function of the job alone, so that both arms print the same one."""
    split = "replicas" if scaling == "weak" or n_gpus == 1 else (f"token rows sharded by {shard}")
    return {"workload": w.name, "desc": w.desc, "rows": w.rows, "dim": w.dim, "heads": f"{w.H}x{w.D}", "F": w.F, "chain": chain,
            "io_dtype": "bf16 activations, fp32 residual and arithmetic", "bytes_per_row": w.bytes_per_row(),
            "parallelism": f"{n_gpus} GPU(s), {split}, no collective in the timed loop",
            "l2": "alternating buffer sets, together > 3x the 126 MB L2"}


def run_reference_cpu(args, W, why=None):
    """The CPU restatement of the reference kernels on all host threads, on a bounded row sample."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    w = W[args.workload]
    rows = args.cpu_rows or min(w.rows, 1088)
    cb = cpu_baseline(w, rows, max(min(args.steps, 20), 1))
    scaling = args.scaling or ("strong" if args.gpus > 1 else "weak")
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_block_scaled"],
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": job_config(w, "dropin", args.gpus, scaling, args.shard or "rows"),
        "reference_kind": "cpu port of the reference's CUDA kernels (oracle/liboracle_fast.so)",
        "note": "ms_per_step is the sample's time scaled to the workload's rows",
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if why:
        line["fallback"] = why
    print(json.dumps(line), flush=True)


# ---- reference CUDA kernels ----------------------------------------------------------------------

def ref_cuda_chain(w, buf, stream_ptr, mark=None):
    """One block pass with the REFERENCE's kernels (src/kernels/ops.cu rebuilt for sm_100a) on the
    buffers of `buf`; `mark()` (optional) is called before the first launch and after each launch."""
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
    tick = mark or (lambda: None)

    def norm(sc, sh, wgt, out):
        if w.norm_mode == 0:
            return L.ref_layernorm_mod(a.x, rows, d, a.eps, conv(sc), conv(sh), out, stream_ptr)
        return L.ref_rmsnorm_mod(a.x, rows, d, a.eps, wgt, conv(sc), conv(sh), out, stream_ptr)

    def go():
        tick()
        rc = norm(a.scale1, a.shift1, a.norm1_w, a.h1)
        tick()
        rc |= L.ref_head_norm_rope(a.q_in, rows, a.qkv_stride, a.q_col0, a.H, a.D, a.norm_q, a.eps, a.cos, a.sin, a.rot,
                                   a.rope_mode, a.q_out, stream_ptr)
        tick()
        rc |= L.ref_head_norm_rope(a.k_in, rows, a.qkv_stride, a.k_col0, a.H, a.D, a.norm_k, a.eps, a.cos, a.sin, a.rot,
                                   a.rope_mode, a.k_out, stream_ptr)
        tick()
        if w.packed_qkv:
            rc |= L.ref_head_norm_rope(a.v_in, rows, a.qkv_stride, a.v_col0, a.H, a.D, None, 0.0, None, None, 0, 0,
                                       a.v_out, stream_ptr)
            tick()
        rc |= L.ref_gated_residual(a.x, a.attn_o, rows, d, conv(a.gate1), a.gate_tanh, stream_ptr)
        tick()
        rc |= norm(a.scale2, a.shift2, a.norm2_w, a.h2)
        tick()
        if w.act_mode == 0:
            rc |= L.ref_gelu_tanh_inplace(a.act, rows * Fd, stream_ptr)
        else:
            rc |= L.ref_silu_mul(a.act2, rows, Fd, a.act, stream_ptr)
        tick()
        rc |= L.ref_gated_residual(a.x, a.mlp_o, rows, d, conv(a.gate2), a.gate_tanh, stream_ptr)
        tick()
        if rc:
            raise RuntimeError("reference kernel launch failed: " + L.ref_last_error().decode())
    return go


def dropin_op_names(w):
    return ["norm_mod"] + ["head_norm_rope"] * (3 if w.packed_qkv else 2) + ["gated_residual", "norm_mod", "act", "gated_residual"]


def op_rows(w, names, us_list, rows, peak_gbs):
    ob = w.op_bytes(rows)
    act_name = "gelu_tanh_inplace" if w.act_mode == 0 else "silu_mul"
    ops = []
    for nme, us in zip(names, us_list):
        key = act_name if nme == "act" else nme
        # the token's cos/sin row is charged to each head_norm_rope call that reads it
        by = ob[key] if key != "head_norm_rope" else ob[key] + 2 * (w.rot // 2) * 4 * rows
        ops.append({"op": key, "us": round(us, 2), "bytes": by, "gbs": round(by / us / 1e3, 1),
                    "frac": round(by / us / 1e3 / peak_gbs, 3)})
    return ops


# ---- GPU arms -----------------------------------------------------------------------------------

class Env:
    """Process-wide handles of a GPU run."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        import miroxen_b200 as mx
        self.torch, self.dist, self.mx, self.args = torch, dist, mx, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.distributed = False
        pk = ROOT / "MEASURED_PEAKS.json"
        peaks = json.loads(pk.read_text()) if pk.exists() else {}
        self.peak_gbs, self.peak_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")

    def start(self, distributed):
        torch = self.torch
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
        torch.cuda.set_device(self.local)
        # host-buffer path: run on (and allocate pinned memory from) the NUMA node next to this rank's GPU
        self.host_placement = {"node": None, "why": "--no-numa-bind"}
        if not self.args.no_numa_bind:
            from miroxen_b200 import hostmem
            self.host_placement = hostmem.bind_to_device_node(self.local)
            self.host_placement["cpus"] = len(self.host_placement.get("cpus", []))
        if distributed and self.world > 1:
            self.dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.distributed = True
        self.mx.lib()
        for kv in self.args.tune:
            k, v = kv.split("=")
            self.mx.set_tuning(k, int(v))
        self.stream = torch.cuda.current_stream()
        self.sp = self.stream.cuda_stream or None

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.distributed:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        if self.distributed:
            t = self.torch.tensor([v], dtype=self.torch.float64, device="cuda")
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            return float(t.item())
        return v

    def sum_over_ranks(self, v):
        if self.distributed:
            t = self.torch.tensor([v], dtype=self.torch.float64, device="cuda")
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
            return float(t.item())
        return v

    def event_ms(self, fn, n):
        """Device time of n calls of fn(i), CUDA events on the launching stream."""
        torch = self.torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(self.stream)
        for i in range(n):
            fn(i)
        e1.record(self.stream)
        e1.synchronize()
        return e0.elapsed_time(e1)


class Job:
    """This rank's rows of one workload: alternating buffer sets and the step function."""

    def __init__(self, env, w, rows, row0, mods=None, chain="dropin", impl="mxk"):
        from miroxen_b200.workloads import BlockBuffers, make_mods, rope_tables_for
        torch = env.torch
        self.env, self.w, self.rows, self.row0, self.impl = env, w, rows, row0, impl
        self.prefix_rows = w.prefix_rows - row0
        if mods is None:
            # made on every rank from the same seed, then broadcast from rank 0 once (set-up, untimed)
            mods = make_mods(w, seed=1000, device="cuda")
            if env.distributed:
                from miroxen_b200 import sharding
                sharding.broadcast_modulation(list(mods.values()), src=0)
        self.mods = mods
        cos, sin = rope_tables_for(w)
        if cos is not None:
            cos, sin = cos[row0:row0 + rows].contiguous(), sin[row0:row0 + rows].contiguous()
        self.cos, self.sin = cos, sin
        one = BlockBuffers(w, rows, self.prefix_rows, seed=0, mods=mods, cos=cos, sin=sin)
        # enough sets that a set is long gone from the 126 MB L2 when its turn comes again
        self.n_sets = max(2, math.ceil(3.2 * L2_BYTES / max(one.nbytes(), 1)))
        self.sets = [one] + [BlockBuffers(w, rows, self.prefix_rows, seed=s, mods=mods, cos=cos, sin=sin)
                             for s in range(1, self.n_sets)]
        self.set_chain(chain)
        self.graphs, self.per_replay = None, 0
        if impl != "mxk":
            self.runners = [ref_cuda_chain(w, b, env.sp) for b in self.sets]

    def set_chain(self, chain):
        self.chain = chain
        for b in self.sets:
            b.args.fused = 1 if chain == "fused" else 0

    def capture_graphs(self):
        env, torch, mx = self.env, self.env.torch, self.env.mx
        for b in self.sets:
            mx.dit_block_ops(b.args, env.stream)  # eager warm-up: resolves the per-device caches
        torch.cuda.synchronize()
        cap = torch.cuda.Stream()
        cap.wait_stream(env.stream)
        self.graphs = []
        for b in self.sets:
            g = torch.cuda.CUDAGraph()
            mx.reset_launch_count()
            with torch.cuda.graph(g, stream=cap):
                mx.dit_block_ops(b.args)
            self.per_replay = mx.launch_count()
            self.graphs.append(g)
        torch.cuda.synchronize()

    def step(self, i):
        if self.impl != "mxk":
            self.runners[i % self.n_sets]()
        elif self.graphs:
            self.graphs[i % self.n_sets].replay()
        else:
            self.env.mx.dit_block_ops(self.sets[i % self.n_sets].args, self.env.stream)

    def set_bytes(self):
        return self.sets[0].nbytes()

    def timed(self, K, warm, repeats=0, clocks=False):
        """`repeats` windows of exactly K steps each (barrier + synchronize either side of every window,
        max over ranks per window).  Returns (median ms per step, stats, launches per window, clock summary)."""
        env = self.env
        for i in range(warm):
            self.step(i)
        env.barrier()
        first = env.max_over_ranks(env.event_ms(self.step, K))
        env.barrier()
        R = repeats or int(min(60, max(5, math.ceil(MIN_TIMED_MS / max(first, 1e-3)))))
        if env.distributed:  # every rank must run the same number of windows
            R = int(env.max_over_ranks(float(R)))
        windows, launches = [], 0
        sampler = ClockSampler(env.local) if clocks else None
        if sampler:
            sampler.__enter__()
        try:
            for _ in range(R):
                env.mx.reset_launch_count()
                ms = env.event_ms(self.step, K)
                launches = env.mx.launch_count() if not self.graphs else self.per_replay * K
                env.barrier()
                windows.append(env.max_over_ranks(ms) / K)
        finally:
            if sampler:
                sampler.__exit__()
        med = statistics.median(windows)
        stats = {"repeats": R, "ms_per_step_min": round(min(windows), 4), "ms_per_step_max": round(max(windows), 4),
                 "timed_ms_total": round(sum(windows) * K, 1)}
        return med, stats, launches, (sampler.summary() if sampler else None)

    def per_op(self, K, fused):
        """Per-op device times inside a timed pass (events between the launches)."""
        env, mx = self.env, self.env.mx
        w = self.w
        keep_chain = self.chain
        ot = mx.OpTimes()
        saved = []
        for b in self.sets:
            b.args.fused = fused
            saved.append(b.args.chunk_rows)
            b.args.chunk_rows = 0
        acc = None
        for i in range(3):
            ot.run(self.sets[i % self.n_sets].args, env.stream)
        env.barrier()
        for i in range(K):
            ot.run(self.sets[i % self.n_sets].args, env.stream)
            t = ot.read()
            acc = t if acc is None else [a + b for a, b in zip(acc, t)]
        ot.close()
        for b, c in zip(self.sets, saved):
            b.args.chunk_rows = c
        self.set_chain(keep_chain)
        names = ["norm_mod", "qkv_norm_rope", "gated_residual_norm", "act", "gated_residual"] if fused else dropin_op_names(w)
        ops = op_rows(w, names, [t / K * 1e3 for t in acc], self.rows, env.peak_gbs)
        return {"us_per_block": round(sum(o["us"] for o in ops), 1), "ops": ops}

    def per_op_marginal(self, K, fused):
        """Each op's cost inside the chain, launches overlapping as in the timed region: the chain's prefixes
        (first op; first two ops; ...) are timed like the whole block and consecutive prefixes subtracted.
        The figures add up to the block time by construction."""
        env, mx, w = self.env, self.env.mx, self.w
        keep_chain = self.chain
        saved = []
        for b in self.sets:
            b.args.fused = fused
            saved.append(b.args.chunk_rows)
            b.args.chunk_rows = 0
        names = ["norm_mod", "qkv_norm_rope", "gated_residual_norm", "act", "gated_residual"] if fused else dropin_op_names(w)
        totals = []
        for n in range(1, len(names) + 1):
            step = lambda i, n=n: mx.dit_block_ops_prefix(self.sets[i % self.n_sets].args, n, env.stream)
            for i in range(3):
                step(i)
            env.barrier()
            totals.append(statistics.median([env.event_ms(step, K) / K * 1e3 for _ in range(5)]))
        for b, c in zip(self.sets, saved):
            b.args.chunk_rows = c
        self.set_chain(keep_chain)
        us = [totals[0]] + [max(totals[i] - totals[i - 1], 1e-3) for i in range(1, len(totals))]
        ops = op_rows(w, names, us, self.rows, env.peak_gbs)
        return {"us_per_block": round(totals[-1], 1), "ops": ops}

    def per_op_isolated(self, K):
        """Each op of the block timed on its own: K back-to-back launches of the same op over the rotating
        buffer sets (inputs never in L2; each launch's write-backs drain during the next launch of the same
        op, so a launch window moves exactly the op's own bytes).  This is the per-op figure the in-chain
        numbers are compared with: inside the chain an op also pays for the previous op's draining writes."""
        env, mx, w, rows = self.env, self.env.mx, self.w, self.rows
        st, n = env.stream, self.n_sets
        pl = self.prefix_rows

        def mod(b, name):
            return mx.row_mod(b.mods[name + "_t"], b.mods[name + "_p"], pl)

        def norm(b, k, out):
            if w.norm_mode == 0:
                mx.layernorm_mod(b.x, rows, w.dim, w.eps, mod(b, "scale" + k), mod(b, "shift" + k), out, st)
            else:
                mx.rmsnorm_mod(b.x, rows, w.dim, w.eps, b.mods["norm" + k + "_w"], mod(b, "scale" + k), mod(b, "shift" + k), out, st)

        inner = w.inner
        stride = 3 * inner if w.packed_qkv else inner

        def rope(b, which):
            src = b.qkv if w.packed_qkv else (b.q_in if which == 0 else b.k_in)
            col0 = which * inner if w.packed_qkv else 0
            out = (b.q_out, b.k_out, getattr(b, "v_out", None))[which]
            if which < 2:
                mx.head_norm_rope(src, rows, stride, col0, w.H, w.D, b.mods["norm_q" if which == 0 else "norm_k"], w.eps, b.cos, b.sin,
                                  w.rot, w.rope_mode, out, st)
            else:
                mx.head_norm_rope(src, rows, stride, col0, w.H, w.D, None, 0.0, None, None, 0, 0, out, st)

        def qkv(b):
            specs = [mx.HeadSpec(b.qkv if w.packed_qkv else b.q_in, stride, 0, b.mods["norm_q"], b.q_out, w.rot, w.rope_mode),
                     mx.HeadSpec(b.qkv if w.packed_qkv else b.k_in, stride, inner if w.packed_qkv else 0, b.mods["norm_k"], b.k_out, w.rot, w.rope_mode)]
            if w.packed_qkv:
                specs.append(mx.HeadSpec(b.qkv, stride, 2 * inner, None, b.v_out, 0, 0))
            mx.qkv_norm_rope(specs, rows, w.H, w.D, w.eps, b.cos, b.sin, st)

        def act(b):
            if w.act_mode == 0:
                mx.gelu_tanh_inplace(b.act, rows * w.F, st)
            else:
                mx.silu_mul(b.act2, rows, w.F, b.act, st)

        def res_norm(b):
            mx.gated_residual_norm(b.x, b.attn_o, rows, w.dim, mod(b, "gate1"), w.gate_tanh, w.norm_mode, w.eps,
                                   b.mods.get("norm2_w"), mod(b, "scale2"), mod(b, "shift2"), b.h2, st)

        ob = w.op_bytes(rows)
        tab = 2 * (w.rot // 2) * 4 * rows
        act_name = "gelu_tanh_inplace" if w.act_mode == 0 else "silu_mul"
        ops = [("norm_mod", lambda b: norm(b, "1", b.h1), ob["norm_mod"]),
               ("head_norm_rope", lambda b: rope(b, 0), ob["head_norm_rope"] + tab)]
        if w.packed_qkv:
            ops.append(("head_norm_rope (v copy)", lambda b: rope(b, 2), ob["head_norm_rope"]))
        ops += [("gated_residual", lambda b: mx.gated_residual(b.x, b.attn_o, rows, w.dim, mod(b, "gate1"), w.gate_tanh, st), ob["gated_residual"]),
                (act_name, act, ob[act_name]),
                ("qkv_norm_rope", qkv, ob["qkv_norm_rope"]),
                ("gated_residual_norm", res_norm, ob["gated_residual_norm"])]
        out = []
        for name, fn, by in ops:
            step = lambda i, fn=fn: fn(self.sets[i % n])
            for i in range(3):
                step(i)
            env.barrier()
            reps = [env.event_ms(step, K) / K * 1e3 for _ in range(3)]
            us = statistics.median(reps)
            out.append({"op": name, "us": round(us, 2), "bytes": by, "gbs": round(by / us / 1e3, 1),
                        "frac": round(by / us / 1e3 / env.peak_gbs, 3)})
        return out

    def close(self):
        self.sets, self.graphs = [], None
        if self.impl != "mxk":
            self.runners = []
        self.env.torch.cuda.empty_cache()


def shard_of(w, n, rank, by):
    from miroxen_b200 import sharding
    if by == "frames" and w.frames:
        return sharding.shard_frames(w.frames, w.rows_per_frame, w.rows - w.frames * w.rows_per_frame, n, rank)
    return sharding.shard_rows(w.rows, n, rank)


def quant_rows(env, job, K, impl):
    """The step that follows these ops on the reference's fp8 / fp4 path: the activation block-scale
    quantiser, timed on this block's norm output [rows, dim] and MLP activation [rows, F]."""
    torch, mx = env.torch, env.mx
    w, rows, sets, n_sets, stream, sp, peak_gbs = job.w, job.rows, job.sets, job.n_sets, env.stream, env.sp, env.peak_gbs
    prefix_rows = job.prefix_rows

    def time_us(fn):
        for i in range(3):
            fn(i)
        env.barrier()
        return env.event_ms(fn, K) / K * 1e3

    if impl != "mxk":
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
            us = time_us(lambda i: quant(mode, srcs[i % n_sets], cols, outs[i % n_sets]))
            by = per_el * rows * cols
            q_ops.append({"op": f"quantize_{mname}", "input": f"{src_name} [{rows}, {cols}]", "us": round(us, 2),
                          "bytes": int(by), "gbs": round(by / us / 1e3, 1), "frac": round(by / us / 1e3 / peak_gbs, 3)})
            del outs
    res = {"quantize_blockscaled": q_ops,
           "note": "bytes = bf16 read + codes + scales; nvfp4 reads the input twice (tensor amax first)"}
    if impl != "mxk":
        return res

    def pair_us(one, two):
        return round(time_us(one), 2), round(time_us(two), 2)

    def mod(b, name):
        return mx.row_mod(b.mods[name + "_t"], b.mods[name + "_p"], min(max(prefix_rows, 0), rows))

    # the MLP activation and its quantisation in one pass, against the same two calls in a row
    am = mx.ops.ACT_GELU_TANH if w.act_mode == 0 else mx.ops.ACT_SILU_MUL
    srcs = [b.act if w.act_mode == 0 else b.act2 for b in sets]
    outs = [mx.ops.act_quantize_mxfp8(am, t, rows, w.F, stream=stream) for t in srcs]
    tmp = [b.act for b in sets]

    def act_two(i):
        if w.act_mode == 0:
            mx.ops.gelu_tanh_inplace(tmp[i % n_sets], rows * w.F, stream)
        else:
            mx.ops.silu_mul(srcs[i % n_sets], rows, w.F, tmp[i % n_sets], stream)
        mx.ops.quantize_blockscaled(mx.ops.Q_MXFP8, tmp[i % n_sets], w.F, rows, w.F, outs[i % n_sets], stream)

    one, two = pair_us(lambda i: mx.ops.act_quantize_mxfp8(am, srcs[i % n_sets], rows, w.F, outs[i % n_sets], stream), act_two)
    by = ((2 if w.act_mode == 0 else 4) + 1 + 1 / 32) * rows * w.F
    res["act_quantize_mxfp8"] = {"act": "gelu_tanh" if w.act_mode == 0 else "silu_mul", "input": f"[{rows}, {w.F}]",
                                 "us": one, "us_two_calls": two, "bytes": int(by), "gbs": round(by / one / 1e3, 1),
                                 "frac": round(by / one / 1e3 / peak_gbs, 3)}
    del outs
    # the block's first norm and its quantisation in one pass, against the two calls
    nouts = [mx.ops.QMat(torch.empty(rows * w.dim, dtype=torch.uint8, device="cuda"),
                         torch.empty(mx.ops.qscale_bytes(1, rows, w.dim), dtype=torch.uint8, device="cuda")) for _ in sets]

    def norm_one(i):
        b = sets[i % n_sets]
        if w.norm_mode == 0:
            mx.ops.layernorm_mod_quant_mxfp8(b.x, rows, w.dim, 1e-6, mod(b, "scale1"), mod(b, "shift1"), nouts[i % n_sets], stream)
        else:
            mx.ops.rmsnorm_mod_quant_mxfp8(b.x, rows, w.dim, 1e-6, b.mods["norm1_w"], mod(b, "scale1"), mod(b, "shift1"), nouts[i % n_sets], stream)

    def norm_two(i):
        b = sets[i % n_sets]
        if w.norm_mode == 0:
            mx.ops.layernorm_mod(b.x, rows, w.dim, 1e-6, mod(b, "scale1"), mod(b, "shift1"), b.h1, stream)
        else:
            mx.ops.rmsnorm_mod(b.x, rows, w.dim, 1e-6, b.mods["norm1_w"], mod(b, "scale1"), mod(b, "shift1"), b.h1, stream)
        mx.ops.quantize_blockscaled(mx.ops.Q_MXFP8, b.h1, w.dim, rows, w.dim, nouts[i % n_sets], stream)

    one, two = pair_us(norm_one, norm_two)
    by = (4 + 1 + 1 / 32) * rows * w.dim
    res["norm_mod_quant_mxfp8"] = {"norm": "layernorm" if w.norm_mode == 0 else "rmsnorm", "input": f"[{rows}, {w.dim}]",
                                   "us": one, "us_two_calls": two, "bytes": int(by), "gbs": round(by / one / 1e3, 1),
                                   "frac": round(by / one / 1e3 / peak_gbs, 3)}
    # NVFP4 in one pass: the producing op leaves the tensor maximum behind, the quantiser skips its first read pass
    amax = [torch.zeros(1, dtype=torch.float32, device="cuda") for _ in sets]
    fouts = [mx.ops.QMat(torch.empty(mx.ops.qdata_bytes(2, rows, w.dim), dtype=torch.uint8, device="cuda"),
                         torch.empty(mx.ops.qscale_bytes(2, rows, w.dim), dtype=torch.uint8, device="cuda"), amax[i]) for i in range(n_sets)]

    def norm_amax(i):
        b = sets[i % n_sets]
        if w.norm_mode == 0:
            mx.ops.layernorm_mod_amax(b.x, rows, w.dim, 1e-6, mod(b, "scale1"), mod(b, "shift1"), b.h1, amax[i % n_sets], stream)
        else:
            mx.ops.rmsnorm_mod_amax(b.x, rows, w.dim, 1e-6, b.mods["norm1_w"], mod(b, "scale1"), mod(b, "shift1"), b.h1, amax[i % n_sets], stream)

    def norm_plain(i):
        b = sets[i % n_sets]
        if w.norm_mode == 0:
            mx.ops.layernorm_mod(b.x, rows, w.dim, 1e-6, mod(b, "scale1"), mod(b, "shift1"), b.h1, stream)
        else:
            mx.ops.rmsnorm_mod(b.x, rows, w.dim, 1e-6, b.mods["norm1_w"], mod(b, "scale1"), mod(b, "shift1"), b.h1, stream)

    def fp4_one(i):
        norm_amax(i)
        mx.ops.quantize_nvfp4_known_amax(sets[i % n_sets].h1, w.dim, rows, w.dim, amax[i % n_sets], fouts[i % n_sets], stream)

    def fp4_two(i):
        norm_plain(i)
        mx.ops.quantize_blockscaled(mx.ops.Q_NVFP4, sets[i % n_sets].h1, w.dim, rows, w.dim, fouts[i % n_sets], stream)

    one, two = pair_us(fp4_one, fp4_two)
    na, npl = pair_us(norm_amax, norm_plain)
    res["norm_then_nvfp4"] = {"norm": "layernorm" if w.norm_mode == 0 else "rmsnorm", "input": f"[{rows}, {w.dim}]",
                              "us_norm_amax_then_one_pass_quantiser": one, "us_norm_then_two_pass_quantiser": two,
                              "us_norm_with_amax": na, "us_norm": npl,
                              "note": "same bytes out; the tensor maximum is a by-product of the norm instead of a read pass of the quantiser"}
    del fouts
    # bias add folded into the op that reads the GEMM output next, against add_bias_bf16 + the plain op
    bias_f = torch.randn(2 * w.F, device="cuda") * 0.1
    bias_d = torch.randn(w.dim, device="cuda") * 0.1

    def fold(one_fn, two_fn, bytes_one):
        a, b2 = pair_us(one_fn, two_fn)
        return {"us": a, "us_two_calls": b2, "bytes": int(bytes_one), "gbs": round(bytes_one / a / 1e3, 1),
                "frac": round(bytes_one / a / 1e3 / peak_gbs, 3)}

    if w.act_mode == 0:
        a_one = lambda i: mx.ops.bias_gelu_tanh_inplace(sets[i % n_sets].act, bias_f, rows, w.F, stream)

        def a_two(i):
            mx.ops.add_bias_bf16(sets[i % n_sets].act, bias_f, rows, w.F, stream)
            mx.ops.gelu_tanh_inplace(sets[i % n_sets].act, rows * w.F, stream)
        act_bytes = 4 * rows * w.F
    else:
        a_one = lambda i: mx.ops.bias_silu_mul(sets[i % n_sets].act2, bias_f, rows, w.F, sets[i % n_sets].act, stream)

        def a_two(i):
            mx.ops.add_bias_bf16(sets[i % n_sets].act2, bias_f, rows, 2 * w.F, stream)
            mx.ops.silu_mul(sets[i % n_sets].act2, rows, w.F, sets[i % n_sets].act, stream)
        act_bytes = 6 * rows * w.F
    r_one = lambda i: mx.ops.gated_residual_bias(sets[i % n_sets].x, sets[i % n_sets].attn_o, bias_d, rows, w.dim,
                                                 mod(sets[i % n_sets], "gate1"), w.gate_tanh, stream)

    def r_two(i):
        b = sets[i % n_sets]
        mx.ops.add_bias_bf16(b.attn_o, bias_d, rows, w.dim, stream)
        mx.ops.gated_residual(b.x, b.attn_o, rows, w.dim, mod(b, "gate1"), w.gate_tanh, stream)
    res["bias_folding"] = {"act": dict(op="bias + " + ("gelu_tanh" if w.act_mode == 0 else "silu_mul"), **fold(a_one, a_two, act_bytes)),
                           "gated_residual": dict(op="bias + gated_residual", **fold(r_one, r_two, 10 * rows * w.dim))}
    return res


def reference_cuda_record(env, job, K):
    """The reference's own kernels (src/kernels/ops.cu and blockscale.cu rebuilt for sm_100a) on this job's
    buffers with the same event method: block time, per op, and its quantiser."""
    from oracle import binding as orc
    if not orc.have_ref_ops():
        return {"unavailable": "oracle/_ref/libmx_ref_ops.so not built (needs the reference tree at build time)"}
    torch, w = env.torch, job.w
    runners = [ref_cuda_chain(w, b, env.sp) for b in job.sets]
    step = lambda i: runners[i % job.n_sets]()
    for i in range(3):
        step(i)
    env.barrier()
    windows = [env.event_ms(step, K) / K for _ in range(3)]
    ms = statistics.median(windows)
    # per op: events between its launches
    evs = []

    def mark():
        e = torch.cuda.Event(enable_timing=True)
        e.record(env.stream)
        evs.append(e)
    marked = [ref_cuda_chain(w, b, env.sp, mark) for b in job.sets]
    names = dropin_op_names(w)
    acc = [0.0] * len(names)
    n_pass = min(K, 10)
    for i in range(n_pass):
        evs.clear()
        marked[i % job.n_sets]()
        torch.cuda.synchronize()
        for j in range(len(names)):
            acc[j] += evs[j].elapsed_time(evs[j + 1])
    ops = op_rows(w, names, [t / n_pass * 1e3 for t in acc], job.rows, env.peak_gbs)
    by = w.bytes_per_row() * job.rows
    rec = {"what": "the reference's src/kernels/ops.cu rebuilt for sm_100a, same device buffers, same event timing",
           "us_per_block": round(ms * 1e3, 1), "gbs": round(by / (ms * 1e-3) / 1e9, 1),
           "frac_of_hbm_peak": round(by / (ms * 1e-3) / 1e9 / env.peak_gbs, 4), "launches_per_block": len(names), "per_op": ops}
    q = quant_rows(env, job, K, "reference-cuda")
    rec["quantize_blockscaled"] = q.get("quantize_blockscaled", q)
    return rec


def e2e_mxk(env, w, rows, row0, mods, chain, cos, sin, K, total_bytes):
    """End to end through the public host-buffer call: pinned host buffers in, results back in host
    memory, every step; wall clock between synchronizes, max over ranks."""
    from miroxen_b200.workloads import BlockBuffers
    args, mx, torch = env.args, env.mx, env.torch
    hb = BlockBuffers(w, rows, w.prefix_rows - row0, seed=7, mods=mods, cos=cos, sin=sin, host=True)
    hb.args.fused = 1 if chain == "fused" else 0
    pipe = mx.HostPipeline(args.e2e_chunk_rows, w.dim, w.F, w.H, w.D, w.rot, with_v=w.packed_qkv, act_mode=w.act_mode)
    up = down = 0
    for _ in range(2):
        up, down = pipe.run(hb.args)
    env.barrier()
    Ke = max(3, min(K, 10))
    t0 = time.perf_counter()
    for _ in range(Ke):
        pipe.run(hb.args)
    torch.cuda.synchronize()
    dt = env.max_over_ranks((time.perf_counter() - t0) / Ke)
    env.barrier()
    pipe.close()
    up_all, down_all = env.sum_over_ranks(float(up)), env.sum_over_ranks(float(down))
    return {"value": round(total_bytes / dt / 1e9, 2), "unit": UNIT, "ms_per_step": round(dt * 1e3, 3),
            "h2d_bytes_per_step": int(up_all), "d2h_bytes_per_step": int(down_all), "steps": Ke,
            "bytes_note": "summed over the ranks' copies",
            "api": f"mxk_dit_block_ops_host (pinned host buffers, {args.e2e_chunk_rows}-row chunks, 3 streams per GPU)",
            "host_placement": env.host_placement}


def e2e_reference(env, job, K):
    """The reference's kernels fed from pinned host buffers the plain way: upload every input, run
    its launchers, download every output, on one stream (its API has no host-buffer entry point)."""
    from miroxen_b200.workloads import BlockBuffers
    torch, w = env.torch, job.w
    hb = BlockBuffers(w, job.rows, job.prefix_rows, seed=7, mods=job.mods, cos=job.cos, sin=job.sin, host=True)
    db = job.sets[0]
    ins = ["x", "attn_o", "mlp_o", "cos", "sin"] + (["qkv"] if w.packed_qkv else ["q_in", "k_in"]) + (["act"] if w.act_mode == 0 else ["act2"])
    outs = ["h1", "q_out", "k_out", "h2", "act", "x"] + (["v_out"] if w.packed_qkv else [])
    run = ref_cuda_chain(w, db, env.sp)
    up = sum(getattr(hb, k).numel() * getattr(hb, k).element_size() for k in ins)
    down = sum(getattr(hb, k).numel() * getattr(hb, k).element_size() for k in outs)

    def step():
        for k in ins:
            getattr(db, k).copy_(getattr(hb, k), non_blocking=True)
        run()
        for k in outs:
            getattr(hb, k).copy_(getattr(db, k), non_blocking=True)
        torch.cuda.synchronize()
    for _ in range(2):
        step()
    Ke = max(3, min(K, 10))
    t0 = time.perf_counter()
    for _ in range(Ke):
        step()
    dt = (time.perf_counter() - t0) / Ke
    return {"value": round(w.bytes_per_row() * job.rows / dt / 1e9, 2), "unit": UNIT, "ms_per_step": round(dt * 1e3, 3),
            "h2d_bytes_per_step": int(up), "d2h_bytes_per_step": int(down), "steps": Ke,
            "api": "pinned host buffers -> cudaMemcpyAsync -> the reference's launchers -> cudaMemcpyAsync, one stream"}


def run_reference_cuda(args, W):
    """--impl reference: the reference's own implementation of this path is CUDA (src/kernels/ops.cu), so
    this arm runs those kernels, rebuilt unmodified for sm_100a (oracle/_ref), on one GPU over the whole
    workload; the CPU restatement is reported beside it as `cpu_baseline`."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import binding as orc
    if not orc.have_ref_ops():
        if args.impl == "reference-cuda":
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libmx_ref_ops.so not built (needs the reference tree at build time)"}), flush=True)
            return
        return run_reference_cpu(args, W, why="oracle/_ref/libmx_ref_ops.so (the reference's CUDA kernels) is absent: "
                                              "the CPU restatement was timed instead")
    env = Env(args)
    env.start(distributed=False)
    w = W[args.workload]
    K, Wm = max(args.steps, 1), max(args.warmup, 3)
    job = Job(env, w, w.rows, 0, chain="dropin", impl="reference-cuda")
    ms, stats, _, clocks = job.timed(K, Wm, args.repeats, clocks=True)
    by = w.bytes_per_row() * w.rows
    scaling = args.scaling or ("strong" if args.gpus > 1 else "weak")
    n_launch = len(dropin_op_names(w))
    line = {
        "impl": "reference", "metric": METRIC, "value": round(by / (ms * 1e-3) / 1e9, 1), "unit": UNIT, "n_gpus": args.gpus,
        "steps": K, "warmup": Wm, "ms_per_step": round(ms, 4), "us_per_block": round(ms * 1e3, 1), "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": job_config(w, "dropin", args.gpus, scaling, args.shard or "rows"),
        "reference_kind": "the reference's CUDA kernels (src/kernels/ops.cu, unmodified, rebuilt for sm_100a), one GPU, "
                          "the whole workload" + ("; the other ranks of this launch do no work" if args.gpus > 1 else ""),
        "timing": stats, "frac_of_hbm_peak": round(by / (ms * 1e-3) / 1e9 / env.peak_gbs, 4), "hbm_peak_gbs": env.peak_gbs,
        "hbm_peak_source": env.peak_src, "clocks": clocks, "gpu_launches": n_launch * K,
    }
    if not args.no_extras:
        rec = reference_cuda_record(env, job, min(K, 20))
        line["per_op"] = {"dropin": {"us_per_block": round(sum(o["us"] for o in rec["per_op"]), 1), "ops": rec["per_op"]}}
        line["next_rows"] = {"quantize_blockscaled": rec["quantize_blockscaled"]}
    if not args.no_e2e:
        line["e2e"] = e2e_reference(env, job, K)
    job.close()
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(w, args.cpu_rows or min(w.rows, 1088), 3)
    print(json.dumps(line), flush=True)


def interleaved_windows(env, K, arms, rounds=5):
    """µs per call of every arm: `rounds` rounds, each one window of K calls per arm in turn (CUDA events), median per
    arm.  The arms alternate so that a drift of the clocks under the power cap during these milliseconds-long
    GEMMs falls on all of them alike.  Returns ({arm: µs}, [min, max] of the first arm's windows)."""
    for _, fn in arms:
        for i in range(3):
            fn(i)
    env.barrier()
    win = {key: [] for key, _ in arms}
    for _ in range(rounds):
        for key, fn in arms:
            win[key].append(env.event_ms(fn, K) / K * 1e3)
    first = win[arms[0][0]]
    return {key: statistics.median(v) for key, v in win.items()}, [round(min(first), 1), round(max(first), 1)]


def linear_rows(env, w, rows, K):
    """The two projections that feed a gated_residual (attention out-projection: K = H*D; second MLP
    projection: K = F), as one tensor-core kernel with bias + gate + residual in its epilogue, against what it
    replaces: the library GEMM (torch.matmul on bf16 = cuBLAS, the reference's linear()) + add_bias_bf16 +
    gated_residual, and against the GEMM + this library's one-pass bias + residual."""
    torch, mx = env.torch, env.mx
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak_tf, src = (peaks["bf16_tflops"], "measured (burst)") if "bf16_tflops" in peaks else (1590.0, "fallback")
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    N = w.dim
    out = []
    for name, Kd in (("attention out-projection", w.inner), ("second MLP projection", w.F)):
        n_sets = max(2, math.ceil(3.2 * L2_BYTES / (rows * Kd * 2 + rows * N * 4)))
        A = [torch.randn((rows, Kd), generator=g, device="cuda").to(torch.bfloat16) for _ in range(n_sets)]
        W = (torch.randn((N, Kd), generator=g, device="cuda") / Kd ** 0.5).to(torch.bfloat16)
        bias = torch.randn(N, generator=g, device="cuda") * 0.1
        gate = mx.row_mod(torch.randn(N, generator=g, device="cuda") * 0.5)
        x = [torch.randn((rows, N), generator=g, device="cuda") for _ in range(n_sets)]
        y = [torch.empty((rows, N), dtype=torch.bfloat16, device="cuda") for _ in range(n_sets)]

        def fused(i):
            mx.ops.linear_gated_residual(A[i % n_sets], W, bias, rows, N, Kd, x[i % n_sets], gate, w.gate_tanh, env.stream)

        def gemm_only(i):
            torch.matmul(A[i % n_sets], W.T, out=y[i % n_sets])

        def three_calls(i):
            j = i % n_sets
            torch.matmul(A[j], W.T, out=y[j])
            mx.ops.add_bias_bf16(y[j], bias, rows, N, env.stream)
            mx.ops.gated_residual(x[j], y[j], rows, N, gate, w.gate_tanh, env.stream)

        def two_calls(i):
            j = i % n_sets
            torch.matmul(A[j], W.T, out=y[j])
            mx.ops.gated_residual_bias(x[j], y[j], bias, rows, N, gate, w.gate_tanh, env.stream)

        t, spread = interleaved_windows(env, K, (("fused", fused), ("cublas_gemm", gemm_only), ("cublas_bias_residual", three_calls),
                                                 ("cublas_fused_bias_residual", two_calls)))
        flops = 2.0 * rows * N * Kd
        out.append({"layer": name, "M": rows, "N": N, "K": Kd, "us": round(t["fused"], 1), "us_min_max": spread,
                    "tflops": round(flops / t["fused"] / 1e6, 1), "frac_of_bf16_peak": round(flops / t["fused"] / 1e6 / peak_tf, 3),
                    "us_cublas_gemm_alone": round(t["cublas_gemm"], 1),
                    "us_cublas_then_bias_then_residual": round(t["cublas_bias_residual"], 1),
                    "us_cublas_then_fused_bias_residual": round(t["cublas_fused_bias_residual"], 1),
                    "speedup_vs_reference_sequence": round(t["cublas_bias_residual"] / t["fused"], 3)})
        del A, W, x, y
    # the QKV projection with head norm + rope in its epilogue, against cuBLAS + add_bias_bf16 + qkv_norm_rope
    inner, Kd, Nq = w.inner, w.dim, 3 * w.inner
    n_sets = max(2, math.ceil(3.2 * L2_BYTES / (rows * Kd * 2 + rows * Nq * 2)))
    A = [torch.randn((rows, Kd), generator=g, device="cuda").to(torch.bfloat16) for _ in range(n_sets)]
    W = (torch.randn((Nq, Kd), generator=g, device="cuda") / Kd ** 0.5).to(torch.bfloat16)
    bias = torch.randn(Nq, generator=g, device="cuda") * 0.1
    nq = 1 + 0.05 * torch.randn(w.D, generator=g, device="cuda")
    nk = 1 + 0.05 * torch.randn(w.D, generator=g, device="cuda")
    ang = torch.rand((rows, max(w.rot // 2, 1)), generator=g, device="cuda") * 6.2 - 3.1
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    y = [torch.empty((rows, Nq), dtype=torch.bfloat16, device="cuda") for _ in range(n_sets)]
    outs = [[torch.empty((rows, w.H, w.D), dtype=torch.bfloat16, device="cuda") for _ in range(3)] for _ in range(n_sets)]
    norms, rots, modes = [nq, nk, None], [w.rot, w.rot, 0], [w.rope_mode, w.rope_mode, 0]
    fused_specs = [[mx.HeadSpec(None, 0, 0, norms[i], o[i], rots[i], modes[i]) for i in range(3)] for o in outs]
    sep_specs = [[mx.HeadSpec(y[j], Nq, i * inner, norms[i], outs[j][i], rots[i], modes[i]) for i in range(3)] for j in range(n_sets)]

    def q_fused(i):
        mx.ops.linear_qkv_norm_rope(A[i % n_sets], W, bias, rows, Kd, w.H, w.D, fused_specs[i % n_sets], w.eps, cos, sin, env.stream)

    def q_sep(i):
        j = i % n_sets
        torch.matmul(A[j], W.T, out=y[j])
        mx.ops.add_bias_bf16(y[j], bias, rows, Nq, env.stream)
        mx.qkv_norm_rope(sep_specs[j], rows, w.H, w.D, w.eps, cos, sin, env.stream)

    def q_gemm(i):
        torch.matmul(A[i % n_sets], W.T, out=y[i % n_sets])

    if w.D == 128 and w.H % 2 == 0:
        t, spread = interleaved_windows(env, K, (("fused", q_fused), ("cublas_gemm", q_gemm), ("separate", q_sep)))
        flops = 2.0 * rows * Nq * Kd
        out.append({"layer": "QKV projection + head norm + rope", "M": rows, "N": Nq, "K": Kd, "us": round(t["fused"], 1), "us_min_max": spread,
                    "tflops": round(flops / t["fused"] / 1e6, 1), "frac_of_bf16_peak": round(flops / t["fused"] / 1e6 / peak_tf, 3),
                    "us_cublas_gemm_alone": round(t["cublas_gemm"], 1),
                    "us_cublas_then_bias_then_qkv_norm_rope": round(t["separate"], 1),
                    "speedup_vs_reference_sequence": round(t["separate"] / t["fused"], 3)})
    del A, W, y, outs
    # the first MLP projection with its activation in the epilogue, against cuBLAS + add_bias_bf16 + the activation
    Kd, F = w.dim, w.F
    swiglu = w.act_mode == 1
    Nw = 2 * F if swiglu else F
    n_sets = max(2, math.ceil(3.2 * L2_BYTES / (rows * Kd * 2 + rows * Nw * 2)))
    A = [torch.randn((rows, Kd), generator=g, device="cuda").to(torch.bfloat16) for _ in range(n_sets)]
    W = (torch.randn((Nw, Kd), generator=g, device="cuda") / Kd ** 0.5).to(torch.bfloat16)
    bias = torch.randn(Nw, generator=g, device="cuda") * 0.1
    y = [torch.empty((rows, Nw), dtype=torch.bfloat16, device="cuda") for _ in range(n_sets)]
    mid = [torch.empty((rows, F), dtype=torch.bfloat16, device="cuda") for _ in range(n_sets)]

    def f_fused(i):
        j = i % n_sets
        if swiglu:
            mx.ops.linear_silu_mul(A[j], W, bias, rows, F, Kd, mid[j], env.stream)
        else:
            mx.ops.linear_act(A[j], W, bias, rows, F, Kd, w.act_mode, mid[j], env.stream)

    def f_sep(i):
        j = i % n_sets
        torch.matmul(A[j], W.T, out=y[j])
        mx.ops.add_bias_bf16(y[j], bias, rows, Nw, env.stream)
        if swiglu:
            mx.ops.silu_mul(y[j], rows, F, mid[j], env.stream)
        else:
            mx.ops.gelu_tanh_inplace(y[j], rows * F, env.stream)

    def f_gemm(i):
        torch.matmul(A[i % n_sets], W.T, out=y[i % n_sets])

    t, spread = interleaved_windows(env, K, (("fused", f_fused), ("cublas_gemm", f_gemm), ("separate", f_sep)))
    flops = 2.0 * rows * Nw * Kd
    out.append({"layer": "first MLP projection + " + ("silu_mul" if swiglu else "gelu_tanh"), "M": rows, "N": Nw, "K": Kd,
                "us": round(t["fused"], 1), "us_min_max": spread, "tflops": round(flops / t["fused"] / 1e6, 1),
                "frac_of_bf16_peak": round(flops / t["fused"] / 1e6 / peak_tf, 3), "us_cublas_gemm_alone": round(t["cublas_gemm"], 1),
                "us_cublas_then_bias_then_activation": round(t["separate"], 1),
                "speedup_vs_reference_sequence": round(t["separate"] / t["fused"], 3)})
    del A, W, y, mid
    return {"what": "linear() + add_bias_bf16 + gated_residual (or head_norm_rope, or the MLP activation) as one tcgen05 kernel against cuBLAS + the separate ops",
            "bf16_peak_tflops": peak_tf, "peak_source": src, "layers": out}


def exchange_rows(env, w, K):
    """Head exchange of the sequence-parallel attention path on this job's ranks: every rank norm+ropes the q / k / v
    heads of its row shard and stores each head group into its owner's [S, H/G, D] buffer (peer stores over NVLink),
    then gathers all heads of its rows back from everybody's buffer (peer loads).  Times are max over ranks."""
    from miroxen_b200.head_exchange import ExchangePlan, HeadExchange
    torch, mx = env.torch, env.mx
    G, rank = env.world, env.rank
    plan = ExchangePlan(w.rows, w.H, w.D, G)
    sh = plan.rows(rank)
    g = torch.Generator(device="cuda")
    g.manual_seed(100 + rank)
    inner = w.inner
    n_sets = max(2, math.ceil(3.2 * L2_BYTES / (sh.rows * 3 * inner * 2)))
    qkv = [torch.randn((sh.rows, 3 * inner), generator=g, device="cuda").to(torch.bfloat16) for _ in range(n_sets)]
    nq = 1 + 0.05 * torch.randn(w.D, generator=g, device="cuda")
    nk = 1 + 0.05 * torch.randn(w.D, generator=g, device="cuda")
    ang = torch.rand((sh.rows, max(w.rot // 2, 1)), generator=g, device="cuda") * 6.2 - 3.1
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    out = torch.empty((sh.rows, inner), dtype=torch.bfloat16, device="cuda")
    ex = HeadExchange(plan, rank)
    try:
        def specs(t):
            return [mx.HeadSpec(t, 3 * inner, 0, nq, None, w.rot, w.rope_mode), mx.HeadSpec(t, 3 * inner, inner, nk, None, w.rot, w.rope_mode),
                    mx.HeadSpec(t, 3 * inner, 2 * inner, None, None, 0, 0)]
        sp = [specs(t) for t in qkv]
        scatter = lambda i: ex.scatter_qkv(sp[i % n_sets], sh.rows, w.eps, cos, sin, stream=env.stream)
        gather = lambda i: ex.gather_heads(out, buffer=0, stream=env.stream)
        res = {}
        for name, fn in (("scatter_qkv", scatter), ("gather_heads", gather)):
            for i in range(3):
                fn(i)
            env.barrier()
            reps = []
            for _ in range(5):
                ms = env.event_ms(fn, K) / K
                env.barrier()
                reps.append(env.max_over_ranks(ms))
            res[name] = statistics.median(reps) * 1e3
        # the local (single-GPU) form of the same work, for the cost of going over NVLink
        dense = [torch.empty((sh.rows, w.H, w.D), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
        dsp = [[mx.HeadSpec(t.in_, t.in_stride, t.col0, t.norm_w, o, t.rot, t.mode) for t, o in zip(s_, dense)] for s_ in sp]
        local = lambda i: mx.qkv_norm_rope(dsp[i % n_sets], sh.rows, w.H, w.D, w.eps, cos, sin, env.stream)
        for i in range(3):
            local(i)
        env.barrier()
        res["local_qkv_norm_rope"] = env.max_over_ranks(env.event_ms(local, K) / K) * 1e3
        env.barrier()
    finally:
        ex.barrier()
        ex.close()
    send = plan.send_bytes(rank, 3)
    back = sh.rows * inner * 2 * (G - 1) // G
    link = 770.0  # GB/s per direction per GPU, the measured peer-copy rate on this pool (900 nominal)
    rec = {"workload": w.name, "n_gpus": G, "rows_per_gpu": sh.rows, "heads_per_group": plan.heads_per_group,
           "scatter_qkv": {"us": round(res["scatter_qkv"], 1), "nvlink_bytes_per_rank": send,
                           "formula": "3 * rows * H * D * 2 * (G - 1) / G",
                           "nvlink_gbs_per_rank": round(send / res["scatter_qkv"] / 1e3, 1) if G > 1 else 0.0,
                           "frac_of_peer_copy_rate": round(send / res["scatter_qkv"] / 1e3 / link, 3) if G > 1 else None,
                           "us_local_qkv_norm_rope": round(res["local_qkv_norm_rope"], 1),
                           "hbm_bytes_per_rank": sh.rows * (3 * inner * 2 * 2 + 2 * (w.rot // 2) * 4)},
           "gather_heads": {"us": round(res["gather_heads"], 1), "nvlink_bytes_per_rank": back,
                            "nvlink_gbs_per_rank": round(back / res["gather_heads"] / 1e3, 1) if G > 1 else 0.0,
                            "frac_of_peer_copy_rate": round(back / res["gather_heads"] / 1e3 / link, 3) if G > 1 else None},
           "link_rate_gbs": link,
           "note": "one process per GPU, CUDA IPC peer buffers, plain peer stores / loads from this library's kernels; the only "
                   "collective is the barrier between the two phases (untimed)"}
    return rec


def strong_record(env, w, K, splits):
    """Strong scaling of one workload inside this run: the whole workload on one GPU (every rank runs it,
    max over ranks), then each split of its rows over the ranks.  Times are ms per block, max over ranks."""
    world, rank = env.world, env.rank
    rec = {"workload": w.name, "rows": w.rows, "n_gpus": world, "chains": {}}
    whole = Job(env, w, w.rows, 0)
    base = {}
    for chain in ("dropin", "fused"):
        whole.set_chain(chain)
        base[chain], _, _, _ = whole.timed(K, 3, repeats=3)
    mods = whole.mods
    whole.close()
    for by in splits:
        sh = shard_of(w, world, rank, by)
        job = Job(env, w, sh.rows, sh.row0, mods=mods)
        rows_max = int(env.max_over_ranks(float(sh.rows)))
        entry = {"rows_per_gpu_max": rows_max, "ceiling": round(w.rows / rows_max, 2)}
        for chain in ("dropin", "fused"):
            job.set_chain(chain)
            ms, _, _, _ = job.timed(K, 3, repeats=5)
            entry[chain] = {"ms_per_block": round(ms, 4), "ms_per_block_1gpu": round(base[chain], 4),
                            "speedup": round(base[chain] / ms, 2),
                            "gbs": round(w.bytes_per_row() * w.rows / (ms * 1e-3) / 1e9, 1)}
        rec["chains"][by] = entry
        job.close()
    rec["note"] = ("speedup = this run's 1-GPU ms_per_block / the sharded ms_per_block; `ceiling` = rows / the largest shard "
                   "(a by-frame split of 21 frames over 8 GPUs is 3,3,3,3,3,2,2,2 frames: at most 7.11x)")
    return rec


def main():
    args = parse()
    from miroxen_b200.workloads import WORKLOADS as W
    if args.workload not in W:
        raise SystemExit(f"unknown workload {args.workload}; one of {sorted(W)}")
    if args.impl == "reference-cpu":
        return run_reference_cpu(args, W)
    if args.impl in ("reference", "reference-cuda"):
        return run_reference_cuda(args, W)

    env = Env(args)
    env.start(distributed=True)
    mx, torch = env.mx, env.torch
    world, rank = env.world, env.rank
    w = W[args.workload]
    n_gpus = world
    scaling = args.scaling or ("strong" if n_gpus > 1 else "weak")
    shard_by = args.shard or "rows"
    K, Wm = max(args.steps, 1), max(args.warmup, 3)

    # rows of this rank
    if scaling == "strong" and n_gpus > 1:
        sh = shard_of(w, n_gpus, rank, shard_by)
        rows, row0 = sh.rows, sh.row0
    else:
        rows, row0 = w.rows, 0
    if args.rows > 0:
        if not (args.ops_only or args.quant_only or args.linear_only):
            raise SystemExit("--rows goes with --ops-only / --quant-only / --linear-only: the bench line is defined on the whole workload")
        rows = min(rows, args.rows)
    total_rows = w.rows * (n_gpus if scaling == "weak" else 1)
    job = Job(env, w, rows, row0, chain=args.chain)
    if args.graph:
        job.capture_graphs()

    if args.ops_only:
        if rank == 0:
            print(json.dumps({"impl": args.impl, "workload": w.name, "rows": rows, "steps": K, "tune": args.tune,
                              "per_op_isolated": job.per_op_isolated(K)}), flush=True)
        return
    if args.exchange_only:
        job.close()
        wl = W["h3video"] if args.workload == "qwen1024" else w   # the reference's sequence-parallel path is the video model's
        rec = exchange_rows(env, wl, K)
        if rank == 0:
            print(json.dumps({"impl": args.impl, "steps": K, "head_exchange": rec}), flush=True)
        if env.distributed:
            env.dist.destroy_process_group()
        return
    if args.linear_only:
        job.close()
        if rank == 0:
            with ClockSampler(env.local) as sampler:
                rec = linear_rows(env, w, rows, K)
            print(json.dumps({"impl": args.impl, "workload": w.name, "rows": rows, "steps": K, "tune": args.tune, "linear_epilogue": rec,
                              "clocks": sampler.summary()}), flush=True)
        return
    if args.quant_only:
        if rank == 0:
            print(json.dumps({"impl": args.impl, "workload": w.name, "steps": K, "next_rows": quant_rows(env, job, K, "mxk")}), flush=True)
        return

    ms, stats, launches, clocks = job.timed(K, Wm, args.repeats, clocks=True)
    job_bytes = w.bytes_per_row() * total_rows
    value = job_bytes / (ms * 1e-3) / 1e9
    rows_max = int(env.max_over_ranks(float(rows)))

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": n_gpus, "steps": K, "warmup": Wm,
        "ms_per_step": round(ms, 4), "us_per_block": round(ms * 1e3, 1), "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": job_config(w, args.chain, n_gpus, scaling, shard_by),
        "layout": {"rows_per_gpu": rows_max, "rows_total": total_rows,
                   "launch": "cuda graph replay" if args.graph else "stream launches (programmatic dependent launch)",
                   "buffer_sets": job.n_sets, "set_mb": round(job.set_bytes() / 1e6)},
        "timing": dict(stats, ms_x_sm_mhz=(round(ms * clocks["sm_mhz"], 1) if clocks and clocks.get("sm_mhz") else None),
                       method="median over `repeats` windows of exactly `steps` steps, CUDA events on the launching "
                              "stream, barrier + synchronize around every window, max over ranks per window"),
        "frac_of_hbm_peak": round(value / n_gpus / env.peak_gbs, 4), "hbm_peak_gbs": env.peak_gbs, "hbm_peak_source": env.peak_src,
        "clocks": clocks, "gpu_launches": int(launches),
    }
    if scaling == "strong" and n_gpus > 1:
        line["timing"]["speedup_ceiling"] = round(w.rows / rows_max, 2)

    if not args.no_extras:
        chunked = w.chunk_rows > 0 and w.chunk_rows < rows
        per_chain = {"dropin": job.per_op_marginal(K, 0), "fused": job.per_op_marginal(K, 1)}
        line["per_op"] = per_chain
        line["per_op_events"] = {"dropin": job.per_op(K, 0), "fused": job.per_op(K, 1)}
        line["per_op_isolated"] = job.per_op_isolated(K)
        line["per_op_note"] = ("per_op: each op's cost inside the chain, by timing the chain's prefixes and subtracting (the "
                               "launches overlap as in the timed region and the figures add up to the block"
                               + (", issued as one chunk here" if chunked else "") + "); per_op_events: events "
                               "recorded between the launches, which serialises them (each interval also holds one whole launch "
                               "latency and the previous op's write-backs); per_op_isolated: the op launched back to back over "
                               "rotating buffer sets")
        ops = per_chain[args.chain]["ops"]
        top = max(ops, key=lambda o: o["us"])
        line["roofline"] = {"bound": "hbm", "kernel": top["op"], "achieved": top["gbs"], "peak": env.peak_gbs, "unit": "GB/s",
                            "frac": round(top["gbs"] / env.peak_gbs, 4), "traffic": None, "peak_source": env.peak_src}
        tr = ROOT / "profiles" / "dram_traffic.json"
        if tr.exists():
            try:
                doc = json.loads(tr.read_text())
                t = doc.get(w.name, {}).get(top["op"])
                if t:
                    line["roofline"]["traffic"] = int(t["bytes_per_row"] * rows)
                    line["roofline"]["traffic_note"] = ("from the ncu capture named in profiles/dram_traffic.json, scaled by rows; "
                                                        "a lower bound for writes (lines still in L2 when the launch ends are not counted)")
            except Exception:
                pass
        # the other chain, clean timing
        other = "fused" if args.chain == "dropin" else "dropin"
        job.set_chain(other)
        ms2, st2, l2, _ = job.timed(K, 3, repeats=5)
        line["other_chain"] = {"chain": other, "ms_per_step": round(ms2, 4), "value": round(job_bytes / (ms2 * 1e-3) / 1e9, 1),
                               "gpu_launches": int(l2), "ms_per_step_min": st2["ms_per_step_min"], "ms_per_step_max": st2["ms_per_step_max"]}
        job.set_chain(args.chain)

    if not args.no_extras and n_gpus == 1:
        line["next_rows"] = quant_rows(env, job, K, "mxk")
        line["reference_cuda"] = reference_cuda_record(env, job, min(K, 20))
        if "us_per_block" in line["reference_cuda"]:
            line["reference_cuda"]["speedup_of_this_library"] = round(line["reference_cuda"]["us_per_block"] / (ms * 1e3), 2)

    mods, cos, sin = job.mods, job.cos, job.sin
    job.close()

    if not args.no_extras and n_gpus == 1 and w.rows >= 8 * 64:
        # the same chain at the row count one rank of an 8-GPU job owns: what strong scaling is limited by
        sh8 = shard_of(w, 8, 0, shard_by)
        small = Job(env, w, sh8.rows, 0, mods=mods, chain=args.chain)
        ms8, _, _, _ = small.timed(K, 3, repeats=5)
        line["shard_size"] = {"rows": sh8.rows, "of": "one rank of an 8-way row split", "us_per_block": round(ms8 * 1e3, 1),
                              "speedup_if_all_ranks_match": round(ms / ms8, 2),
                              "per_op": {"dropin": small.per_op_marginal(K, 0), "fused": small.per_op_marginal(K, 1)},
                              "per_op_isolated": small.per_op_isolated(K)}
        small.set_chain("fused")
        msf, _, _, _ = small.timed(K, 3, repeats=5)
        line["shard_size"]["us_per_block_fused"] = round(msf * 1e3, 1)
        small.close()

    if not args.no_extras and n_gpus > 1 and scaling == "strong":
        # BASELINE.json's video shape (sharded by frame, the reference's split, and by equal row ranges) and the 2048^2 image
        line["video_strong"] = strong_record(env, W["h3video"], min(K, 20), ("frames", "rows"))
        line["strong_records"] = [strong_record(env, W["qwen2048"], min(K, 20), ("rows",))]
        # replicas of the main workload, for the per-GPU rate next to the sharded one
        rep = Job(env, w, w.rows, 0, mods=mods, chain=args.chain)
        msr, _, _, _ = rep.timed(K, 3, repeats=3)
        line["replicas"] = {"ms_per_step": round(msr, 4), "value": round(w.bytes_per_row() * w.rows * n_gpus / (msr * 1e-3) / 1e9, 1),
                            "speedup": round(msr / ms, 2)}
        rep.close()

    if not args.no_extras and n_gpus == 1:
        # the linear layers either side of the chain, with the chain's op in their epilogue (after job.close(): they need the memory)
        line["next_rows"]["linear_epilogue"] = linear_rows(env, w, rows, min(K, 10))

    if not args.no_e2e:
        line["e2e"] = e2e_mxk(env, w, rows, row0, mods, args.chain, cos, sin, K, job_bytes)

    if rank == 0 and n_gpus == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(w, args.cpu_rows or min(w.rows, 2176), 3)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if env.distributed:
        env.dist.destroy_process_group()


if __name__ == "__main__":
    main()
