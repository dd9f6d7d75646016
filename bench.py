#!/usr/bin/env python
"""Benchmark of the fused expert gather/scatter path: routed tokens/s for one full step
(gather forward, scatter forward, both backwards) plus roofline and CPU-baseline figures.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl b200|reference]

One JSON line on stdout (rank 0).  The default workload is the same on every box and for every N: the multi-GPU
configuration (global batch 512) strong-scaled over the ranks, which at N=1 is the largest single-GPU configuration.
For N > 1 launch with torchrun; the batch is sharded over the ranks and the two weight gradients are all-reduced (NCCL)
inside the timed step.  At N=1 the line also carries a `configs` array with the five benchmark configurations.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from expertscattergather_b200 import workloads as wl  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
METRIC = "gather+scatter fwd+bwd routed tokens/s"
DEFAULT_WORKLOAD = "cfg4"
ALL_CONFIGS = ("cfg0", "cfg1-sweep", "cfg2", "cfg3", "cfg4")
E2E_MICRO_BATCH = 64     # batch elements per micro-batch of the end-to-end leg (a pass of at most this size is one copy)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def ncu_traffic_table():
    """DRAM bytes per routed slot of each operator's kernels, from the ncu captures summarised under profiles/
    (profiles/ncu_traffic.json: per entry the capture's command, kernel, DRAM bytes per launch and slots per launch)."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    table = {}
    if os.path.exists(path):
        with open(path) as f:
            for ent in json.load(f)["entries"]:
                table[(ent["op"], ent["config"])] = ent["dram_bytes_per_launch"] / ent["slots_per_launch"]
    return table


def resolve_workload(name):
    """Names -> list of Workload passes that make up one step."""
    if name is None:
        name = DEFAULT_WORKLOAD
    if name == "cfg1-sweep":
        return name, [wl.WORKLOADS[k] for k in wl.CFG1_SWEEP]
    if name in wl.WORKLOADS:
        return name, [wl.WORKLOADS[name]]
    raise SystemExit(f"unknown workload {name!r}; choose from cfg1-sweep, " + ", ".join(wl.WORKLOADS))


def describe_config(name, passes, world):
    """The workload description both arms print (identical for the same workload and N)."""
    return {"workload": name,
            "passes": [f"{w.name}: B={w.B} T={w.T} E={w.E} K={w.K} I={w.I} J={w.J} {str(w.dtype).replace('torch.', '')} "
                       f"Ind={w.index}" for w in passes],
            "routed_tokens_per_step": sum(w.routed for w in passes),
            "parallelism": f"dp{world} (batch sharded over the ranks, dW_g and dW_s all-reduced)"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t_from=None, t_to=None):
        """Summary of the samples taken in [t_from, t_to] (perf_counter times); all samples when none fall inside."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [ln for t, ln in self.lines if t_from is None or (t_from - 0.02 <= t <= t_to + 0.02)]
        if not rows:
            rows = [ln for _, ln in self.lines]
        sm, mx, reasons = [], [], set()
        for ln in rows:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def quantiles(xs):
    xs = sorted(xs)

    def q(p):
        if len(xs) == 1:
            return xs[0]
        pos = p * (len(xs) - 1)
        lo = int(pos)
        hi = min(lo + 1, len(xs) - 1)
        return xs[lo] + (xs[hi] - xs[lo]) * (pos - lo)
    return {"median": q(0.5), "p20": q(0.2), "p80": q(0.8)}


# -------------------------------------------------------------------------------------------------------------
# CPU arm: the checker's torch restatement of the reference path, timed on the host cores
# -------------------------------------------------------------------------------------------------------------
def cpu_baseline(passes, budget_s=20.0, reps=3, full_size=False, keep_outputs=False):
    """Times oracle.torch_step on the host for a bounded sample of each pass; returns routed tokens/s.
    With keep_outputs the sample's inputs and the checker's outputs come back too (the parity check uses them)."""
    from oracle import egs_oracle as orc   # the one place the benchmark executes the checker
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    tokens = 0.0
    seconds = 0.0
    samples, kept = [], []
    for w in passes:
        # slice the batch so that one repetition costs about budget/(reps+1)/len(passes) seconds
        flops = 12 * w.E * w.K * w.I * w.J
        est_per_b = flops / 2e10 + w.T * w.I * 4e-8
        b = w.B if full_size else max(1, min(w.B, int(budget_s / (reps + 1) / len(passes) / max(est_per_b, 1e-6))))
        ins = wl.make_inputs(w, B=b)
        out = orc.torch_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            orc.torch_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
            ts.append(time.perf_counter() - t0)
        t = statistics.median(ts)
        tokens += b * w.E * w.K
        seconds += t
        samples.append(f"{w.name}: B={b} of {w.B}, {t * 1e3:.1f} ms")
        if keep_outputs:
            kept.append((w, ins, out))
    res = {"value": tokens / seconds, "unit": "tokens/s", "cores": cores, "kind": "port",
           "sample": "; ".join(samples) + " (median of %d; batch slices scale linearly in B)" % reps}
    return res, seconds, kept


def run_reference_arm(args, name, passes):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    base = None
    t_all = time.perf_counter()
    for i in range(args.warmup + args.steps):
        base, secs, _ = cpu_baseline(passes, budget_s=6.0, reps=1)
        if i >= args.warmup:
            vals.append((base["value"], secs))
    v = statistics.median(x[0] for x in vals)
    base["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": statistics.median(x[1] for x in vals) * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": str(passes[0].dtype).replace("torch.", ""), "data": "synthetic",
            "config": describe_config(name, passes, args.gpus),
            "run": {"device": "host CPU", "note": "torch restatement of egs/baselines.py (gather + einsum + scatter_add_, "
                    "gradients by autograd); each step is a bounded batch slice of the workload"},
            "cpu_baseline": base,
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": time.perf_counter() - t_all}
    print(json.dumps(line), flush=True)


# -------------------------------------------------------------------------------------------------------------
# GPU arm
# -------------------------------------------------------------------------------------------------------------
def op_work(w, B, U, op, dense_write=True):
    """Algorithmic (flops, bytes) of one operator launch group.  dense_write=False: the scatter adds into a given,
    already filled output, so instead of the dense [B,T,I] write only the U touched rows are read and written (the fill
    is accounted for in its own `fill_out` row)."""
    s = torch.empty((), dtype=w.dtype).element_size()
    N = B * w.E * w.K
    WB = w.E * w.I * w.J * s
    fl = 2 * N * w.I * w.J
    if op in ("gather_fwd", "scatter_bwd_dY"):
        return fl, U * w.I * s + WB + 8 * N + N * w.J * s
    out_bytes = B * w.T * w.I * s if dense_write else 2 * U * w.I * s
    if op in ("scatter_fwd", "gather_bwd_dX"):
        return fl, N * w.J * s + WB + 8 * N + out_bytes
    if op in ("pair_fwd", "pair_bwd"):
        # fused G -> S: token rows read once, both weights, the middle tensor written once, the output written once
        return 2 * fl, U * w.I * s + 2 * WB + 8 * N + N * w.J * s + out_bytes
    if op == "fill_out":
        return 0, B * w.T * w.I * s
    return fl, U * w.I * s + N * w.J * s + 8 * N + WB      # dW_g, dW_s


def tensor_peak(dtype, peaks, dev, cache={}):
    """Tensor-core peak in TFLOP/s for the roofline: the bf16 figure of MEASURED_PEAKS.json for 16-bit tensors; for float32
    a TF32 torch.matmul measured here the same way (8192^3, best of 12), since that file has no TF32 figure."""
    if dtype != torch.float32:
        return peaks["bf16_tflops"]
    if "tf32" not in cache:
        a = torch.randn(8192, 8192, device=dev); b = torch.randn(8192, 8192, device=dev)
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        best = float("inf")
        for _ in range(12):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); torch.matmul(a, b); e1.record(); e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        torch.backends.cuda.matmul.allow_tf32 = prev
        cache["tf32"] = 2 * 8192 ** 3 / (best * 1e-3) / 1e12
    return cache["tf32"]


class StepRunner:
    """Inputs of one workload resident on this rank's GPU and the step over them (graph-replayed where possible)."""

    def __init__(self, passes, rank, world, dev, use_graph):
        from expertscattergather_b200 import distributed as egd
        self.passes, self.rank, self.world, self.dev = passes, rank, world, dev
        self.host, self.devs, self.shard_B = [], [], []
        for w in passes:
            lo, hi = egd.shard_bounds(w.B, rank, world)
            h = wl.make_inputs(w, B=hi - lo, b0=lo)
            h = {k: v.pin_memory() for k, v in h.items()}
            self.host.append(h)
            self.devs.append({k: v.to(dev, non_blocking=True) for k, v in h.items()})
            self.shard_B.append(hi - lo)
        torch.cuda.synchronize()
        self.tokens_per_step = sum(w.routed for w in passes)            # whole job, all ranks
        footprint = sum(sum(v.numel() * v.element_size() for v in d.values()) for d in self.devs)
        self.flush_buf = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev) if footprint < 4 * L2_BYTES else None
        self.graph = None
        self.graph_outs = None
        self.use_graph = use_graph
        self.all_reduce = True

    def one_step(self):
        from expertscattergather_b200 import distributed as egd
        from expertscattergather_b200.step import train_step
        outs = []
        for d in self.devs:
            if self.world > 1 and self.all_reduce:
                outs.append(egd.dp_train_step(d["X"], d["Wg"], d["Ws"], d["Ind"], d["G"]))
            elif self.world > 1:
                # same operator order as the data-parallel step, reductions left out (phase timing)
                outs.append(train_step(d["X"], d["Wg"], d["Ws"], d["Ind"], d["G"], on_weight_grad=lambda n, t: None))
            else:
                outs.append(train_step(d["X"], d["Wg"], d["Ws"], d["Ind"], d["G"]))
        return outs

    def capture(self):
        """Captures the step in a CUDA graph (after two eager steps on a side stream); plain launches if refused."""
        self.graph = None
        if not self.use_graph:
            return
        try:
            side = torch.cuda.Stream(self.dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self.one_step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.graph_outs = self.one_step()      # keeps the captured outputs alive
            self.graph = g
        except Exception as exc:          # capture refused: time plain launches instead
            sys.stderr.write(f"CUDA graph capture failed ({type(exc).__name__}: {exc}); timing plain launches\n")
            self.graph = None
            torch.cuda.synchronize()

    def run(self):
        if self.graph is not None:
            self.graph.replay()
            return self.graph_outs
        return self.one_step()

    def barrier(self):
        if self.world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def timed(self, steps, warmup):
        """warmup untimed steps, then `steps` steps between barrier + synchronize on both sides; one CUDA event pair per
        step.  Returns (per-step ms of this rank, wall-clock interval of the timed region)."""
        from expertscattergather_b200 import ops
        fills = ops.fill_stream(self.dev)
        for _ in range(warmup):
            if self.flush_buf is not None:
                self.flush_buf.zero_()
            self.run()
        self.barrier()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        self.barrier()
        t0 = time.perf_counter()
        for i in range(steps):
            if self.flush_buf is not None:
                self.flush_buf.zero_()
            starts[i].record()
            if self.graph is None:
                fills.wait_event(starts[i])      # plain launches: the zero fills of step i stay inside its interval
            self.run()
            stops[i].record()
        self.barrier()
        t1 = time.perf_counter()
        return [a.elapsed_time(b) for a, b in zip(starts, stops)], (t0, t1)


def time_call(fn, reps, flush_buf):
    """Device time of one operator call (its kernels only): the call is captured into a CUDA graph so that host launch
    overhead stays out of the events; L2 is flushed between repetitions.  Median in ms."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    g = None
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            keep = fn()   # noqa: F841
    except Exception:
        g = None
        torch.cuda.synchronize()
    ts = []
    for _ in range(reps + 2):
        if flush_buf is not None:
            flush_buf.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        if g is not None:
            g.replay()
        else:
            fn()
        b.record(); b.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts[2:])


def operator_breakdown(runner, peaks, reps):
    """Per operator of every pass: device time, algorithmic work and the fraction of its own roofline.  Scatter
    operators are timed adding into a given output, their zero fill is a row of its own."""
    from expertscattergather_b200 import ops
    from expertscattergather_b200.step import takes_fused_pairs
    rows = []
    strict = ops.get_precision() == "strict"
    for w, d, h, b in zip(runner.passes, runner.devs, runner.host, runner.shard_B):
        U = wl.algorithmic_work(w, Ind=h["Ind"], B=b)["U"]
        tc = tensor_peak(w.dtype, peaks, runner.dev)
        Y = ops.gather_gemm(d["X"], d["Wg"], d["Ind"])
        dY = ops.gather_gemm(d["G"], d["Ws"], d["Ind"], w_layout="nc")
        out_buf = torch.zeros((b, w.T, w.I), device=runner.dev, dtype=w.dtype)
        if takes_fused_pairs(d["X"], d["Wg"], d["Ind"]):
            calls = {
                "pair_fwd": lambda: ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], d["Ind"], out=out_buf),
                "scatter_bwd_dW": lambda: ops.dweight(d["G"], Y, d["Ind"], out_layout="direct_rows"),
                "pair_bwd": lambda: ops.gather_scatter_pair(d["G"], d["Ws"], d["Wg"], d["Ind"], w_layout="nc", out=out_buf),
                "gather_bwd_dW": lambda: ops.dweight(d["X"], dY, d["Ind"]),
            }
        else:
            calls = {
                "gather_fwd": lambda: ops.gather_gemm(d["X"], d["Wg"], d["Ind"]),
                "scatter_fwd": lambda: ops.gemm_scatter(Y, d["Ws"], d["Ind"], w.T, out=out_buf),
                "scatter_bwd_dY": lambda: ops.gather_gemm(d["G"], d["Ws"], d["Ind"], w_layout="nc"),
                "scatter_bwd_dW": lambda: ops.dweight(d["G"], Y, d["Ind"], out_layout="direct_rows"),
                "gather_bwd_dX": lambda: ops.gemm_scatter(dY, d["Wg"], d["Ind"], w.T, w_layout="nc", out=out_buf),
                "gather_bwd_dW": lambda: ops.dweight(d["X"], dY, d["Ind"]),
            }
        calls["fill_out"] = lambda: ops.fill_zero(out_buf)
        for op, fn in calls.items():
            ms = time_call(fn, reps, runner.flush_buf)
            fl, by = op_work(w, b, U, op, dense_write=False)
            t_hbm = by / (peaks["hbm_gbs"] * 1e9)
            t_tc = fl * (3 if (w.dtype == torch.float32 and strict) else 1) / (tc * 1e12)
            bound = "hbm" if t_hbm >= t_tc else "tensor"
            rows.append({"pass": w.name, "op": op, "ms": ms, "flops": fl, "bytes": by, "bound": bound,
                         "achieved": (by / (ms * 1e-3) / 1e9) if bound == "hbm" else (fl / (ms * 1e-3) / 1e12),
                         "unit": "GB/s" if bound == "hbm" else "TFLOP/s",
                         "frac_of_roofline": max(t_hbm, t_tc) / (ms * 1e-3)})
        del Y, dY, out_buf
    return rows


def step_floor_ms(runner, peaks):
    alg = [wl.algorithmic_work(w, Ind=h["Ind"], B=b) for w, h, b in zip(runner.passes, runner.host, runner.shard_B)]
    return sum(max(a["bytes"] / (peaks["hbm_gbs"] * 1e9),
                   a["flops"] / (tensor_peak(w.dtype, peaks, runner.dev) * 1e12))
               for a, w in zip(alg, runner.passes)) * 1e3


def parity_check(rank, world, dev):
    """Data-parallel parity before timing: a small slice of the default workload (two batch elements per rank) goes
    through the sharded step with its all-reduces; every rank's reduced dW_g / dW_s must be bitwise equal, and rank 0
    compares all six outputs of its shard and the reduced weight gradients with the CPU checker run unsharded."""
    from expertscattergather_b200 import distributed as egd, ops
    w = wl.WORKLOADS[DEFAULT_WORKLOAD].with_batch(2 * world)
    lo, hi = egd.shard_bounds(w.B, rank, world)
    ins = wl.make_inputs(w, B=hi - lo, b0=lo)
    d = {k: v.to(dev) for k, v in ins.items()}
    if world > 1:
        out = egd.dp_train_step(d["X"], d["Wg"], d["Ws"], d["Ind"], d["G"])
    else:
        from expertscattergather_b200.step import train_step
        out = train_step(d["X"], d["Wg"], d["Ws"], d["Ind"], d["G"])
    torch.cuda.synchronize()
    ops.check_status()
    res = {"case": f"{w.name} slice, B={w.B} over {world} rank(s)"}
    if world > 1:
        same = True
        for k in ("dWg", "dWs"):
            mine = out[k].contiguous().view(torch.int16).to(torch.int32)
            lo_t, hi_t = mine.clone(), mine.clone()
            torch.distributed.all_reduce(lo_t, op=torch.distributed.ReduceOp.MIN)
            torch.distributed.all_reduce(hi_t, op=torch.distributed.ReduceOp.MAX)
            same = same and bool(torch.equal(lo_t, hi_t))
        res["dW_bitwise_equal_across_ranks"] = same
    if rank == 0:
        from oracle import egs_oracle as orc      # checker only (the CPU leg of the benchmark)
        full = wl.make_inputs(w)
        ref = orc.torch_step(full["X"], full["Wg"], full["Ws"], full["Ind"], full["G"])
        errs = {}
        for k in ("Y", "Out", "dY", "dX"):
            errs[k] = orc.rel_err(out[k].cpu(), ref[k][lo:hi])
        for k in ("dWg", "dWs"):
            errs[k] = orc.rel_err(out[k].cpu(), ref[k])
        res["max_rel_err_vs_cpu_checker"] = {k: float(f"{v:.3e}") for k, v in errs.items()}
        res["tolerance"] = 3e-2
        res["ok"] = bool(all(v <= 3e-2 for v in errs.values()) and res.get("dW_bitwise_equal_across_ranks", True))
    return res


def config_entry(cname, rank, dev, peaks, args, traffic):
    """One entry of the `configs` array: the step and its operators at one benchmark configuration (single GPU)."""
    name, passes = resolve_workload(cname)
    runner = StepRunner(passes, 0, 1, dev, use_graph=not args.no_graph)
    runner.capture()
    steps = max(5, min(args.steps, 20))
    ms, _ = runner.timed(steps, 3)
    q = quantiles(ms)
    floor = step_floor_ms(runner, peaks)
    ops_rows = operator_breakdown(runner, peaks, reps=5)
    ent = {"workload": name, "dtype": str(passes[0].dtype).replace("torch.", ""),
           "routed_tokens_per_step": runner.tokens_per_step,
           "ms_per_step": {k: round(v, 5) for k, v in q.items()}, "tokens_per_s": runner.tokens_per_step / (q["median"] * 1e-3),
           "step_floor_ms": round(floor, 5), "step_frac_of_floor": floor / q["median"],
           "cuda_graph": runner.graph is not None,
           "l2": "flush buffer written between steps" if runner.flush_buf is not None else "inputs larger than L2",
           "operators": [{k: (round(v, 5) if isinstance(v, float) else v) for k, v in r.items()} for r in ops_rows]}
    if cname in ("cfg0", "cfg1-sweep") and not args.no_cpu_baseline:
        base, _, _ = cpu_baseline(passes, reps=3, full_size=True)
        ent["cpu_tokens_per_s_full_size"] = base["value"]
        ent["cpu_cores"] = base["cores"]
    del runner
    torch.cuda.empty_cache()
    return ent


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=None)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--precision", default=None, choices=["strict", "tf32"])
    ap.add_argument("--batch", type=int, default=None, help="override the global batch size B of the workload")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="leave out the per-configuration array (N=1)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    name, passes = resolve_workload(args.workload)
    if args.batch is not None:
        passes = [w.with_batch(args.batch) for w in passes]
        name = f"{name} (B={args.batch})"
    if args.impl == "reference":
        run_reference_arm(args, name, passes)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    from expertscattergather_b200 import distributed as egd, ops
    import expertscattergather_b200 as egs

    rank, world, local = egd.init_from_env()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if args.precision:
        ops.set_precision(args.precision)
    peaks = measured_peaks()
    traffic = ncu_traffic_table()

    # ---- parity of the (sharded) step against the CPU checker, before anything is timed ----
    parity = parity_check(rank, world, dev)

    # ---- inputs: generated on the host (so the CPU arm sees identical bits), pinned, copied once ----
    runner = StepRunner(passes, rank, world, dev, use_graph=not args.no_graph)
    host, devs = runner.host, runner.devs
    tokens_per_step = runner.tokens_per_step
    l2_mode = "flush buffer written between steps" if runner.flush_buf is not None else "inputs larger than L2"

    # launches per step, counted by the library
    runner.one_step(); torch.cuda.synchronize()
    c0 = ops.launch_count(); runner.one_step(); torch.cuda.synchronize()
    launches_per_step = ops.launch_count() - c0
    ops.check_status()

    runner.capture()
    sampler = ClockSampler(local)
    sampler.start()
    step_ms, (t0, t1) = runner.timed(args.steps, args.warmup)
    clocks = sampler.stop(t0, t1)
    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(total_ms, op=torch.distributed.ReduceOp.MAX)
    total_ms = float(total_ms.item())
    ops.check_status()
    ms_per_step = total_ms / args.steps
    value = tokens_per_step / (ms_per_step * 1e-3)
    step_q = quantiles(step_ms)
    used_graph = runner.graph is not None

    # ---- N > 1: the same step without the reductions, so that the exposed communication is a number ----
    phases = None
    if world > 1:
        runner.all_reduce = False
        runner.capture()
        ms_nc, _ = runner.timed(max(5, args.steps // 2), 3)
        t_nc = torch.tensor([statistics.median(ms_nc)], dtype=torch.float64, device=dev)
        torch.distributed.all_reduce(t_nc, op=torch.distributed.ReduceOp.MAX)
        runner.all_reduce = True
        phases = {"step_ms_median_this_rank": step_q["median"], "compute_only_ms": float(t_nc.item()),
                  "exposed_reduction_ms": step_q["median"] - float(t_nc.item())}

    # ---- per-operator timing -> dominant operator and its roofline ----
    breakdown = operator_breakdown(runner, peaks, reps=max(5, min(args.steps, 20)))
    dom = max((r for r in breakdown if r["op"] != "fill_out"), key=lambda r: r["ms"])
    tc_peak = tensor_peak(passes[0].dtype, peaks, dev)
    if passes[0].dtype == torch.float32:
        peaks["tf32_tflops_measured_here"] = tc_peak
    roof = {"bound": dom["bound"], "achieved": dom["achieved"], "unit": dom["unit"],
            "peak": peaks["hbm_gbs"] if dom["bound"] == "hbm" else tc_peak}
    roof["frac"] = roof["achieved"] / roof["peak"]
    dom_w = next(w for w in passes if w.name == dom["pass"])
    dom_b = runner.shard_B[passes.index(dom_w)]
    per_slot = traffic.get((dom["op"], dom["pass"].split(" ")[0]))
    roof.update({"traffic": per_slot * dom_b * dom_w.E * dom_w.K if per_slot is not None else None,
                 "kernel": f'{dom["op"]} @ {dom["pass"]}', "peak_source": peaks["source"] + " (burst)",
                 "ms_per_launch": dom["ms"], "algorithmic": dom["bytes"] if dom["bound"] == "hbm" else dom["flops"],
                 "frac_of_sustained_peak": (dom["achieved"] / peaks["bf16_tflops_sustained"])
                 if (dom["bound"] == "tensor" and passes[0].dtype != torch.float32) else None})
    floor_ms = step_floor_ms(runner, peaks)

    # ---- end to end through the public modules with host buffers ----
    e2e = None
    if not args.no_e2e:
        mods = []
        for w, d in zip(passes, devs):
            g = egs.ExpertGather(w.E, w.I, w.J).to(dev)
            s = egs.ExpertScatter(w.E, w.J, w.I).to(dev)
            g.W = torch.nn.Parameter(d["Wg"].clone()); s.W = torch.nn.Parameter(d["Ws"].clone())
            mods.append((g, s))
        reducer = egd.GradAllReducer()
        for g, s in mods:
            reducer.attach([g.W, s.W])
        res_host = [(torch.empty_like(h["Wg"]).pin_memory(), torch.empty_like(h["Ws"]).pin_memory(),
                     torch.empty(1).pin_memory()) for h in host]
        h2d = sum(h[k].numel() * h[k].element_size() for h in host for k in ("X", "Ind", "G"))
        d2h = sum(a.numel() * a.element_size() + b.numel() * b.element_size() + 4 for a, b, _ in res_host)
        copy_stream = torch.cuda.Stream(dev)
        # A pass whose batch is large goes through the modules in micro-batches of E2E_MICRO_BATCH batch elements, the
        # way a training loop feeds host-resident data: the copy of micro-batch i+1 runs under the kernels of
        # micro-batch i, the weight gradients accumulate in .grad, and only the accumulated gradient is reduced over the
        # ranks (GradAllReducer.no_sync) and copied back.
        def micro_slices(nb):
            mb = E2E_MICRO_BATCH if (nb > E2E_MICRO_BATCH and nb % E2E_MICRO_BATCH == 0) else nb
            return [(lo, lo + mb) for lo in range(0, nb, mb)]
        micro = [micro_slices(h["X"].shape[0]) for h in host]

        def e2e_step():
            # all host->device copies of the step are queued on a copy stream at its start (pinned buffers, one event per
            # micro-batch); the compute stream waits for each micro-batch's event
            main_s = torch.cuda.current_stream(dev)
            copy_stream.wait_stream(main_s)
            staged = []
            with torch.cuda.stream(copy_stream):
                for h, sl in zip(host, micro):
                    chunks = []
                    for lo, hi in sl:
                        t = tuple(h[k][lo:hi].to(dev, non_blocking=True) for k in ("X", "Ind", "G"))
                        chunks.append((t, copy_stream.record_event()))
                    staged.append(chunks)
            for w, chunks, (g, s), (rg, rs, rl) in zip(passes, staged, mods, res_host):
                g.W.grad = None; s.W.grad = None
                loss_sum = None
                for ci, (t, ready) in enumerate(chunks):
                    main_s.wait_event(ready)
                    for x in t:
                        x.record_stream(main_s)
                    X, Ind, G = t[0].requires_grad_(True), t[1], t[2]
                    with (reducer.no_sync() if ci + 1 < len(chunks) else contextlib.nullcontext()):
                        Out = s(g(X, Ind), Ind, w.T)
                        loss = (Out * G).sum()
                        loss.backward()
                    loss_sum = loss.detach().float() if loss_sum is None else loss_sum + loss.detach().float()
                reducer.finish()
                rg.copy_(g.W.grad, non_blocking=True); rs.copy_(s.W.grad, non_blocking=True)
                rl.copy_(loss_sum.reshape(1), non_blocking=True)
            torch.cuda.synchronize()

        for _ in range(3):
            e2e_step()
        runner.barrier()
        n_e2e = max(3, min(args.steps, 10))
        t0e = time.perf_counter()
        for _ in range(n_e2e):
            e2e_step()
        runner.barrier()
        dt = torch.tensor([time.perf_counter() - t0e], dtype=torch.float64, device=dev)
        if world > 1:
            torch.distributed.all_reduce(dt, op=torch.distributed.ReduceOp.MAX)
        e2e = {"value": tokens_per_step * n_e2e / float(dt.item()), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": n_e2e,
               "copied_in": "X, Ind, G (pinned host buffers) every step",
               "micro_batches": [len(sl) for sl in micro],
               "copied_back": "dW_g, dW_s and the loss every step (dX stays on the device)",
               "api": "ExpertGather / ExpertScatter modules + autograd"}
        ops.check_status()
        del mods, res_host

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu, _, _ = cpu_baseline(passes)

    configs = None
    if rank == 0 and world == 1 and not args.no_configs and args.workload is None and args.batch is None:
        del runner
        torch.cuda.empty_cache()
        configs = []
        for cname in ALL_CONFIGS:
            if cname == DEFAULT_WORKLOAD:
                configs.append({"workload": cname, "dtype": str(passes[0].dtype).replace("torch.", ""),
                                "routed_tokens_per_step": tokens_per_step,
                                "ms_per_step": {k: round(v, 5) for k, v in step_q.items()},
                                "tokens_per_s": tokens_per_step / (step_q["median"] * 1e-3),
                                "step_floor_ms": round(floor_ms, 5), "step_frac_of_floor": floor_ms / step_q["median"],
                                "cuda_graph": used_graph, "l2": l2_mode,
                                "operators": [{k: (round(v, 5) if isinstance(v, float) else v) for k, v in r.items()}
                                              for r in breakdown]})
            else:
                configs.append(config_entry(cname, rank, dev, peaks, args, traffic))

    if rank == 0:
        cfg = describe_config(name, passes, world)
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": {torch.float32: "f32 (tf32 tensor cores, %s)" % ops.get_precision(), torch.bfloat16: "bf16",
                      torch.float16: "f16"}[passes[0].dtype],
            "data": "synthetic",
            "config": cfg,
            "run": {"l2": l2_mode,
                    "cuda_graph": used_graph, "precision": ops.get_precision(),
                    "streams": "weight gradients on a side stream next to the main chain; float32 outputs zero-filled on a fill stream",
                    "ms_per_step_quantiles_this_rank": {k: round(v, 5) for k, v in step_q.items()}},
            "gpu_launches": int(launches_per_step * args.steps),
            "clocks": clocks,
            "ms_per_step_at_max_clock": (ms_per_step * clocks["sm_mhz"] / clocks["sm_max_mhz"])
            if clocks.get("sm_mhz") and clocks.get("sm_max_mhz") else None,
            "roofline": roof,
            "step_floor_ms": floor_ms, "step_frac_of_floor": floor_ms / ms_per_step,
            "per_gpu_tokens_per_s": value / world,
            "parity": parity,
            "operators": [{k: (round(v, 5) if isinstance(v, float) else v) for k, v in r.items()} for r in breakdown],
        }
        if phases is not None:
            line["phases"] = phases
        if e2e is not None:
            line["e2e"] = e2e
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if configs is not None:
            line["configs"] = configs
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
