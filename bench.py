#!/usr/bin/env python
"""Benchmark of the fused expert gather/scatter path: routed tokens/s for one full step
(gather forward, scatter forward, both backwards) plus roofline and CPU-baseline figures.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl b200|reference]

One JSON line on stdout (rank 0).  For N > 1 launch with torchrun; the batch is sharded over the ranks and the
two weight gradients are all-reduced (NCCL) inside the timed step.
"""
from __future__ import annotations

import argparse
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

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of the kernels of one operator call, from the ncu
# captures summarised under profiles/ (bytes per routed slot of the captured case; scaled by the slots of the run).
NCU_TRAFFIC_PER_SLOT = {
    ("pair_fwd", "cfg1-T16384"): (75.96e6 + 18.61e6) / 16384,       # fill_zero + fused pair kernel
    ("pair_bwd", "cfg1-T16384"): (75.08e6 + 18.61e6) / 16384,
    ("scatter_fwd", "cfg4"): (326.6e6 + 110.4e6) / 262144,          # captured at B=64
    ("gather_bwd_dX", "cfg4"): (326.8e6 + 111.0e6) / 262144,
    ("scatter_bwd_dW", "cfg4"): (368.4e6 + 23.1e6) / 262144,
    ("gather_bwd_dW", "cfg4"): (368.5e6 + 23.0e6) / 262144,
    ("gather_fwd", "cfg4"): (265.6e6 + 114.5e6) / 262144,
    ("scatter_bwd_dY", "cfg4"): (260.5e6 + 113.1e6) / 262144,
}
L2_BYTES = 126 * 1024 * 1024
METRIC = "gather+scatter fwd+bwd routed tokens/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def resolve_workload(name, n_gpus):
    """Names -> list of Workload passes that make up one step, and the scaling mode."""
    if name is None:
        multi_box = n_gpus > 1 or (torch.cuda.is_available() and torch.cuda.device_count() > 1)
        name = "cfg4" if multi_box else "cfg1-sweep"
    if name == "cfg1-sweep":
        return name, [wl.WORKLOADS[k] for k in wl.CFG1_SWEEP]
    if name in wl.WORKLOADS:
        return name, [wl.WORKLOADS[name]]
    raise SystemExit(f"unknown workload {name!r}; choose from cfg1-sweep, " + ", ".join(wl.WORKLOADS))


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
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
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


# -------------------------------------------------------------------------------------------------------------
# CPU arm: the checker's torch restatement of the reference path, timed on the host cores
# -------------------------------------------------------------------------------------------------------------
def cpu_baseline(passes, budget_s=20.0, reps=3):
    """Times oracle.torch_step on the host for a bounded sample of each pass; returns routed tokens/s."""
    from oracle import egs_oracle as orc   # the one place the benchmark executes the checker
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    tokens = 0.0
    seconds = 0.0
    samples = []
    for w in passes:
        # slice the batch so that one repetition costs about budget/(reps+1)/len(passes) seconds
        flops = 12 * w.E * w.K * w.I * w.J
        est_per_b = flops / 2e10 + w.T * w.I * 4e-8
        b = max(1, min(w.B, int(budget_s / (reps + 1) / len(passes) / max(est_per_b, 1e-6))))
        ins = wl.make_inputs(w, B=b)
        orc.torch_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            orc.torch_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
            ts.append(time.perf_counter() - t0)
        t = statistics.median(ts)
        tokens += b * w.E * w.K
        seconds += t
        samples.append(f"{w.name}: B={b} of {w.B}, {t * 1e3:.1f} ms")
    return {"value": tokens / seconds, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": "; ".join(samples) + " (median of %d, batch slices scale linearly in B)" % reps}, seconds


def run_reference_arm(args, name, passes):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    base = None
    t_all = time.perf_counter()
    for i in range(args.warmup + args.steps):
        base, secs = cpu_baseline(passes, budget_s=6.0, reps=1)
        if i >= args.warmup:
            vals.append((base["value"], secs))
    v = statistics.median(x[0] for x in vals)
    base["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": statistics.median(x[1] for x in vals) * 1e3,
            "higher_is_better": True, "scaling": "strong" if name.startswith("cfg4") else "weak", "vs_baseline": None,
            "dtype": str(passes[0].dtype).replace("torch.", ""), "data": "synthetic",
            "config": {"workload": name, "device": "host CPU", "note": "torch restatement of egs/baselines.py; "
                       "each step is a bounded batch slice of the workload"},
            "cpu_baseline": base,
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": time.perf_counter() - t_all}
    print(json.dumps(line), flush=True)


# -------------------------------------------------------------------------------------------------------------
# GPU arm
# -------------------------------------------------------------------------------------------------------------
def op_work(w, B, U, op):
    """Algorithmic (flops, bytes) of one operator launch group."""
    s = torch.empty((), dtype=w.dtype).element_size()
    N = B * w.E * w.K
    WB = w.E * w.I * w.J * s
    fl = 2 * N * w.I * w.J
    if op in ("gather_fwd", "scatter_bwd_dY"):
        return fl, U * w.I * s + WB + 8 * N + N * w.J * s
    if op in ("scatter_fwd", "gather_bwd_dX"):
        return fl, N * w.J * s + WB + 8 * N + B * w.T * w.I * s
    if op in ("pair_fwd", "pair_bwd"):
        # fused G -> S: token rows read once, both weights, the middle tensor written once, the output written once
        return 2 * fl, U * w.I * s + 2 * WB + 8 * N + N * w.J * s + B * w.T * w.I * s
    return fl, U * w.I * s + N * w.J * s + 8 * N + WB      # dW_g, dW_s


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=None)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--precision", default=None, choices=["strict", "tf32"])
    ap.add_argument("--batch", type=int, default=None, help="override the global batch size B of the workload")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    name, passes = resolve_workload(args.workload, args.gpus)
    if args.batch is not None:
        passes = [w.with_batch(args.batch) for w in passes]
        name = f"{name} (B={args.batch})"
    if args.impl == "reference":
        run_reference_arm(args, name, passes)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    from expertscattergather_b200 import distributed as egd, ops
    from expertscattergather_b200.step import takes_fused_pairs, train_step
    import expertscattergather_b200 as egs

    rank, world, local = egd.init_from_env()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if args.precision:
        ops.set_precision(args.precision)
    peaks = measured_peaks()

    # ---- inputs: generated on the host (so the CPU arm could see identical bits), pinned, copied once ----
    host, devs, shard_B = [], [], []
    for w in passes:
        lo, hi = egd.shard_bounds(w.B, rank, world)
        h = wl.make_inputs(w, B=hi - lo, b0=lo)
        h = {k: v.pin_memory() for k, v in h.items()}
        host.append(h)
        devs.append({k: v.to(dev, non_blocking=True) for k, v in h.items()})
        shard_B.append(hi - lo)
    torch.cuda.synchronize()
    tokens_per_step = sum(w.routed for w in passes)            # whole job, all ranks
    footprint = sum(sum(v.numel() * v.element_size() for v in d.values()) for d in devs)
    flush_buf = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev) if footprint < 4 * L2_BYTES else None

    def one_step(reducer_group=None):
        outs = []
        for d in devs:
            if world > 1:
                outs.append(egd.dp_train_step(d["X"], d["Wg"], d["Ws"], d["Ind"], d["G"]))
            else:
                outs.append(train_step(d["X"], d["Wg"], d["Ws"], d["Ind"], d["G"]))
        return outs

    # launches per step, counted by the library
    one_step(); torch.cuda.synchronize()
    c0 = ops.launch_count(); one_step(); torch.cuda.synchronize()
    launches_per_step = ops.launch_count() - c0
    ops.check_status()

    use_graph = (world == 1) and not args.no_graph
    graph = None
    if use_graph:
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    one_step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_outs = one_step()   # noqa: F841  (keeps the captured outputs alive)
        except Exception as exc:          # capture refused: time plain launches instead
            sys.stderr.write(f"CUDA graph capture failed ({exc}); timing plain launches\n")
            graph = None
            torch.cuda.synchronize()

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            one_step()

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        if flush_buf is not None:
            flush_buf.zero_()
        run_step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    for i in range(args.steps):
        if flush_buf is not None:
            flush_buf.zero_()
        starts[i].record()
        run_step()
        stops[i].record()
    barrier()
    step_ms = [a.elapsed_time(b) for a, b in zip(starts, stops)]
    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(total_ms, op=torch.distributed.ReduceOp.MAX)
    total_ms = float(total_ms.item())
    ops.check_status()
    ms_per_step = total_ms / args.steps
    value = tokens_per_step / (ms_per_step * 1e-3)

    # ---- per-operator timing on this stream -> dominant operator and its roofline ----
    def time_op(fn, reps):
        """Device time of one operator call (its kernels only): the call is captured into a CUDA graph so that
        host launch overhead stays out of the events; L2 is flushed between repetitions."""
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

    breakdown = []
    reps = max(5, min(args.steps, 20))
    for w, d, b in zip(passes, devs, shard_B):
        U = wl.algorithmic_work(w, Ind=host[passes.index(w)]["Ind"], B=b)["U"]
        Y = ops.gather_gemm(d["X"], d["Wg"], d["Ind"])
        dY = ops.gather_gemm(d["G"], d["Ws"], d["Ind"], w_layout="nc")
        if takes_fused_pairs(d["X"], d["Wg"], d["Ind"]):
            # the step runs each pair as one fused kernel: time what it runs
            calls = {
                "pair_fwd": lambda: ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], d["Ind"]),
                "scatter_bwd_dW": lambda: ops.dweight(d["G"], Y, d["Ind"], out_layout="direct_rows"),
                "pair_bwd": lambda: ops.gather_scatter_pair(d["G"], d["Ws"], d["Wg"], d["Ind"], w_layout="nc"),
                "gather_bwd_dW": lambda: ops.dweight(d["X"], dY, d["Ind"]),
            }
        else:
            calls = {
                "gather_fwd": lambda: ops.gather_gemm(d["X"], d["Wg"], d["Ind"]),
                "scatter_fwd": lambda: ops.gemm_scatter(Y, d["Ws"], d["Ind"], w.T),
                "scatter_bwd_dY": lambda: ops.gather_gemm(d["G"], d["Ws"], d["Ind"], w_layout="nc"),
                "scatter_bwd_dW": lambda: ops.dweight(d["G"], Y, d["Ind"], out_layout="direct_rows"),
                "gather_bwd_dX": lambda: ops.gemm_scatter(dY, d["Wg"], d["Ind"], w.T, w_layout="nc"),
                "gather_bwd_dW": lambda: ops.dweight(d["X"], dY, d["Ind"]),
            }
        for op, fn in calls.items():
            ms = time_op(fn, reps)
            fl, by = op_work(w, b, U, op)
            breakdown.append({"pass": w.name, "op": op, "ms": ms, "flops": fl, "bytes": by})
        del Y, dY
    clocks = sampler.stop()      # sampled from the start of the timed steps to the end of the per-operator timing
    dom = max(breakdown, key=lambda r: r["ms"])
    if passes[0].dtype == torch.float32:
        # no TF32 figure in MEASURED_PEAKS.json: measure a TF32 torch.matmul the same way (8192^3, best of 10)
        a = torch.randn(8192, 8192, device=dev); bmat = torch.randn(8192, 8192, device=dev)
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        best = float("inf")
        for _ in range(12):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); torch.matmul(a, bmat); e1.record(); e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        torch.backends.cuda.matmul.allow_tf32 = prev
        del a, bmat
        tc_peak = 2 * 8192 ** 3 / (best * 1e-3) / 1e12
        peaks["tf32_tflops_measured_here"] = tc_peak
    else:
        tc_peak = peaks["bf16_tflops"]
    t_hbm = dom["bytes"] / (peaks["hbm_gbs"] * 1e9)
    t_tc = dom["flops"] * (3 if (passes[0].dtype == torch.float32 and ops.get_precision() == "strict") else 1) / (tc_peak * 1e12)
    if t_hbm >= t_tc:
        ach = dom["bytes"] / (dom["ms"] * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"]}
    else:
        ach = dom["flops"] / (dom["ms"] * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": tc_peak, "unit": "TFLOP/s", "frac": ach / tc_peak}
    dom_w = next(w for w in passes if w.name == dom["pass"])
    dom_b = shard_B[passes.index(dom_w)]
    per_slot = NCU_TRAFFIC_PER_SLOT.get((dom["op"], dom["pass"].split(" ")[0]))
    traffic = per_slot * dom_b * dom_w.E * dom_w.K if per_slot is not None else None
    roof.update({"traffic": traffic, "kernel": f'{dom["op"]} @ {dom["pass"]}', "peak_source": peaks["source"],
                 "ms_per_launch": dom["ms"], "algorithmic": dom["bytes"] if roof["bound"] == "hbm" else dom["flops"]})
    # whole-step floor for context
    alg = [wl.algorithmic_work(w, Ind=h["Ind"], B=b) for w, h, b in zip(passes, host, shard_B)]
    step_floor_ms = sum(max(a["bytes"] / (peaks["hbm_gbs"] * 1e9), a["flops"] / (tc_peak * 1e12)) for a in alg) * 1e3

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

        def e2e_step():
            # the host->device copies of all passes are queued on a copy stream at the start of the step (pinned
            # buffers, one event per pass); the compute stream waits for each pass's event, so the copies of the next
            # pass run under the kernels of the current one, as an input prefetcher of a training loop would do
            main = torch.cuda.current_stream(dev)
            copy_stream.wait_stream(main)
            staged = []
            with torch.cuda.stream(copy_stream):
                for h in host:
                    t = tuple(h[k].to(dev, non_blocking=True) for k in ("X", "Ind", "G"))
                    staged.append((t, copy_stream.record_event()))
            for w, (t, ready), (g, s), (rg, rs, rl) in zip(passes, staged, mods, res_host):
                main.wait_event(ready)
                for x in t:
                    x.record_stream(main)
                X, Ind, G = t[0].requires_grad_(True), t[1], t[2]
                g.W.grad = None; s.W.grad = None
                Out = s(g(X, Ind), Ind, w.T)
                loss = (Out * G).sum()
                loss.backward()
                reducer.finish()
                rg.copy_(g.W.grad, non_blocking=True); rs.copy_(s.W.grad, non_blocking=True)
                rl.copy_(loss.detach().float().reshape(1), non_blocking=True)
            torch.cuda.synchronize()

        for _ in range(3):
            e2e_step()
        barrier()
        n_e2e = max(3, min(args.steps, 10))
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            e2e_step()
        barrier()
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
        if world > 1:
            torch.distributed.all_reduce(dt, op=torch.distributed.ReduceOp.MAX)
        e2e = {"value": tokens_per_step * n_e2e / float(dt.item()), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": n_e2e}
        ops.check_status()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu, _ = cpu_baseline(passes)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if name.startswith("cfg4") else "weak", "vs_baseline": None,
            "dtype": {torch.float32: "f32 (tf32 tensor cores, %s)" % ops.get_precision(), torch.bfloat16: "bf16",
                      torch.float16: "f16"}[passes[0].dtype],
            "data": "synthetic",
            "config": {"workload": name, "passes": [f"{w.name}: B={w.B} T={w.T} E={w.E} K={w.K} I={w.I} J={w.J}" for w in passes],
                       "routed_tokens_per_step": tokens_per_step, "parallelism": f"dp{world} (batch-sharded, dW all-reduce)",
                       "l2": "flush buffer written between steps" if flush_buf is not None else "inputs larger than L2",
                       "cuda_graph": bool(graph is not None), "precision": ops.get_precision(),
                       "streams": "output zero fills on a fill stream, weight gradients on a side stream, next to the G->S->dY->dX chain"},
            "gpu_launches": int(launches_per_step * args.steps),
            "clocks": clocks,
            "roofline": roof,
            "step_floor_ms": step_floor_ms, "step_frac_of_floor": step_floor_ms / ms_per_step,
            "per_gpu_tokens_per_s": value / world,
            "operators": [{k: (round(v, 5) if isinstance(v, float) else v) for k, v in r.items()} for r in breakdown],
        }
        if e2e is not None:
            line["e2e"] = e2e
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
