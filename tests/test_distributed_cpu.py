"""Batch sharding + weight-gradient all-reduce over gloo (world_size 2), with the CPU checker as the
per-rank step, compared with the unsharded result."""
import contextlib
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_step(X, Wg, Ws, Ind, G, on_weight_grad=None):
    from oracle import egs_oracle as orc
    out = orc.torch_step(X, Wg, Ws, Ind, G)
    if on_weight_grad is not None:
        on_weight_grad("Ws", out["dWs"])
        on_weight_grad("Wg", out["dWg"])
    return out


def _worker(rank, world, port, B, result_dir):
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from expertscattergather_b200 import distributed as egd, workloads
    from expertscattergather_b200.workloads import Workload
    r, w, _ = egd.init_from_env("gloo")
    assert (r, w) == (rank, world)
    wl = Workload("t", B, 12, 3, 4, 8, 6, torch.float64, "distinct", 77)
    full = workloads.make_inputs(wl)
    sl = {k: (egd.shard_batch(v, rank, world) if k in ("X", "Ind", "G") else v) for k, v in full.items()}
    # (a) explicit step with overlapped reductions
    out = egd.dp_train_step(sl["X"], sl["Wg"], sl["Ws"], sl["Ind"], sl["G"], step_fn=_oracle_step)
    # (b) autograd modules + GradAllReducer hooks
    from oracle import egs_oracle as orc
    Wg = torch.nn.Parameter(full["Wg"].clone())
    Ws = torch.nn.Parameter(full["Ws"].clone())
    red = egd.GradAllReducer().attach([Wg, Ws])
    Y = orc.torch_gather(sl["X"], Wg, sl["Ind"])
    O = orc.torch_scatter(Y, Ws, sl["Ind"], wl.T)
    (O * sl["G"]).sum().backward()
    red.finish()
    red.detach()
    # (c) the same with the slice cut into micro-batches: gradients accumulate locally, one reduction at the end
    Wg2 = torch.nn.Parameter(full["Wg"].clone())
    Ws2 = torch.nn.Parameter(full["Ws"].clone())
    red2 = egd.GradAllReducer().attach([Wg2, Ws2])
    nb = sl["X"].shape[0]
    for b in range(nb):
        ctx = red2.no_sync() if b < nb - 1 else contextlib.nullcontext()
        with ctx:
            Yb = orc.torch_gather(sl["X"][b:b + 1], Wg2, sl["Ind"][b:b + 1])
            Ob = orc.torch_scatter(Yb, Ws2, sl["Ind"][b:b + 1], wl.T)
            (Ob * sl["G"][b:b + 1]).sum().backward()
    red2.finish()
    red2.detach()
    torch.save({"dWg": out["dWg"], "dWs": out["dWs"], "dX": out["dX"], "hook_dWg": Wg.grad, "hook_dWs": Ws.grad,
                "micro_dWg": Wg2.grad, "micro_dWs": Ws2.grad},
               os.path.join(result_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("B", [4, 5])
def test_two_rank_sharded_step_matches_unsharded(tmp_path, B):
    from expertscattergather_b200 import workloads
    from expertscattergather_b200.distributed import shard_bounds
    from expertscattergather_b200.workloads import Workload
    from oracle import egs_oracle as orc
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), B, str(tmp_path)), nprocs=world, join=True)
    wl = Workload("t", B, 12, 3, 4, 8, 6, torch.float64, "distinct", 77)
    full = workloads.make_inputs(wl)
    ref = orc.torch_step(full["X"], full["Wg"], full["Ws"], full["Ind"], full["G"])
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    for r, p in enumerate(parts):
        for k in ("dWg", "dWs"):
            assert torch.allclose(p[k], ref[k], rtol=1e-12, atol=1e-12), (r, k)
            assert torch.allclose(p["hook_" + k], ref[k], rtol=1e-12, atol=1e-12), (r, "hook", k)
            assert torch.allclose(p["micro_" + k], ref[k], rtol=1e-12, atol=1e-12), (r, "micro-batches", k)
        lo, hi = shard_bounds(B, r, world)
        assert torch.allclose(p["dX"], ref["dX"][lo:hi], rtol=1e-12, atol=1e-12)


# ---------------------------------------------------------------------------------------------------------
# sequence-sharded scatter: experts split over the ranks, the output split over the token axis
# ---------------------------------------------------------------------------------------------------------
def _t_shard_worker(rank, world, port, T, result_dir):
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from expertscattergather_b200 import distributed as egd, workloads
    from expertscattergather_b200.workloads import Workload
    from oracle import egs_oracle as orc
    egd.init_from_env("gloo")
    wl = Workload("ts", 3, T, 4, 5, 8, 6, torch.float64, "replace", 83)
    full = workloads.make_inputs(wl)
    Y = orc.torch_gather(full["X"], full["Wg"], full["Ind"])
    e_lo, e_hi = egd.shard_bounds(wl.E, rank, world)                      # this rank's experts
    out = egd.t_sharded_scatter(Y[:, e_lo:e_hi].contiguous(), full["Ws"][e_lo:e_hi].contiguous(),
                                full["Ind"][:, e_lo:e_hi].contiguous(), wl.T, scatter_fn=orc.torch_scatter)
    torch.save(out, os.path.join(result_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("T", [12, 13])
def test_two_rank_sequence_sharded_scatter(tmp_path, T):
    from expertscattergather_b200 import workloads
    from expertscattergather_b200.distributed import shard_bounds
    from expertscattergather_b200.workloads import Workload
    from oracle import egs_oracle as orc
    world = 2
    mp.spawn(_t_shard_worker, args=(world, _free_port(), T, str(tmp_path)), nprocs=world, join=True)
    wl = Workload("ts", 3, T, 4, 5, 8, 6, torch.float64, "replace", 83)
    full = workloads.make_inputs(wl)
    ref = orc.torch_scatter(orc.torch_gather(full["X"], full["Wg"], full["Ind"]), full["Ws"], full["Ind"], T)
    for r in range(world):
        lo, hi = shard_bounds(T, r, world)
        got = torch.load(os.path.join(tmp_path, f"rank{r}.pt"))
        assert got.shape == (wl.B, hi - lo, wl.I)
        assert torch.allclose(got, ref[:, lo:hi], rtol=1e-12, atol=1e-12), r


# ---------------------------------------------------------------------------------------------------------
# failures among the ranks, made on the host: nothing here touches a GPU
# ---------------------------------------------------------------------------------------------------------
def _join_all(ctx, seconds):
    """mp.spawn(join=False).join() returns as soon as ONE process has ended: wait for all of them, with a deadline."""
    import time
    deadline = time.time() + seconds
    while not ctx.join(timeout=2):
        assert time.time() < deadline, "ranks still running after the deadline"


def _leaving_worker(rank, world, port, result_dir):
    """Rank 1 takes part in step 0 and then leaves between steps (no collective of its own in flight).  Rank 0 starts
    step 1: its weight-gradient reductions can never complete, and finish() must raise within the process group's
    timeout instead of hanging."""
    import datetime
    import sys
    import time
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from expertscattergather_b200 import distributed as egd, workloads
    from expertscattergather_b200.workloads import Workload
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
    wl = Workload("f", 4, 12, 3, 4, 8, 6, torch.float64, "distinct", 79)
    full = workloads.make_inputs(wl)
    sl = {k: (egd.shard_batch(v, rank, world) if k in ("X", "Ind", "G") else v) for k, v in full.items()}
    egd.dp_train_step(sl["X"], sl["Wg"], sl["Ws"], sl["Ind"], sl["G"], step_fn=_oracle_step)      # step 0: everybody
    outcome = "left"
    if rank == 0:
        t0 = time.time()
        try:
            egd.dp_train_step(sl["X"], sl["Wg"], sl["Ws"], sl["Ind"], sl["G"], step_fn=_oracle_step)
            outcome = "completed"
        except Exception as exc:   # the survivor learns of the loss as an error of its collective
            outcome = f"raised {type(exc).__name__} after {time.time() - t0:.1f}s"
    with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)          # no destroy_process_group: the group is broken on purpose


def test_a_rank_that_leaves_between_steps_makes_the_survivor_raise(tmp_path):
    world = 2
    ctx = mp.spawn(_leaving_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=False)
    _join_all(ctx, 120)
    out0 = open(os.path.join(tmp_path, "rank0.txt")).read()
    assert open(os.path.join(tmp_path, "rank1.txt")).read() == "left"
    assert out0.startswith("raised"), out0
    seconds = float(out0.split("after ")[1].rstrip("s"))
    assert seconds < 60, out0


def _mismatch_worker(rank, world, port, result_dir):
    """Rank 1 shows up with weights of another shape: the element counts of the reductions differ, which the collective
    reports as an error (or times out on) instead of summing garbage."""
    import datetime
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from expertscattergather_b200 import distributed as egd, workloads
    from expertscattergather_b200.workloads import Workload
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
    wl = Workload("m", 4, 12, 3, 4, 8, 6 if rank == 0 else 7, torch.float64, "distinct", 79)
    full = workloads.make_inputs(wl)
    sl = {k: (egd.shard_batch(v, rank, world) if k in ("X", "Ind", "G") else v) for k, v in full.items()}
    try:
        egd.dp_train_step(sl["X"], sl["Wg"], sl["Ws"], sl["Ind"], sl["G"], step_fn=_oracle_step)
        outcome = "completed"
    except Exception as exc:
        outcome = f"raised {type(exc).__name__}"
    with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)


def test_mismatched_weight_shapes_across_ranks_are_an_error(tmp_path):
    """Either a rank's collective raises, or the transport aborts the rank outright (gloo enforces equal message sizes in
    a background thread): in no case do both ranks come back with a summed gradient."""
    world = 2
    ctx = mp.spawn(_mismatch_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=False)
    crashed = False
    try:
        _join_all(ctx, 120)
    except Exception:        # torch.multiprocessing reports a rank that died
        crashed = True
    outs = [open(p).read() if os.path.exists(p) else "died" for p in (os.path.join(tmp_path, f"rank{r}.txt") for r in range(world))]
    assert crashed or any(o.startswith("raised") or o == "died" for o in outs), outs
    assert not all(o == "completed" for o in outs), outs
