"""Two ranks on two GPUs (NCCL): batch-sharded step with overlapped weight-gradient all-reduces, compared with the
unsharded CPU checker.  Skipped on boxes with fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import torch.distributed as dist
    from expertscattergather_b200 import distributed as egd, ops, workloads
    from expertscattergather_b200.workloads import Workload
    import expertscattergather_b200 as egs
    r, w, local = egd.init_from_env("nccl")
    dev = torch.device("cuda", local)
    wl = Workload("dp", 6, 128, 4, 32, 64, 32, torch.float32, "distinct", 55)
    full = workloads.make_inputs(wl)
    lo, hi = egd.shard_bounds(wl.B, rank, world)
    sl = {k: (v[lo:hi] if k in ("X", "Ind", "G") else v).to(dev) for k, v in full.items()}
    out = egd.dp_train_step(sl["X"], sl["Wg"], sl["Ws"], sl["Ind"], sl["G"])
    # module path with gradient hooks
    g = egs.ExpertGather(wl.E, wl.I, wl.J).to(dev)
    s = egs.ExpertScatter(wl.E, wl.J, wl.I).to(dev)
    g.W = torch.nn.Parameter(sl["Wg"].clone())
    s.W = torch.nn.Parameter(sl["Ws"].clone())
    red = egd.GradAllReducer().attach([g.W, s.W])
    Out = s(g(sl["X"], sl["Ind"]), sl["Ind"], wl.T)
    (Out * sl["G"]).sum().backward()
    red.finish()
    torch.cuda.synchronize()
    ops.check_status()
    torch.save({"dWg": out["dWg"].cpu(), "dWs": out["dWs"].cpu(), "dX": out["dX"].cpu(), "hook_dWg": g.W.grad.cpu(),
                "hook_dWs": s.W.grad.cpu()}, os.path.join(result_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_sharded_step_matches_unsharded_checker(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from expertscattergather_b200 import workloads
    from expertscattergather_b200.distributed import shard_bounds
    from expertscattergather_b200.workloads import Workload
    from oracle import egs_oracle as orc
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    wl = Workload("dp", 6, 128, 4, 32, 64, 32, torch.float32, "distinct", 55)
    full = workloads.make_inputs(wl)
    ref = orc.torch_step(full["X"], full["Wg"], full["Ws"], full["Ind"], full["G"])
    for r in range(world):
        p = torch.load(os.path.join(tmp_path, f"rank{r}.pt"))
        lo, hi = shard_bounds(wl.B, r, world)
        for k in ("dWg", "dWs"):
            assert orc.rel_err(p[k], ref[k]) <= 1e-5, (r, k)
            assert orc.rel_err(p["hook_" + k], ref[k]) <= 1e-5, (r, "hook", k)
        assert orc.rel_err(p["dX"], ref["dX"][lo:hi]) <= 1e-5
