"""Batch sharding + weight-gradient all-reduce over gloo (world_size 2), with the CPU checker as the
per-rank step, compared with the unsharded result."""
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
    torch.save({"dWg": out["dWg"], "dWs": out["dWs"], "dX": out["dX"], "hook_dWg": Wg.grad, "hook_dWs": Ws.grad},
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
        lo, hi = shard_bounds(B, r, world)
        assert torch.allclose(p["dX"], ref["dX"][lo:hi], rtol=1e-12, atol=1e-12)
