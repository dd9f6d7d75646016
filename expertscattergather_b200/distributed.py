"""Batch-sharded data parallelism for the path: one process per GPU, weights replicated, the two weight
gradients summed over ranks.

Every operator is independent across batch elements (the token index never crosses b); only the weight
gradients sum over b.  So each rank runs the single-GPU step on its contiguous slice of the batch and the
only exchange is an all-reduce(sum) of dW_g [E,I,J] and dW_s [E,J,I].  The reference has no multi-GPU code;
this module is new functionality built on ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import os
from typing import Iterable, Optional

import torch
import torch.distributed as dist

__all__ = ["init_from_env", "shard_bounds", "shard_batch", "GradAllReducer", "dp_train_step"]


def init_from_env(backend: Optional[str] = None) -> tuple[int, int, int]:
    """Initialises the default process group from RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* and returns
    (rank, world_size, local_rank).  With WORLD_SIZE unset or 1 nothing is initialised."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend)
    return rank, world, local


def shard_bounds(B: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous batch slice [lo, hi) of `rank`; the first B % world ranks get one extra element."""
    base, extra = divmod(B, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    lo, hi = shard_bounds(t.shape[0], rank, world)
    return t[lo:hi]


class GradAllReducer:
    """Sums parameter gradients over the ranks as soon as autograd has produced them.

    ``attach(params)`` registers a post-accumulate-grad hook per parameter that starts an asynchronous
    all-reduce of ``param.grad``; ``finish()`` waits for all of them.  With the gather and scatter modules in
    one model the scatter weight's reduction is in flight while the gather backward still computes.
    """

    def __init__(self, group=None):
        self.group = group
        self._pending = []
        self._handles = []

    def attach(self, params: Iterable[torch.nn.Parameter]) -> "GradAllReducer":
        for p in params:
            if p.requires_grad:
                self._handles.append(p.register_post_accumulate_grad_hook(self._hook))
        return self

    def _hook(self, param: torch.nn.Parameter) -> None:
        self.reduce_async(param.grad)

    def reduce_async(self, t: torch.Tensor) -> None:
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            self._pending.append(dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    def finish(self) -> None:
        for w in self._pending:
            w.wait()
        self._pending.clear()

    def detach(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles.clear()


def dp_train_step(X, Wg, Ws, Ind, G, group=None, step_fn=None) -> dict:
    """The explicit step on this rank's batch slice with the two weight-gradient all-reduces overlapped.

    ``step_fn`` defaults to the CUDA step (``step.train_step``); the CPU tests pass a checker instead.
    After return dWg and dWs hold the sums over all ranks; every other output is local to the slice.
    """
    if step_fn is None:
        from .step import train_step as step_fn
    reducer = GradAllReducer(group)
    out = step_fn(X, Wg, Ws, Ind, G, on_weight_grad=lambda _name, t: reducer.reduce_async(t))
    reducer.finish()
    return out
