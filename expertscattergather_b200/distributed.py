"""Batch-sharded data parallelism for the path: one process per GPU, weights replicated, the two weight
gradients summed over ranks.

Every operator is independent across batch elements (the token index never crosses b); only the weight
gradients sum over b.  So each rank runs the single-GPU step on its contiguous slice of the batch and the
only exchange is an all-reduce(sum) of dW_g [E,I,J] and dW_s [E,J,I].  The reference has no multi-GPU code;
this module is new functionality built on ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import contextlib
import os
from typing import Iterable, Optional

import torch
import torch.distributed as dist

__all__ = ["init_from_env", "shard_bounds", "shard_batch", "GradAllReducer", "dp_train_step", "t_sharded_scatter"]


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
    Gradient accumulation over micro-batches: run all backward passes but the last inside ``no_sync()`` (the
    meaning of ``DistributedDataParallel.no_sync``), so that only the accumulated gradient is reduced.
    """

    def __init__(self, group=None):
        self.group = group
        self._pending = []
        self._handles = []
        self._sync = True

    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside this context add to ``.grad`` without starting a reduction."""
        old, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = old

    def attach(self, params: Iterable[torch.nn.Parameter]) -> "GradAllReducer":
        for p in params:
            if p.requires_grad:
                self._handles.append(p.register_post_accumulate_grad_hook(self._hook))
        return self

    def _hook(self, param: torch.nn.Parameter) -> None:
        if self._sync:
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



def t_sharded_scatter(Y, W, Ind, T: int, group=None, scatter_fn=None) -> torch.Tensor:
    """Scatter with the experts sharded over the ranks and the OUTPUT sharded over the sequence: for sequences so long
    that no rank should hold (or add into) the whole ``[B,T,I]`` result.

    Every rank passes the slices of its own experts - ``Y`` [B,E_r,K,J], ``W`` [E_r,J,I], ``Ind`` [B,E_r,K] - computes
    their contribution to all token rows with the scatter operator and the ranks' contributions are summed with a
    reduce-scatter over the token axis: rank r returns ``Out[:, lo_r:hi_r, :]`` for its contiguous token range
    (``shard_bounds(T, r, world)``).  T must be divisible by the world size for the NCCL reduce-scatter; otherwise (and
    with backends that have no reduce-scatter, such as gloo) the sum is an all-reduce followed by a slice.
    ``scatter_fn(Y, W, Ind, T) -> [B,T,I]`` defaults to the CUDA operator; the CPU tests pass a checker instead.
    No counterpart in the reference, which is single-GPU.
    """
    if scatter_fn is None:
        from . import ops

        def scatter_fn(y, w, ind, t):
            return ops.gemm_scatter(y, w, ind, t, w_layout="cn")
    partial = scatter_fn(Y, W, Ind, T)
    if not (dist.is_initialized() and dist.get_world_size(group) > 1):
        return partial
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    lo, hi = shard_bounds(T, rank, world)
    if dist.get_backend(group) == "nccl" and T % world == 0:
        # reduce_scatter_tensor splits its input along dim 0: put the token axis first
        tb = partial.transpose(0, 1).contiguous()                     # [T, B, I]
        out = torch.empty((T // world,) + tuple(tb.shape[1:]), device=tb.device, dtype=tb.dtype)
        dist.reduce_scatter_tensor(out, tb, op=dist.ReduceOp.SUM, group=group)
        return out.transpose(0, 1).contiguous()
    dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial[:, lo:hi, :].contiguous()
