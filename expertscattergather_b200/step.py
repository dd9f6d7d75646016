"""One explicit training step of the path: gather -> scatter -> loss = sum(Out * G) -> backward.

The six operator launches are issued directly (no autograd graph), in the order autograd would run them for
the reference's modules.  ``on_weight_grad(name, tensor)`` is called as soon as each weight gradient has been
enqueued, which is where a data-parallel caller starts that gradient's all-reduce so it overlaps the rest of
the backward pass.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import ops

__all__ = ["train_step"]


def train_step(X: torch.Tensor, Wg: torch.Tensor, Ws: torch.Tensor, Ind: torch.Tensor, G: torch.Tensor,
               on_weight_grad: Optional[Callable[[str, torch.Tensor], None]] = None) -> dict:
    """X [B,T,I], Wg [E,I,J], Ws [E,J,I], Ind [B,E,K], G [B,T,I] (the gradient of the loss w.r.t. Out).

    Returns Y, Out, dY, dX, dWg, dWs.  Equivalent to
    ``Y = ExpertGather(X, Ind); Out = ExpertScatter(Y, Ind, T); (Out*G).sum().backward()``.
    """
    T = X.shape[1]
    Y = ops.gather_gemm(X, Wg, Ind, w_layout="cn")                 # gather forward
    Out = ops.gemm_scatter(Y, Ws, Ind, T, w_layout="cn")           # scatter forward
    dY = ops.gather_gemm(G, Ws, Ind, w_layout="nc")                # scatter backward: dY
    dWs = ops.dweight(G, Y, Ind, out_layout="direct_rows")         # scatter backward: dW_s
    if on_weight_grad is not None:
        on_weight_grad("Ws", dWs)
    dX = ops.gemm_scatter(dY, Wg, Ind, T, w_layout="nc")           # gather backward: dX
    dWg = ops.dweight(X, dY, Ind, out_layout="gathered_rows")      # gather backward: dW_g
    if on_weight_grad is not None:
        on_weight_grad("Wg", dWg)
    return {"Y": Y, "Out": Out, "dY": dY, "dX": dX, "dWg": dWg, "dWs": dWs}
