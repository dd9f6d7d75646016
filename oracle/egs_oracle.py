"""CPU oracle for the fused expert gather / scatter path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, the algorithm of the reference's torch path
(``egs/baselines.py``), which is the reference's own parity oracle
(``test_all.py:9-11`` compares the Triton kernels against it).  Nothing in the
shipped package imports this module: only the tests, the smoke check and the
CPU-baseline leg of the benchmark do, and only as the checker / the CPU timing
baseline, never as the product path.

Parity pin: the reference holds no golden vectors, known-answer tests, fixtures
or seeds for this path (its tests draw fresh random tensors and compare two
implementations with each other).  The pin used instead is a set of outputs of
the reference's own modules, produced by importing them in a container that has
the reference checked out (``tests/golden/make_golden.py``) and committed as
``tests/golden/*.npz``; ``tests/test_oracle_golden.py`` checks every function
below against those files.

Two restatements are kept, so that they also check each other:

* ``torch_*``  - the same ATen calls the reference makes (``torch.gather`` +
  ``einsum`` and ``einsum`` + ``scatter_add_``), gradients through autograd.
  This is what is timed as the CPU baseline because it is what the reference's
  CPU path executes.
* ``np_*``     - explicit numpy formulas (take_along_axis / einsum / add.at) for
  the forward operators and for the three gradient operators, evaluated in
  float64.  These are the "truth" used to judge accumulated rounding error.

Tensor layouts follow the reference (``README.md:7-9``):
    X[B,T,I]   W_g[E,I,J]   W_s[E,J,I]   Ind[B,E,K] (ints in [0,T))   Y[B,E,K,J]
"""
from __future__ import annotations

import numpy as np
import torch

__all__ = [
    "torch_gather", "torch_scatter", "torch_gather_module_step", "torch_scatter_module_step",
    "torch_step", "np_gather", "np_scatter", "np_dweight", "np_step", "rel_err",
]


# ---------------------------------------------------------------------------------------------
# torch restatement (what the reference's CPU path runs)
# ---------------------------------------------------------------------------------------------

def torch_gather(X: torch.Tensor, W: torch.Tensor, Ind: torch.Tensor) -> torch.Tensor:
    """Y[b,e,k,:] = X[b, Ind[b,e,k], :] @ W[e].

    Follows ``TorchReshapedGatherEinsum.forward`` (``egs/baselines.py:69-76``): the index is
    flattened to [B, E*K], broadcast over I, used by ``torch.gather`` along the token axis, and the
    gathered [B,E,K,I] block is contracted with W by ``einsum('beki,eij->bekj')``.
    """
    B, T, I = X.shape
    _, E, K = Ind.shape
    flat = Ind.reshape(B, E * K).to(torch.int64)
    rows = torch.gather(X, 1, flat.unsqueeze(-1).expand(B, E * K, I)).reshape(B, E, K, I)
    return torch.einsum("beki,eij->bekj", rows, W)


def torch_scatter(Y: torch.Tensor, W: torch.Tensor, Ind: torch.Tensor, T: int) -> torch.Tensor:
    """Out[b,t,:] = sum over (e,k) with Ind[b,e,k]==t of Y[b,e,k,:] @ W[e].

    Follows ``TorchEinsumScatter.forward`` (``egs/baselines.py:174-184``):
    ``einsum('bekj,eji->beki')`` then ``scatter_add_`` along the token axis into zeros.
    """
    B, E, K, J = Y.shape
    I = W.shape[-1]
    pre = torch.einsum("bekj,eji->beki", Y, W)
    out = torch.zeros(B, T, I, dtype=Y.dtype, device=Y.device)
    idx = Ind.to(torch.int64).unsqueeze(-1).expand(B, E, K, I).reshape(B, E * K, I)
    out.scatter_add_(1, idx, pre.reshape(B, E * K, I))
    return out


def torch_gather_module_step(X, W, Ind, GY):
    """Forward + backward of the gather module alone with loss = sum(Y * GY).

    Mirrors ``shape_test_gather`` (``test_all.py:13-45``) with a non-trivial upstream gradient.
    Returns Y, dX, dW.
    """
    X = X.detach().clone().requires_grad_(True)
    W = W.detach().clone().requires_grad_(True)
    Y = torch_gather(X, W, Ind)
    (Y * GY).sum().backward()
    return {"Y": Y.detach(), "dX": X.grad, "dW": W.grad}


def torch_scatter_module_step(Y, W, Ind, T, GO):
    """Forward + backward of the scatter module alone with loss = sum(Out * GO).

    Mirrors ``shape_test_scatter`` (``test_all.py:47-77``).  Returns Out, dY, dW.
    """
    Y = Y.detach().clone().requires_grad_(True)
    W = W.detach().clone().requires_grad_(True)
    Out = torch_scatter(Y, W, Ind, T)
    (Out * GO).sum().backward()
    return {"Out": Out.detach(), "dY": Y.grad, "dW": W.grad}


def torch_step(X, Wg, Ws, Ind, G):
    """One full step: Y = gather(X); Out = scatter(Y); loss = sum(Out*G); backward.

    Returns Y, Out, dX, dWg, dWs (and dY, the gradient reaching Y).
    """
    T = X.shape[1]
    X = X.detach().clone().requires_grad_(True)
    Wg = Wg.detach().clone().requires_grad_(True)
    Ws = Ws.detach().clone().requires_grad_(True)
    Y = torch_gather(X, Wg, Ind)
    Y.retain_grad()
    Out = torch_scatter(Y, Ws, Ind, T)
    (Out * G).sum().backward()
    return {"Y": Y.detach(), "Out": Out.detach(), "dY": Y.grad, "dX": X.grad,
            "dWg": Wg.grad, "dWs": Ws.grad}


# ---------------------------------------------------------------------------------------------
# numpy restatement in float64 (explicit forward and gradient formulas)
# ---------------------------------------------------------------------------------------------

def _f64(a):
    if isinstance(a, torch.Tensor):
        a = a.detach().to(torch.float64).cpu().numpy()
    return np.asarray(a, dtype=np.float64)


def _idx(a):
    if isinstance(a, torch.Tensor):
        a = a.detach().cpu().numpy()
    return np.asarray(a).astype(np.int64)


def np_gather(X, W, Ind):
    """Operator G: gathered rows times W[e] (``egs/triton_kernels.py:70`` states the formula)."""
    X, W, Ind = _f64(X), _f64(W), _idx(Ind)
    B, T, I = X.shape
    _, E, K = Ind.shape
    rows = np.take_along_axis(X, Ind.reshape(B, E * K, 1), axis=1).reshape(B, E, K, I)
    # batched matmul over experts: [E, B*K, I] @ [E, I, J]
    per_expert = np.matmul(rows.transpose(1, 0, 2, 3).reshape(E, B * K, I), W)
    return np.ascontiguousarray(per_expert.reshape(E, B, K, -1).transpose(1, 0, 2, 3))


def np_scatter(Y, W, Ind, T):
    """Operator S: (Y @ W[e]) added at rows Ind, duplicates accumulate (``egs/triton_kernels.py:618``)."""
    Y, W, Ind = _f64(Y), _f64(W), _idx(Ind)
    B, E, K, J = Y.shape
    pre = np.matmul(Y.transpose(1, 0, 2, 3).reshape(E, B * K, J), W).reshape(E, B, K, -1).transpose(1, 0, 2, 3)
    out = np.zeros((B, T, W.shape[-1]), dtype=np.float64)
    b_idx = np.broadcast_to(np.arange(B).reshape(B, 1, 1), Ind.shape)
    np.add.at(out, (b_idx.reshape(-1), Ind.reshape(-1)), pre.reshape(B * E * K, -1))
    return out


def np_dweight(Xsrc, Ysrc, Ind):
    """Operator D: dW[e,i,j] = sum_{b,k} Xsrc[b,Ind[b,e,k],i] * Ysrc[b,e,k,j] (``egs/triton_kernels.py:283``)."""
    Xsrc, Ysrc, Ind = _f64(Xsrc), _f64(Ysrc), _idx(Ind)
    B, T, I = Xsrc.shape
    _, E, K = Ind.shape
    rows = np.take_along_axis(Xsrc, Ind.reshape(B, E * K, 1), axis=1).reshape(B, E, K, I)
    a = rows.transpose(1, 3, 0, 2).reshape(E, I, B * K)
    return np.matmul(a, Ysrc.transpose(1, 0, 2, 3).reshape(E, B * K, -1))


def np_step(X, Wg, Ws, Ind, G):
    """Full step in float64 from the explicit formulas (no autograd)."""
    T = _f64(X).shape[1]
    Wg64, Ws64 = _f64(Wg), _f64(Ws)
    Y = np_gather(X, Wg64, Ind)
    Out = np_scatter(Y, Ws64, Ind, T)
    # scatter backward: dY is operator G on dOut with W_s read transposed; dW_s[e,j,i] = sum Y * gathered dOut
    dY = np_gather(G, np.swapaxes(Ws64, 1, 2), Ind)
    dWs = np.swapaxes(np_dweight(G, Y, Ind), 1, 2)
    # gather backward: dX is operator S on dY with W_g read transposed; dW_g from gathered X and dY
    dX = np_scatter(dY, np.swapaxes(Wg64, 1, 2), Ind, T)
    dWg = np_dweight(X, dY, Ind)
    return {"Y": Y, "Out": Out, "dY": dY, "dX": dX, "dWg": dWg, "dWs": dWs}


def rel_err(a, ref) -> float:
    """max|a - ref| / max|ref| : the error measure the parity tolerances are stated in."""
    a, ref = _f64(a), _f64(ref)
    denom = float(np.max(np.abs(ref))) if ref.size else 0.0
    if a.size == 0:
        return 0.0
    num = float(np.max(np.abs(a - ref)))
    return num / denom if denom > 0 else num
