"""``ExpertGather`` and ``ExpertScatter``: parameter holders over the autograd functions.

Drop-in for the reference's ``egs/torch_interface.py`` (constructor arguments, parameter names ``W`` and
``bias``, shapes, initialisation and forward signatures are the same, so state dicts interchange).
Deviations: the optional bias is tested with ``is not None`` (the reference's ``if self.bias:`` raises for any
multi-element bias, ``egs/torch_interface.py:55,111``), the constructor does not query a CUDA device (the
reference's Volta check at ``:23-33`` fails on a host without a GPU), and ``.to()`` is the standard
``nn.Module.to`` (the reference re-wraps the parameters, ``:59-63``).
"""
from __future__ import annotations

import math

import torch
from torch import nn

from .kernels import (ExpertGatherBiasFunction, ExpertGatherFunction, ExpertGatherScatterFunction, ExpertScatterBiasFunction,
                      ExpertScatterFunction, create_kernels)

__all__ = ["ExpertGather", "ExpertScatter", "ExpertGatherScatter"]


class ExpertGather(nn.Module):
    """Gathers the K tokens routed to each expert and multiplies them by that expert's weights.

    ``forward(x [B,T,I], Ind [B,E,K]) -> [B,E,K,J]``   (reference: ``egs/torch_interface.py:11-57``)
    """

    def __init__(self, E: int, I: int, J: int, bias: bool = False):
        super().__init__()
        self.E, self.I, self.J = E, I, J
        self.W = nn.Parameter(torch.empty(E, I, J))
        if bias:
            self.bias = nn.Parameter(torch.empty(E, 1, J))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()
        create_kernels()

    def reset_parameters(self) -> None:
        bound = 1 / math.sqrt(self.I)
        nn.init.uniform_(self.W, -bound, bound)
        if self.bias is not None:
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, x: torch.Tensor, Ind: torch.Tensor) -> torch.Tensor:
        if self.bias is not None:
            # y + bias ([E,1,J] broadcast over batch and slot, the reference's expression at :55-56), fused into the kernel
            return ExpertGatherBiasFunction.apply(x, self.W, self.bias, Ind)
        return ExpertGatherFunction.apply(x, self.W, Ind)


class ExpertScatter(nn.Module):
    """Multiplies each expert's K rows by that expert's weights and adds them back at their token positions.

    ``forward(Y [B,E,K,J], Ind [B,E,K], T) -> [B,T,I]``   (reference: ``egs/torch_interface.py:66-113``)
    The initialisation bound uses ``1/sqrt(I)`` like the reference does (``:93``), although J is the fan-in.

    Bias ([E,1,I], the reference's parameter shape).  The reference adds it to the scattered output with ``out + self.bias``
    (``:111``), an expression that only broadcasts against ``[B,T,I]`` when E is 1 or B and then pairs expert e with batch
    element e.  ``bias_mode="per_slot"`` (default) gives the parameter a meaning for every shape: each routed slot of
    expert e contributes ``Y[b,e,k,:] @ W[e] + bias[e]`` to its token row (fused into the scatter kernel).
    ``bias_mode="reference"`` evaluates the reference's expression as it stands (and raises where it cannot broadcast).
    """

    def __init__(self, E: int, J: int, I: int, bias: bool = False, bias_mode: str = "per_slot"):
        super().__init__()
        if bias_mode not in ("per_slot", "reference"):
            raise ValueError("bias_mode must be 'per_slot' or 'reference'")
        self.bias_mode = bias_mode
        self.E, self.J, self.I = E, J, I
        self.W = nn.Parameter(torch.empty(E, J, I))
        if bias:
            self.bias = nn.Parameter(torch.empty(E, 1, I))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()
        create_kernels()

    def reset_parameters(self) -> None:
        bound = 1 / math.sqrt(self.I)
        nn.init.uniform_(self.W, -bound, bound)
        if self.bias is not None:
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, Y: torch.Tensor, Ind: torch.Tensor, T: int) -> torch.Tensor:
        if self.bias is not None and self.bias_mode == "per_slot":
            return ExpertScatterBiasFunction.apply(Y, self.W, self.bias, Ind, T)
        out = ExpertScatterFunction.apply(Y, self.W, Ind, T)
        if self.bias is not None:
            out = out + self.bias   # the reference's expression: broadcasts only when E == B or E == 1
        return out


class ExpertGatherScatter(nn.Module):
    """The gather -> scatter block of a model as one module: ``forward(x [B,T,I], Ind [B,E,K]) -> [B,T,I]``, equal to
    ``scatter(gather(x, Ind), Ind, T)`` of an ``ExpertGather(E, I, J)`` and an ``ExpertScatter(E, J, I)`` (the usage
    the reference's ``README.md:23-32`` shows).  The two sub-modules are ordinary ``ExpertGather`` / ``ExpertScatter``
    instances (``.gather``, ``.scatter``), so their state dicts interchange with separately built ones.

    Without biases the block runs as one autograd node (``ExpertGatherScatterFunction``), which uses the fused
    kernel where it applies; with a bias on either side it falls back to calling the two sub-modules.
    No counterpart class in the reference.
    """

    def __init__(self, E: int, I: int, J: int, bias: bool = False):
        super().__init__()
        self.gather = ExpertGather(E, I, J, bias=bias)
        self.scatter = ExpertScatter(E, J, I, bias=bias)

    def forward(self, x: torch.Tensor, Ind: torch.Tensor) -> torch.Tensor:
        if self.gather.bias is not None or self.scatter.bias is not None:
            return self.scatter(self.gather(x, Ind), Ind, x.shape[1])
        return ExpertGatherScatterFunction.apply(x, self.gather.W, self.scatter.W, Ind)
