"""Seeded synthetic inputs for the expert gather/scatter path.

The generators run on the CPU with an explicit ``torch.Generator`` so that a CPU checker and the
GPU path can be fed identical bits.  Shapes, dtypes and index distributions are those of the five
benchmark configurations of this build; the extra ``randint`` generator reproduces the index
distribution of the reference's own tests (``test_all.py:16``: with replacement, int16).
"""
from __future__ import annotations

import dataclasses
import math

import torch

__all__ = ["Workload", "WORKLOADS", "make_inputs", "indices_distinct", "indices_zipf",
           "indices_with_replacement", "algorithmic_work"]


@dataclasses.dataclass(frozen=True)
class Workload:
    name: str
    B: int
    T: int
    E: int
    K: int
    I: int
    J: int
    dtype: torch.dtype
    index: str = "distinct"      # "distinct" | "zipf" | "replace"
    seed: int = 1234

    @property
    def routed(self) -> int:
        """Routed token slots per step, N = B*E*K (the unit of the throughput metric)."""
        return self.B * self.E * self.K

    def with_batch(self, B: int) -> "Workload":
        return dataclasses.replace(self, B=B)


def _cfg1(T: int, k: int) -> Workload:
    return Workload(f"cfg1-T{T}", 16, T, 32, 32, 128, 64, torch.float32, "distinct", 1235 + 16 * k)


WORKLOADS = {
    "cfg0": Workload("cfg0", 64, 256, 32, 32, 128, 64, torch.float32, "distinct", 1234),
    "cfg1-T256": _cfg1(256, 0),
    "cfg1-T1024": _cfg1(1024, 1),
    "cfg1-T4096": _cfg1(4096, 2),
    "cfg1-T16384": _cfg1(16384, 3),
    "cfg2": Workload("cfg2", 32, 1024, 256, 16, 512, 128, torch.bfloat16, "zipf", 1236),
    "cfg3": Workload("cfg3", 8, 2048, 64, 128, 2048, 512, torch.bfloat16, "distinct", 1237),
    "cfg4": Workload("cfg4", 512, 1024, 64, 64, 1024, 256, torch.bfloat16, "distinct", 1238),
}
CFG1_SWEEP = ("cfg1-T256", "cfg1-T1024", "cfg1-T4096", "cfg1-T16384")


def indices_distinct(B, E, K, T, gen) -> torch.Tensor:
    """For each (b,e): K distinct tokens uniform in [0,T).  Different experts may pick the same token."""
    if K > T:
        raise ValueError("distinct indices need K <= T")
    # chunk over B to bound the [B,E,T] random block
    out = torch.empty(B, E, K, dtype=torch.int64)
    step = max(1, (1 << 24) // max(1, E * T))
    for b0 in range(0, B, step):
        b1 = min(B, b0 + step)
        out[b0:b1] = torch.rand(b1 - b0, E, T, generator=gen).argsort(-1)[..., :K]
    return out


def indices_zipf(B, E, K, T, gen, s: float = 1.1) -> torch.Tensor:
    """Per batch element a Zipf(s) popularity over a random permutation of the tokens; per expert K
    distinct tokens drawn from it without replacement (skewed: hot tokens collide heavily)."""
    out = torch.empty(B, E, K, dtype=torch.int64)
    base = torch.arange(1, T + 1, dtype=torch.float64).pow(-s)
    for b in range(B):
        perm = torch.randperm(T, generator=gen)
        p = torch.empty(T, dtype=torch.float64)
        p[perm] = base
        out[b] = torch.multinomial(p.expand(E, T), K, replacement=False, generator=gen)
    return out


def indices_with_replacement(B, E, K, T, gen, dtype=torch.int16) -> torch.Tensor:
    """``torch.randint(0, T)``: duplicates may occur inside one (b,e) as well (``test_all.py:16``)."""
    return torch.randint(0, T, (B, E, K), generator=gen).to(dtype)


def make_inputs(w: Workload, B: int | None = None, integer_valued: bool = False, b0: int = 0):
    """Returns dict(X, Wg, Ws, Ind, G) on the CPU in ``w.dtype``.

    ``b0`` is the global index of the first batch element to generate (a rank's slice of a sharded batch):
    batch elements b0 .. b0+B-1 of the full workload are produced.

    ``B`` overrides the batch (a prefix-independent slice for CPU checks: each batch element is
    generated from its own sub-seed so a smaller B yields the same leading batch elements).
    ``integer_valued`` draws small integers instead of normals so that every sum is exact in fp32
    and the result is independent of the accumulation order (bit-exact index tests).
    """
    B = w.B if B is None else B
    gw = torch.Generator().manual_seed(w.seed)
    if integer_valued:
        Wg = torch.randint(-1, 2, (w.E, w.I, w.J), generator=gw).float()
        Ws = torch.randint(-1, 2, (w.E, w.J, w.I), generator=gw).float()
    else:
        Wg = torch.randn(w.E, w.I, w.J, generator=gw) / math.sqrt(w.I)
        Ws = torch.randn(w.E, w.J, w.I, generator=gw) / math.sqrt(w.J)
    X = torch.empty(B, w.T, w.I)
    G = torch.empty(B, w.T, w.I)
    Ind = torch.empty(B, w.E, w.K, dtype=torch.int64)
    for b in range(B):
        gb = torch.Generator().manual_seed(w.seed * 100003 + b0 + b)
        if integer_valued:
            X[b] = torch.randint(-2, 3, (w.T, w.I), generator=gb).float()
            G[b] = torch.randint(-1, 2, (w.T, w.I), generator=gb).float()
        else:
            X[b] = torch.randn(w.T, w.I, generator=gb)
            G[b] = torch.randn(w.T, w.I, generator=gb)
        if w.index == "distinct":
            Ind[b] = indices_distinct(1, w.E, w.K, w.T, gb)[0]
        elif w.index == "zipf":
            Ind[b] = indices_zipf(1, w.E, w.K, w.T, gb)[0]
        elif w.index == "replace":
            Ind[b] = indices_with_replacement(1, w.E, w.K, w.T, gb, torch.int64)[0]
        else:
            raise ValueError(w.index)
    d = w.dtype
    return {"X": X.to(d), "Wg": Wg.to(d), "Ws": Ws.to(d), "Ind": Ind, "G": G.to(d)}


def algorithmic_work(w: Workload, Ind: torch.Tensor | None = None, B: int | None = None):
    """Algorithmic FLOPs and bytes of one full step (gather fwd, scatter fwd, both backwards).

    FLOPs = 12*N*I*J (six contractions of 2*N*I*J).  Bytes count every tensor once per operator
    pair that needs it and no intermediate: U = number of distinct (b,t) rows referenced by Ind
    (exact if Ind is given, else its expectation for uniform draws), s = element size, 8-byte ids.
    """
    B = w.B if B is None else B
    s = torch.empty((), dtype=w.dtype).element_size()
    N = B * w.E * w.K
    if Ind is not None:
        flat = Ind.to(torch.int64) + (torch.arange(Ind.shape[0]).view(-1, 1, 1) * w.T)
        U = int(torch.unique(flat).numel())
    else:
        U = int(round(B * w.T * (1.0 - (1.0 - w.K / w.T) ** w.E)))
    WB = w.E * w.I * w.J * s
    g_fwd = U * w.I * s + WB + 8 * N + N * w.J * s
    s_fwd = N * w.J * s + WB + 8 * N + B * w.T * w.I * s
    s_bwd = U * w.I * s + N * w.J * s + WB + 8 * N + N * w.J * s + WB
    g_bwd = N * w.J * s + U * w.I * s + WB + 8 * N + B * w.T * w.I * s + WB
    return {"flops": 12 * N * w.I * w.J, "bytes": g_fwd + s_fwd + s_bwd + g_bwd, "U": U, "N": N,
            "parts": {"gather_fwd": g_fwd, "scatter_fwd": s_fwd, "scatter_bwd": s_bwd, "gather_bwd": g_bwd}}
