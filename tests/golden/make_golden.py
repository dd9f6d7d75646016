"""Generates the golden vectors under tests/golden/ by running the REFERENCE's own torch modules.

Usage (in a container that has the reference checked out; it cannot run where the reference is absent):

    python tests/golden/make_golden.py /path/to/ExpertScatterGather

It imports ``egs.baselines`` from that path (``TorchReshapedGatherEinsum``, ``egs/baselines.py:62-79``
and ``TorchEinsumScatter``, ``egs/baselines.py:167-187`` - the classes the reference's tests compare its
kernels against), feeds them explicit seeded inputs, and stores inputs and outputs as float32 / int64
arrays in one ``.npz`` per case.  bf16 cases store the bf16 values widened to float32 (exact).
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name: (B, T, E, K, I, J, dtype, index mode, value mode)
CASES = {
    "odd_small_f32": (3, 17, 5, 7, 12, 9, torch.float32, "replace", "normal"),
    "ones_dims_f32": (1, 1, 1, 1, 1, 1, torch.float32, "replace", "normal"),
    "mini_cfg0_f32": (2, 32, 4, 8, 16, 8, torch.float32, "distinct", "normal"),
    "aligned_f32": (2, 64, 3, 40, 32, 16, torch.float32, "distinct", "normal"),
    "integer_exact_f32": (2, 24, 3, 10, 16, 8, torch.float32, "replace", "integer"),
    "heavy_collision_f32": (2, 4, 6, 9, 8, 8, torch.float32, "replace", "normal"),
    "mini_bf16": (2, 32, 4, 8, 16, 8, torch.bfloat16, "distinct", "normal"),
    "integer_exact_bf16": (2, 24, 3, 10, 16, 8, torch.bfloat16, "replace", "integer"),
}


def build_inputs(name):
    B, T, E, K, I, J, dtype, imode, vmode = CASES[name]
    g = torch.Generator().manual_seed(sum(map(ord, name)) * 7919)
    if vmode == "integer":
        X = torch.randint(-2, 3, (B, T, I), generator=g).float()
        Wg = torch.randint(-1, 2, (E, I, J), generator=g).float()
        Ws = torch.randint(-1, 2, (E, J, I), generator=g).float()
        G = torch.randint(-1, 2, (B, T, I), generator=g).float()
        GY = torch.randint(-1, 2, (B, E, K, J), generator=g).float()
        Yin = torch.randint(-2, 3, (B, E, K, J), generator=g).float()
    else:
        X = torch.randn(B, T, I, generator=g)
        Wg = torch.randn(E, I, J, generator=g) / I ** 0.5
        Ws = torch.randn(E, J, I, generator=g) / J ** 0.5
        G = torch.randn(B, T, I, generator=g)
        GY = torch.randn(B, E, K, J, generator=g)
        Yin = torch.randn(B, E, K, J, generator=g)
    if imode == "distinct":
        Ind = torch.rand(B, E, T, generator=g).argsort(-1)[..., :K].contiguous()
    else:
        Ind = torch.randint(0, T, (B, E, K), generator=g)
    cast = lambda t: t.to(dtype)
    return dict(X=cast(X), Wg=cast(Wg), Ws=cast(Ws), G=cast(G), GY=cast(GY), Yin=cast(Yin), Ind=Ind, T=T)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from egs.baselines import TorchEinsumScatter, TorchReshapedGatherEinsum  # noqa: E402 (the reference)

    for name in CASES:
        B, T, E, K, I, J, dtype, _, _ = CASES[name]
        d = build_inputs(name)
        out = {}
        # (1) gather module alone, loss = sum(Y*GY)
        gm = TorchReshapedGatherEinsum(E, I, J)
        gm.W = torch.nn.Parameter(d["Wg"].clone())
        X = d["X"].clone().requires_grad_(True)
        Y = gm(X, d["Ind"])
        (Y * d["GY"]).sum().backward()
        out.update(g_Y=Y.detach(), g_dX=X.grad, g_dW=gm.W.grad)
        # (2) scatter module alone, loss = sum(Out*G)
        sm = TorchEinsumScatter(E, J, I)
        sm.W = torch.nn.Parameter(d["Ws"].clone())
        Yin = d["Yin"].clone().requires_grad_(True)
        O = sm(Yin, d["Ind"], T)
        (O * d["G"]).sum().backward()
        out.update(s_Out=O.detach(), s_dY=Yin.grad, s_dW=sm.W.grad)
        # (3) the full step gather -> scatter -> sum(Out*G)
        gm2 = TorchReshapedGatherEinsum(E, I, J)
        gm2.W = torch.nn.Parameter(d["Wg"].clone())
        sm2 = TorchEinsumScatter(E, J, I)
        sm2.W = torch.nn.Parameter(d["Ws"].clone())
        X2 = d["X"].clone().requires_grad_(True)
        Y2 = gm2(X2, d["Ind"])
        O2 = sm2(Y2, d["Ind"], T)
        (O2 * d["G"]).sum().backward()
        out.update(f_Y=Y2.detach(), f_Out=O2.detach(), f_dX=X2.grad, f_dWg=gm2.W.grad, f_dWs=sm2.W.grad)

        arrays = {"dtype": np.array(str(dtype).replace("torch.", "")), "T": np.array(T)}
        for k in ("X", "Wg", "Ws", "G", "GY", "Yin"):
            arrays["in_" + k] = d[k].float().numpy()
        arrays["in_Ind"] = d["Ind"].numpy().astype(np.int64)
        for k, v in out.items():
            arrays["ref_" + k] = v.detach().float().numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(f"{name}: wrote {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
