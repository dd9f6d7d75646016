"""Bias epilogues: ExpertGather(bias=True) and ExpertScatter(bias=True) on the GPU against the CPU oracle plus the bias
terms written out in torch, forward and all gradients, on both kernel families."""
import pytest
import torch

import expertscattergather_b200 as egs
from expertscattergather_b200 import ops, workloads
from expertscattergather_b200.workloads import Workload
from gpu_util import tol_for
from oracle import egs_oracle as orc

pytestmark = pytest.mark.gpu

CASES = [
    ("f32-default-shape", Workload("b0", 8, 256, 32, 32, 128, 64, torch.float32, "distinct", 41), "auto"),
    ("f32-odd", Workload("b1", 3, 37, 5, 11, 27, 13, torch.float32, "replace", 42), "auto"),          # generic kernels
    ("bf16-collisions", Workload("b2", 4, 64, 16, 32, 128, 64, torch.bfloat16, "zipf", 43), "auto"),  # float32-row scatter
    ("bf16-persistent", Workload("b3", 40, 512, 16, 64, 128, 256, torch.bfloat16, "distinct", 44), "auto"),
    ("f16-generic", Workload("b4", 2, 40, 3, 16, 64, 32, torch.float16, "distinct", 45), "generic"),
]


def _reference(ins, bg, bs, T):
    """Oracle forward/backward with the bias terms added in plain torch (float64): gather bias broadcast over (b, k);
    scatter bias added per routed slot before scatter_add_."""
    X = ins["X"].double().requires_grad_(True)
    Wg = ins["Wg"].double().requires_grad_(True)
    Ws = ins["Ws"].double().requires_grad_(True)
    bg = bg.double().requires_grad_(True)
    bs = bs.double().requires_grad_(True)
    Ind = ins["Ind"]
    Y = orc.torch_gather(X, Wg, Ind) + bg                               # [B,E,K,J] + [E,1,J]
    B, E, K, J = Y.shape
    pre = torch.einsum("bekj,eji->beki", Y, Ws) + bs.unsqueeze(0)       # [B,E,K,I] + [1,E,1,I]
    out = torch.zeros(B, T, Ws.shape[-1], dtype=torch.float64)
    idx = Ind.to(torch.int64).unsqueeze(-1).expand(B, E, K, Ws.shape[-1]).reshape(B, E * K, -1)
    out = out.scatter_add(1, idx, pre.reshape(B, E * K, -1))
    (out * ins["G"].double()).sum().backward()
    return {"Y": Y.detach(), "Out": out.detach(), "dX": X.grad, "dWg": Wg.grad, "dWs": Ws.grad, "dbg": bg.grad, "dbs": bs.grad}


@pytest.mark.parametrize("label,w,path", CASES, ids=[c[0] for c in CASES])
def test_bias_modules_forward_and_gradients(cuda_device, label, w, path):
    ins = workloads.make_inputs(w)
    g = torch.Generator().manual_seed(w.seed)
    bg = (torch.randn(w.E, 1, w.J, generator=g) * 0.5).to(w.dtype)
    bs = (torch.randn(w.E, 1, w.I, generator=g) * 0.5).to(w.dtype)
    ref = _reference(ins, bg, bs, w.T)
    dev = cuda_device
    old = ops.get_path()
    ops.set_path(path)
    try:
        gm = egs.ExpertGather(w.E, w.I, w.J, bias=True).to(dev).to(w.dtype)
        sm = egs.ExpertScatter(w.E, w.J, w.I, bias=True).to(dev).to(w.dtype)
        with torch.no_grad():
            gm.W.copy_(ins["Wg"]); sm.W.copy_(ins["Ws"]); gm.bias.copy_(bg); sm.bias.copy_(bs)
        X = ins["X"].to(dev).requires_grad_(True)
        Ind = ins["Ind"].to(dev)
        ops.reset_status()
        Y = gm(X, Ind)
        Out = sm(Y, Ind, w.T)
        (Out.float() * ins["G"].to(dev).float()).sum().backward()
        torch.cuda.synchronize()
        ops.check_status()
    finally:
        ops.set_path(old)
    got = {"Y": Y, "Out": Out, "dX": X.grad, "dWg": gm.W.grad, "dWs": sm.W.grad, "dbg": gm.bias.grad, "dbs": sm.bias.grad}
    tol = tol_for(w.dtype, "strict")
    errs = {k: orc.rel_err(v.detach().cpu(), ref[k]) for k, v in got.items()}
    assert all(e <= tol for e in errs.values()), (label, errs)


def test_scatter_bias_reference_mode_is_the_broadcast_of_the_reference(cuda_device):
    """bias_mode='reference' evaluates `out + bias` as the reference writes it: defined when E == B (or 1), an error otherwise."""
    w = Workload("br", 4, 32, 4, 8, 32, 16, torch.float32, "distinct", 46)          # E == B
    ins = workloads.make_inputs(w)
    sm = egs.ExpertScatter(w.E, w.J, w.I, bias=True, bias_mode="reference").to(cuda_device)
    with torch.no_grad():
        sm.W.copy_(ins["Ws"])
    Y = orc.torch_gather(ins["X"], ins["Wg"], ins["Ind"])
    out = sm(Y.to(cuda_device), ins["Ind"].to(cuda_device), w.T)
    ref = orc.torch_scatter(Y, ins["Ws"], ins["Ind"], w.T) + sm.bias.detach().cpu()
    assert orc.rel_err(out.detach().cpu(), ref) <= 1e-5
    sm2 = egs.ExpertScatter(3, w.J, w.I, bias=True, bias_mode="reference").to(cuda_device)     # E = 3, B = 4: cannot broadcast
    Y3 = torch.zeros(4, 3, 8, w.J, device=cuda_device)
    with pytest.raises(RuntimeError):
        sm2(Y3, torch.zeros(4, 3, 8, dtype=torch.int64, device=cuda_device), w.T)
