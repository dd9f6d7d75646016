"""The modules under torch.compile (the dispatcher ops carry fake implementations so that a compiled graph can trace through
them, as the reference's do, egs/triton_kernels.py:527-567) and under CUDA-graph capture (forward + backward, helper
streams included), both against the CPU oracle."""
import pytest
import torch

import expertscattergather_b200 as egs
from expertscattergather_b200 import ops, workloads
from expertscattergather_b200.workloads import Workload
from gpu_util import tol_for
from oracle import egs_oracle as orc

pytestmark = pytest.mark.gpu


def _modules(w, ins, dev):
    g = egs.ExpertGather(w.E, w.I, w.J).to(dev).to(w.dtype)
    s = egs.ExpertScatter(w.E, w.J, w.I).to(dev).to(w.dtype)
    with torch.no_grad():
        g.W.copy_(ins["Wg"]); s.W.copy_(ins["Ws"])
    return g, s


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_modules_compile_with_fullgraph(cuda_device, dtype):
    """torch.compile(fullgraph=True) over gather -> scatter -> loss: tracing must get through the autograd Functions and the
    four dispatcher ops without a graph break (backend aot_eager: the traced forward and backward graphs run through the
    ops' real implementations; no code generation is involved)."""
    w = Workload("cmp", 4, 64, 6, 16, 64, 32, dtype, "distinct", 51)
    ins = workloads.make_inputs(w)
    ref = orc.torch_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
    g, s = _modules(w, ins, cuda_device)

    def block(x, ind, grad):
        return (s(g(x, ind), ind, w.T).float() * grad.float()).sum()

    compiled = torch.compile(block, fullgraph=True, backend="aot_eager")
    X = ins["X"].to(cuda_device).requires_grad_(True)
    ops.reset_status()
    loss = compiled(X, ins["Ind"].to(cuda_device), ins["G"].to(cuda_device))
    loss.backward()
    torch.cuda.synchronize()
    ops.check_status()
    tol = tol_for(dtype, "strict")
    assert orc.rel_err(X.grad.cpu(), ref["dX"]) <= tol
    assert orc.rel_err(g.W.grad.cpu(), ref["dWg"]) <= tol
    assert orc.rel_err(s.W.grad.cpu(), ref["dWs"]) <= tol
    ref_loss = float((ref["Out"].double() * ins["G"].double()).sum())
    assert abs(float(loss.detach()) - ref_loss) <= tol * max(1.0, float((ref["Out"].double() * ins["G"].double()).abs().sum()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_modules_forward_and_backward_in_a_cuda_graph(cuda_device, dtype):
    """Forward + backward of the modules captured once and replayed on new input values: the helper streams the backward
    pass uses (weight gradients beside dX / dY) fork from and join the capturing stream, so the whole step lands in the graph."""
    w = Workload("cg", 6, 128, 8, 32, 128, 64, dtype, "distinct", 53)
    ins = workloads.make_inputs(w)
    g, s = _modules(w, ins, cuda_device)
    x_static = torch.zeros_like(ins["X"], device=cuda_device).requires_grad_(True)
    ind = ins["Ind"].to(cuda_device)
    grad = ins["G"].to(cuda_device)

    def step():
        g.W.grad = None; s.W.grad = None; x_static.grad = None
        out = s(g(x_static, ind), ind, w.T)
        (out.float() * grad.float()).sum().backward()
        return out

    side = torch.cuda.Stream(cuda_device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = step()
    grads = (x_static.grad, g.W.grad, s.W.grad)
    tol = tol_for(dtype, "strict")
    for trial in range(2):                           # two different inputs through the same graph
        Xv = ins["X"] if trial == 0 else torch.roll(ins["X"], 1, 0)
        ref = orc.torch_step(Xv, ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
        with torch.no_grad():
            x_static.copy_(Xv.to(cuda_device))
        graph.replay()
        torch.cuda.synchronize()
        ops.check_status()
        assert orc.rel_err(out.detach().cpu(), ref["Out"]) <= tol
        assert orc.rel_err(grads[0].cpu(), ref["dX"]) <= tol
        assert orc.rel_err(grads[1].cpu(), ref["dWg"]) <= tol
        assert orc.rel_err(grads[2].cpu(), ref["dWs"]) <= tol
