"""Host-side mirror of the reference interface, workload generators and byte accounting (CPU only)."""
import sys

import pytest
import torch

import expertscattergather_b200 as egs
from expertscattergather_b200 import kernels, ops, workloads
from expertscattergather_b200.distributed import shard_bounds


def test_modules_have_the_reference_parameters():
    g = egs.ExpertGather(3, 8, 4)
    s = egs.ExpertScatter(3, 4, 8, bias=True)
    assert list(g.state_dict()) == ["W"] and tuple(g.W.shape) == (3, 8, 4) and g.bias is None
    assert sorted(s.state_dict()) == ["W", "bias"] and tuple(s.W.shape) == (3, 4, 8) and tuple(s.bias.shape) == (3, 1, 8)
    bound = 1 / 8 ** 0.5
    assert float(g.W.detach().abs().max()) <= bound and float(s.W.detach().abs().max()) <= bound


def test_ops_are_registered_with_the_reference_schemas():
    kernels.create_kernels()
    ns = getattr(torch.ops, kernels.OP_NAMESPACE)
    for name in ("expert_gather_forward_call_fn", "expert_gather_backward_call_fn",
                 "expert_scatter_forward_call_fn", "expert_scatter_backward_call_fn"):
        assert hasattr(ns, name)
    assert kernels.expert_gather_forward_call is ns.expert_gather_forward_call_fn
    kernels.create_kernels()  # second call is a no-op (re-defining the ops would raise)


def test_fake_impls_propagate_shapes():
    kernels.create_kernels()
    with torch._subclasses.FakeTensorMode():
        X = torch.empty(2, 9, 8)
        W = torch.empty(3, 8, 4)
        Ind = torch.empty(2, 3, 5, dtype=torch.int64)
        Y = kernels.expert_gather_forward_call(X, W, Ind, torch.float32)
        assert tuple(Y.shape) == (2, 3, 5, 4)
        Ws = torch.empty(3, 4, 8)
        Out = kernels.expert_scatter_forward_call(Y, Ws, Ind, 9, torch.float32)
        assert tuple(Out.shape) == (2, 9, 8)
        gX, gW = kernels.expert_gather_backward_call(X, W, Ind, Y, torch.float32)
        assert gX.shape == X.shape and gW.shape == W.shape
        gY, gWs = kernels.expert_scatter_backward_call(Y, Ws, Ind, Out, torch.float32)
        assert gY.shape == Y.shape and gWs.shape == Ws.shape


def test_unknown_dtype_raises_like_the_reference():
    assert [ops.dtype_to_type_id(d) for d in (torch.float32, torch.float16, torch.bfloat16)] == [0, 1, 2]
    with pytest.raises(ValueError, match="Unknown dtype"):
        ops.dtype_to_type_id(torch.float64)


def test_cpu_tensors_are_refused():
    g = egs.ExpertGather(2, 4, 4)
    with pytest.raises(RuntimeError, match="no CPU path"):
        g(torch.randn(1, 3, 4), torch.zeros(1, 2, 2, dtype=torch.int64))
    with pytest.raises(ValueError):
        ops.gather_gemm(torch.randn(3, 4), torch.randn(2, 4, 4), torch.zeros(1, 2, 2, dtype=torch.int64))


def test_install_as_egs_aliases():
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "egs" or k.startswith("egs.")}
    try:
        egs.install_as_egs()
        from egs import ExpertGather  # noqa
        from egs.triton_kernels import ExpertGatherFunction, create_kernels  # noqa
        assert ExpertGather is egs.ExpertGather
    finally:
        for k in [k for k in sys.modules if k == "egs" or k.startswith("egs.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_precision_and_path_switches():
    old_p, old_k = ops.get_precision(), ops.get_path()
    try:
        ops.set_precision("tf32"); ops.set_path("generic")
        assert ops.get_precision() == "tf32" and ops.get_path() == "generic"
        with pytest.raises(ValueError):
            ops.set_precision("fp8")
        with pytest.raises(ValueError):
            ops.set_path("cpu")
    finally:
        ops.set_precision(old_p); ops.set_path(old_k)


def test_index_generators():
    g = torch.Generator().manual_seed(1)
    ind = workloads.indices_distinct(3, 4, 5, 9, g)
    assert ind.shape == (3, 4, 5) and int(ind.min()) >= 0 and int(ind.max()) < 9
    assert all(len(set(ind[b, e].tolist())) == 5 for b in range(3) for e in range(4))
    z = workloads.indices_zipf(2, 6, 4, 64, g)
    assert all(len(set(z[b, e].tolist())) == 4 for b in range(2) for e in range(6))
    # skew: the most popular token is picked by many experts
    big = workloads.indices_zipf(1, 128, 8, 256, g)
    assert int(torch.bincount(big.flatten(), minlength=256).max()) > 40
    r = workloads.indices_with_replacement(2, 3, 50, 4, g)
    assert r.dtype == torch.int16 and int(r.max()) < 4


def test_make_inputs_prefix_property_and_dtypes():
    w = workloads.WORKLOADS["cfg1-T256"]
    a = workloads.make_inputs(w, B=2)
    b = workloads.make_inputs(w, B=3)
    assert torch.equal(a["X"], b["X"][:2]) and torch.equal(a["Ind"], b["Ind"][:2]) and torch.equal(a["Wg"], b["Wg"])
    assert a["X"].dtype == torch.float32 and a["Ind"].dtype == torch.int64
    c = workloads.make_inputs(workloads.WORKLOADS["cfg2"].with_batch(1))
    assert c["X"].dtype == torch.bfloat16 and tuple(c["Ind"].shape) == (1, 256, 16)
    i = workloads.make_inputs(w, B=1, integer_valued=True)
    assert torch.equal(i["X"], i["X"].round()) and float(i["X"].abs().max()) <= 2


def test_algorithmic_work_matches_the_published_floors():
    w0 = workloads.WORKLOADS["cfg0"]
    a = workloads.algorithmic_work(w0)
    assert a["flops"] == 12 * 65536 * 128 * 64
    assert abs(a["bytes"] / 1e6 - 133.9) < 1.5
    for name, mb in (("cfg1-T256", 38.2), ("cfg1-T1024", 60.6), ("cfg1-T4096", 117.2), ("cfg1-T16384", 320.6)):
        assert abs(workloads.algorithmic_work(workloads.WORKLOADS[name])["bytes"] / 1e6 - mb) < 0.02 * mb + 0.5
    w3 = workloads.WORKLOADS["cfg3"]
    assert abs(workloads.algorithmic_work(w3)["bytes"] / 1e6 - 1475) < 30
    ind = workloads.make_inputs(w0, B=2)["Ind"]
    exact = workloads.algorithmic_work(w0, Ind=ind, B=2)
    assert exact["U"] == int(torch.unique(ind + torch.arange(2).view(2, 1, 1) * w0.T).numel())


def test_shard_bounds_cover_the_batch():
    for B in (1, 7, 64, 512):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(B, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))


def test_gather_scatter_block_holds_the_two_reference_modules():
    """The fused block's parameters are those of an ExpertGather and an ExpertScatter, so state dicts interchange."""
    import expertscattergather_b200 as egs
    blk = egs.ExpertGatherScatter(3, 16, 8)
    g, s = egs.ExpertGather(3, 16, 8), egs.ExpertScatter(3, 8, 16)
    assert sorted(blk.state_dict()) == ["gather.W", "scatter.W"]
    blk.gather.load_state_dict(g.state_dict())
    blk.scatter.load_state_dict(s.state_dict())
    assert tuple(blk.gather.W.shape) == (3, 16, 8) and tuple(blk.scatter.W.shape) == (3, 8, 16)
    with_bias = egs.ExpertGatherScatter(3, 16, 8, bias=True)
    assert sorted(with_bias.state_dict()) == ["gather.W", "gather.bias", "scatter.W", "scatter.bias"]
