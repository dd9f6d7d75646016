"""Router-side index preparation on the device - top-K routing, the token-major CSR, index compaction - and the scatter
variants that consume the CSR, each against a plain torch / numpy restatement."""
import numpy as np
import pytest
import torch

from expertscattergather_b200 import ops, workloads
from expertscattergather_b200.workloads import Workload
from gpu_util import to_dev, tol_for
from oracle import egs_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,T,E,K", [(3, 257, 5, 16), (2, 1024, 8, 64), (1, 40, 3, 40), (2, 5000, 2, 1024), (4, 64, 7, 1)])
@pytest.mark.parametrize("idx", [torch.int64, torch.int32, torch.int16])
def test_route_topk_matches_torch_topk(cuda_device, B, T, E, K, idx):
    g = torch.Generator().manual_seed(B * 1000 + T)
    scores = torch.randn(B, T, E, generator=g)                 # distinct with probability one
    Ind = ops.route_topk(scores.to(cuda_device), K, index_dtype=idx)
    ref = torch.topk(scores.permute(0, 2, 1), K, dim=-1).indices       # [B,E,K], best first
    assert Ind.dtype == idx and torch.equal(Ind.cpu().long(), ref)


def test_route_topk_breaks_ties_towards_the_lower_token(cuda_device):
    scores = torch.zeros(2, 50, 3)
    scores[:, 10:20, :] = 1.0                                           # ten equal best scores
    scores[0, 30, 1] = 2.0
    Ind = ops.route_topk(scores.to(cuda_device), 6).cpu()
    assert Ind[0, 0].tolist() == [10, 11, 12, 13, 14, 15]
    assert Ind[0, 1].tolist() == [30, 10, 11, 12, 13, 14]
    with pytest.raises(ValueError):
        ops.route_topk(scores.to(cuda_device), 51)                      # K > T


@pytest.mark.parametrize("index", ["distinct", "replace", "zipf"])
def test_index_csr_is_the_counting_sort_of_ind(cuda_device, index):
    w = Workload("csr", 5, 300, 12, 24, 16, 16, torch.float32, index, 61)
    Ind = workloads.make_inputs(w)["Ind"]
    csr = ops.build_index_csr(Ind.to(cuda_device), w.T)
    flat = (Ind + torch.arange(w.B).view(-1, 1, 1) * w.T).reshape(-1)          # token row of every slot
    counts = torch.bincount(flat, minlength=w.B * w.T)
    assert torch.equal(csr.counts.cpu().long(), counts)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)])
    assert torch.equal(csr.offsets.cpu().long(), offsets)
    order = torch.sort(flat, stable=True).indices                                # slots grouped by row, ascending inside
    assert torch.equal(csr.entries.cpu().long(), order)
    s = csr.summary()
    assert s == {"max_per_row": int(counts.max()), "rows_touched": int((counts > 0).sum()), "out_of_range": False,
                 "valid_slots": w.B * w.E * w.K}


def test_index_csr_leaves_out_and_reports_bad_ids(cuda_device):
    Ind = torch.tensor([[[0, 5, 99], [2, -1, 5]]])                               # B=1, E=2, K=3, T=6
    csr = ops.build_index_csr(Ind.to(cuda_device), 6)
    assert csr.summary() == {"max_per_row": 2, "rows_touched": 3, "out_of_range": True, "valid_slots": 4}
    assert csr.counts.cpu().tolist() == [1, 0, 1, 0, 0, 2]
    assert csr.entries.cpu()[:4].tolist() == [0, 3, 1, 5]


def test_compact_index(cuda_device):
    Ind = torch.randint(0, 300, (3, 4, 5))
    for dt in (torch.int16, torch.int32, torch.int64):
        out = ops.compact_index(Ind.to(cuda_device), 300, dt)
        assert out.dtype == dt and torch.equal(out.cpu().long(), Ind)
    with pytest.raises(ValueError):
        ops.compact_index(Ind.to(cuda_device), 40000, torch.int16)               # T does not fit int16
    ops.reset_status()
    ops.compact_index(Ind.to(cuda_device), 200, torch.int32)                     # some ids >= T
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="outside"):
        ops.check_status()


@pytest.mark.parametrize("dtype,index,layout", [(torch.float32, "distinct", "cn"), (torch.float32, "zipf", "nc"),
                                                (torch.bfloat16, "replace", "cn"), (torch.float16, "zipf", "cn")])
def test_csr_scatter_matches_oracle_and_is_reproducible(cuda_device, dtype, index, layout):
    w = Workload("csrs", 4, 96, 10, 20, 40, 72, dtype, index, 67)
    ins = workloads.make_inputs(w)
    d = to_dev(ins, cuda_device)
    Y = orc.torch_gather(ins["X"], ins["Wg"], ins["Ind"])                        # [B,E,K,J]
    csr = ops.build_index_csr(d["Ind"], w.T)
    Wdev = d["Ws"] if layout == "cn" else d["Ws"].transpose(1, 2).contiguous()
    out1 = ops.gemm_scatter_csr(Y.to(cuda_device), Wdev, csr, w_layout=layout)
    out2 = ops.gemm_scatter_csr(Y.to(cuda_device), Wdev, csr, w_layout=layout)
    assert torch.equal(out1, out2)                                               # fixed summation order: same bits
    ref = orc.np_scatter(Y, ins["Ws"], ins["Ind"], w.T)
    assert orc.rel_err(out1.cpu(), ref) <= tol_for(dtype, "strict")
    # rows nothing is routed to are stored as zeros (the output was torch.empty)
    untouched = csr.counts.view(w.B, w.T) == 0
    assert float(out1[untouched].abs().max()) == 0.0 if bool(untouched.any()) else True
    # bias per routed slot and accumulation into a given output
    bias = torch.randn(w.E, 1, w.I).to(dtype)
    base = torch.ones_like(out1)
    out3 = ops.gemm_scatter_csr(Y.to(cuda_device), Wdev, csr, w_layout=layout, out=base, bias=bias.to(cuda_device))
    cnt = torch.zeros(w.B, w.T, w.E, dtype=torch.float64)
    bidx = torch.arange(w.B).view(-1, 1, 1).expand_as(ins["Ind"])
    eidx = torch.arange(w.E).view(1, -1, 1).expand_as(ins["Ind"])
    cnt.index_put_((bidx.reshape(-1), ins["Ind"].reshape(-1), eidx.reshape(-1)), torch.ones(ins["Ind"].numel(), dtype=torch.float64),
                   accumulate=True)
    ref3 = ref + 1.0 + torch.einsum("bte,ei->bti", cnt, bias.double().reshape(w.E, w.I)).numpy()
    assert orc.rel_err(out3.cpu(), ref3) <= tol_for(dtype, "strict")


def test_scatter_takes_its_plan_from_a_prepared_csr(cuda_device):
    """The 16-bit scatter with csr=... must equal the one that counts for itself, in both regimes (few contributions per
    row: direct 16-bit additions; a Zipf index: float32 rows)."""
    for index in ("distinct", "zipf"):
        w = Workload("prep", 4, 256, 48, 32, 64, 128, torch.bfloat16, index, 71)
        d = to_dev(workloads.make_inputs(w), cuda_device)
        Y = ops.gather_gemm(d["X"], d["Wg"], d["Ind"])
        csr = ops.build_index_csr(d["Ind"], w.T)
        a = ops.gemm_scatter(Y, d["Ws"], d["Ind"], w.T)
        b = ops.gemm_scatter(Y, d["Ws"], d["Ind"], w.T, csr=csr)
        ref = orc.np_scatter(Y.cpu(), d["Ws"].cpu(), d["Ind"].cpu(), w.T)
        # (direct 16-bit additions round in the order they happen to run in: both against the float64 truth)
        assert orc.rel_err(a.cpu(), ref) <= 3e-2 and orc.rel_err(b.cpu(), ref) <= 3e-2
        flat = (d["Ind"].cpu() + torch.arange(w.B).view(-1, 1, 1) * w.T).reshape(-1)
        heaviest = int(torch.bincount(flat).max())
        assert csr.summary()["max_per_row"] == heaviest
        assert (heaviest > 32) == (index == "zipf"), heaviest      # the two cases sit on either side of the 32-per-row switch
