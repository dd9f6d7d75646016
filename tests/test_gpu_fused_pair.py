"""The fused pair kernel (gather-GEMM whose output tile feeds the GEMM-scatter without leaving the SM) against the
CPU oracle and against the two separate operators.  Called through the C ABI (egs_gather_scatter_pair)."""
import numpy as np
import pytest
import torch

from expertscattergather_b200 import ops, workloads
from expertscattergather_b200.workloads import Workload
from gpu_util import compare_step, gpu_step, to_dev, tol_for
from oracle import egs_oracle as orc

pytestmark = pytest.mark.gpu


def _pair_both_ways(d, precision):
    """Forward pair (X -> Y -> Out) and backward pair (G -> dY -> dX) through the fused kernel."""
    Y, Out = ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], d["Ind"], w_layout="cn", precision=precision)
    dY, dX = ops.gather_scatter_pair(d["G"], d["Ws"], d["Wg"], d["Ind"], w_layout="nc", precision=precision)
    return Y, Out, dY, dX


# (B, T, E, K, I, J): I = outer width (C1 and N2), J = middle width (N1, a multiple of 32)
SHAPES = [
    (16, 256, 32, 32, 128, 64),      # the default float32 configuration's operator shape
    (3, 50, 5, 7, 128, 64),          # ragged rows: B*K = 21 of 128 tile rows
    (5, 300, 3, 60, 100, 32),        # contraction not a multiple of 32, N2 = 100 (not a multiple of 16)
    (2, 64, 2, 40, 36, 64),          # two stages of contraction, one of them partial
    (9, 40, 4, 33, 64, 32),          # B*K = 297: three row tiles, the last one partial
    (2, 64, 2, 40, 32, 96),          # one stage in phase 1, three in phase 2 on a 2-stage ring; 24 chunks per weight row
    (3, 80, 3, 50, 256, 128),        # TF32 only (strict tiles do not fit): eight + four stages
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("precision", ["strict", "tf32"])
def test_pair_matches_oracle(cuda_device, shape, precision):
    B, T, E, K, I, J = shape
    if not ops.fused_pair_eligible(I, J, I, torch.float32, precision=precision):
        pytest.skip("shape not taken by the fused kernel at this precision")
    w = Workload("pair", B, T, E, K, I, J, torch.float32, "distinct" if K <= T else "replace", 77 + B)
    ins = workloads.make_inputs(w)
    ref = orc.torch_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
    ops.reset_status()
    Y, Out, dY, dX = _pair_both_ways(to_dev(ins, cuda_device), precision)
    torch.cuda.synchronize()
    ops.check_status()
    got = {"Y": Y.cpu(), "Out": Out.cpu(), "dY": dY.cpu(), "dX": dX.cpu()}
    compare_step(got, ref, tol_for(torch.float32, precision), keys=("Y", "Out", "dY", "dX"), what=f"pair {shape} {precision}")


@pytest.mark.parametrize("index", ["distinct", "replace", "zipf"])
def test_pair_is_bit_exact_on_integer_valued_inputs(cuda_device, index):
    """Small-integer inputs make every product and sum exact: the fused kernel, the separate operators and the
    numpy oracle must agree bit for bit, collisions included."""
    w = Workload("pair-int", 4, 48, 6, 24, 64, 32, torch.float32, index, 5)
    ins = workloads.make_inputs(w, integer_valued=True)
    d = to_dev(ins, cuda_device)
    for precision in ("strict", "tf32"):
        Y, Out, dY, dX = _pair_both_ways(d, precision)
        Yr = orc.np_gather(ins["X"], ins["Wg"], ins["Ind"])
        assert np.array_equal(Y.cpu().double().numpy(), Yr)
        assert np.array_equal(Out.cpu().double().numpy(), orc.np_scatter(Yr, ins["Ws"], ins["Ind"], 48))
        assert torch.equal(Y, ops.gather_gemm(d["X"], d["Wg"], d["Ind"], precision=precision))
        assert torch.equal(Out, ops.gemm_scatter(Y, d["Ws"], d["Ind"], 48, precision=precision))
        assert torch.equal(dY, ops.gather_gemm(d["G"], d["Ws"], d["Ind"], w_layout="nc", precision=precision))
        assert torch.equal(dX, ops.gemm_scatter(dY, d["Wg"], d["Ind"], 48, w_layout="nc", precision=precision))


def test_pair_adds_into_a_given_output_and_zero_fills_otherwise(cuda_device):
    w = Workload("pair-acc", 2, 32, 3, 8, 32, 32, torch.float32, "distinct", 9)
    ins = workloads.make_inputs(w, integer_valued=True)
    d = to_dev(ins, cuda_device)
    _, Out = ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], d["Ind"])
    base = torch.full_like(Out, 3.0)
    _, Out2 = ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], d["Ind"], out=base)
    assert Out2 is base
    assert torch.equal(Out2, Out + 3.0)
    _, Out3 = ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], d["Ind"])      # fresh output: zero-filled again
    assert torch.equal(Out3, Out)


def test_pair_skips_and_reports_out_of_range_indices(cuda_device):
    w = Workload("pair-oob", 2, 40, 3, 6, 32, 32, torch.float32, "distinct", 11)
    ins = workloads.make_inputs(w, integer_valued=True)
    bad = ins["Ind"].clone()
    bad[1, 2, 3] = 40
    bad[0, 0, 0] = -1
    d = to_dev(ins, cuda_device)
    ops.reset_status()
    Y, Out = ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], bad.to(cuda_device))
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="outside"):
        ops.check_status()
    Yref = torch.from_numpy(orc.np_gather(ins["X"], ins["Wg"], ins["Ind"])).float()
    Yref[1, 2, 3] = 0
    Yref[0, 0, 0] = 0
    assert torch.equal(Y.cpu(), Yref)
    assert np.array_equal(Out.cpu().double().numpy(), orc.np_scatter(Yref, ins["Ws"], bad.clamp(0, 39), 40))


def test_ineligible_shapes_are_refused_not_miscomputed(cuda_device):
    assert not ops.fused_pair_eligible(128, 48, 128, torch.float32)            # middle width not a multiple of 32
    assert not ops.fused_pair_eligible(128, 24, 128, torch.bfloat16)           # 16-bit: middle width not a multiple of 16
    assert not ops.fused_pair_eligible(128, 512, 128, torch.bfloat16)          # 16-bit: middle width beyond 256
    assert not ops.fused_pair_eligible(128, 64, 512, torch.float32)            # output wider than one tile
    X = torch.zeros(1, 8, 128, device=cuda_device)
    W1 = torch.zeros(2, 128, 48, device=cuda_device)
    W2 = torch.zeros(2, 48, 128, device=cuda_device)
    Ind = torch.zeros(1, 2, 4, dtype=torch.int64, device=cuda_device)
    with pytest.raises(ValueError, match="not eligible"):
        ops.gather_scatter_pair(X, W1, W2, Ind)


def test_train_step_uses_the_pair_on_the_float32_configurations(cuda_device):
    """The explicit step takes the fused kernel where it is eligible: fewer launches, same results."""
    ins = workloads.make_inputs(workloads.WORKLOADS["cfg1-T256"])
    ref = orc.torch_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
    n0 = ops.launch_count()
    got = gpu_step(ins, cuda_device, "auto", "strict")
    launches = ops.launch_count() - n0
    compare_step(got, ref, 1e-5, what="cfg1-T256 fused step")
    assert launches <= 8, launches      # 2 fills + 2 pair kernels + 2 weight gradients (+ their fills)


@pytest.mark.parametrize("name,B", [("cfg1-T256", None), ("cfg0", 8), ("cfg2", 1)])
def test_gather_scatter_module_autograd(cuda_device, name, B):
    """ExpertGatherScatter (one autograd node; fused kernels where they pay, the two operators otherwise) against the
    oracle's forward and gradients: float32 fused (cfg1), float32 multi-wave (cfg0 slice), bf16 (cfg2 slice)."""
    import expertscattergather_b200 as egs
    w = workloads.WORKLOADS[name]
    ins = workloads.make_inputs(w, B=B)
    ref = orc.torch_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
    d = to_dev(ins, cuda_device)
    mod = egs.ExpertGatherScatter(w.E, w.I, w.J).to(cuda_device)
    mod = mod.to(w.dtype)
    with torch.no_grad():
        mod.gather.W.copy_(d["Wg"])
        mod.scatter.W.copy_(d["Ws"])
    x = d["X"].clone().requires_grad_(True)
    ops.reset_status()
    out = mod(x, d["Ind"])
    (out.float() * d["G"].float()).sum().backward()
    torch.cuda.synchronize()
    ops.check_status()
    got = {"Out": out.detach().cpu(), "dX": x.grad.cpu(), "dWg": mod.gather.W.grad.cpu(), "dWs": mod.scatter.W.grad.cpu()}
    compare_step(got, ref, tol_for(w.dtype, "strict"), keys=("Out", "dX", "dWg", "dWs"), what=f"module {name}")


@pytest.mark.parametrize("idx_dtype", [torch.int16, torch.int32, torch.uint8])
def test_pair_index_dtypes(cuda_device, idx_dtype):
    """Ind in every integer width the operators take (narrower ones are widened by the host like the others)."""
    w = Workload("pair-idx", 3, 100, 4, 20, 64, 32, torch.float32, "distinct", 13)
    ins = workloads.make_inputs(w, integer_valued=True)
    d = to_dev(ins, cuda_device)
    Y64, Out64 = ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], d["Ind"])
    Y, Out = ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], d["Ind"].to(idx_dtype))
    assert torch.equal(Y, Y64) and torch.equal(Out, Out64)


# ---- 16-bit tensors: the persistent pair kernel (Y stays in tensor memory between the two contractions) ----------

# (B, T, E, K, I, J): J = middle width (a multiple of 16, at most 256), I a multiple of 8
SHAPES16 = [
    (4, 256, 8, 64, 256, 128),       # full tiles: 2 row blocks per expert, 4 G stages, 4 S tiles
    (3, 50, 5, 7, 128, 64),          # ragged rows: B*K = 21 of 128 tile rows
    (5, 300, 3, 60, 104, 48),        # contraction and output width not multiples of 64; middle width 48
    (2, 64, 2, 40, 40, 16),          # the smallest middle width; one partial G stage
    (9, 40, 4, 33, 72, 80),          # three row blocks per expert, the last partial; two S tiles, the second 8 wide
    (6, 512, 40, 32, 512, 256),      # more row blocks (80) than a wave would need for overlap; widest middle tile
    (40, 128, 16, 64, 64, 32),       # 320 row blocks on 148 CTAs: every CTA walks several, S tiles and G stages interleave
]


@pytest.mark.parametrize("shape", SHAPES16)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_pair16_matches_oracle(cuda_device, shape, dtype):
    B, T, E, K, I, J = shape
    assert ops.fused_pair_eligible(I, J, I, dtype, w_layout="cn") and ops.fused_pair_eligible(I, J, I, dtype, w_layout="nc")
    w = Workload("pair16", B, T, E, K, I, J, dtype, "distinct" if K <= T else "replace", 91 + B)
    ins = workloads.make_inputs(w)
    ref = orc.torch_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
    ops.reset_status()
    Y, Out, dY, dX = _pair_both_ways(to_dev(ins, cuda_device), None)
    torch.cuda.synchronize()
    ops.check_status()
    got = {"Y": Y.cpu(), "Out": Out.cpu(), "dY": dY.cpu(), "dX": dX.cpu()}
    compare_step(got, ref, tol_for(dtype, "strict"), keys=("Y", "Out", "dY", "dX"), what=f"pair16 {shape} {dtype}")


@pytest.mark.parametrize("index", ["distinct", "replace", "zipf"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_pair16_is_bit_exact_on_integer_valued_inputs(cuda_device, index, dtype):
    """Small-integer inputs keep every product, every sum and the 16-bit rounding of the middle tensor exact: the fused
    kernel must agree bit for bit with the numpy oracle, collisions (direct 16-bit adds and float32 rows) included."""
    w = Workload("pair16-int", 6, 48, 6, 40, 64, 32, dtype, index, 5)
    ins = workloads.make_inputs(w, integer_valued=True)
    d = to_dev(ins, cuda_device)
    Y, Out, dY, dX = _pair_both_ways(d, None)
    Yr = orc.np_gather(ins["X"], ins["Wg"], ins["Ind"])
    assert np.array_equal(Y.float().cpu().numpy(), Yr.astype(np.float32))
    Outr = orc.np_scatter(Yr, ins["Ws"], ins["Ind"], w.T)
    if np.abs(Outr).max() < 256:            # integers up to 256 are exact in bf16; beyond that rounding may differ by order
        assert np.array_equal(Out.float().cpu().numpy(), Outr.astype(np.float32))
    dYr = orc.np_gather(ins["G"], np.swapaxes(ins["Ws"].float().numpy(), 1, 2), ins["Ind"])
    assert np.array_equal(dY.float().cpu().numpy(), dYr.astype(np.float32))


def test_pair16_equals_the_two_separate_operators(cuda_device):
    """Same inputs through egs_gather_gemm + egs_gemm_scatter and through the fused kernel: Y identical (same products, same
    rounding), Out equal up to the order of the 16-bit additions."""
    w = Workload("pair16-sep", 8, 256, 8, 32, 256, 128, torch.bfloat16, "distinct", 3)
    d = to_dev(workloads.make_inputs(w), cuda_device)
    Y, Out = ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], d["Ind"])
    Y2 = ops.gather_gemm(d["X"], d["Wg"], d["Ind"])
    Out2 = ops.gemm_scatter(Y2, d["Ws"], d["Ind"], w.T)
    assert torch.equal(Y, Y2)
    assert orc.rel_err(Out.cpu(), Out2.cpu()) <= 2e-2
    # adds into a given output, zero-fills otherwise
    base = torch.ones_like(Out)
    _, Out3 = ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], d["Ind"], out=base.clone())
    assert orc.rel_err(Out3.cpu(), (Out.float() + 1).cpu()) <= 2e-2


def test_pair16_skips_and_reports_out_of_range_indices(cuda_device):
    w = Workload("pair16-oob", 2, 64, 3, 16, 64, 32, torch.bfloat16, "distinct", 21)
    ins = workloads.make_inputs(w, integer_valued=True)
    Ind = ins["Ind"].clone()
    Ind[0, 1, 3] = w.T + 5
    Ind[1, 2, 0] = -1
    d = to_dev(ins, cuda_device)
    ops.reset_status()
    Y, Out = ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], Ind.to(cuda_device))
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="outside"):
        ops.check_status()
    assert float(Y[0, 1, 3].abs().max()) == 0.0 and float(Y[1, 2, 0].abs().max()) == 0.0
    good = Ind.clone()
    good[0, 1, 3] = 0
    good[1, 2, 0] = 0
    X2 = ins["X"].clone()
    Yr = orc.np_gather(X2, ins["Wg"], good)
    Yr[0, 1, 3] = 0
    Yr[1, 2, 0] = 0
    # the skipped slots contribute nothing: scatter of Y with those rows zeroed, to the rows the repaired index names
    Outr = orc.np_scatter(Yr, ins["Ws"], good, w.T)
    assert orc.rel_err(Out.float().cpu(), Outr) <= 1e-2          # (sums beyond 256 are rounded to 16 bits)
