"""Parity of the CUDA path (called through the C ABI) with the CPU oracle and the committed reference
outputs.  Bar: bit-exact for integer-valued inputs (index handling, collisions, zero fill); otherwise
max|a-ref|/max|ref| <= 1e-5 (float32 strict), 2e-2 (tf32), 3e-2 (bf16/fp16)."""
import numpy as np
import pytest
import torch

import expertscattergather_b200 as egs
from conftest import golden_names, load_golden
from expertscattergather_b200 import ops, workloads
from expertscattergather_b200.workloads import Workload
from expertscattergather_b200.step import train_step
from gpu_util import STEP_KEYS, TOL, compare_step, eligible, gpu_step, to_dev, tol_for
from oracle import egs_oracle as orc

pytestmark = pytest.mark.gpu


def _paths_for(ins):
    return ["generic", "tensor"] if eligible(ins) else ["generic"]


# ---------------------------------------------------------------------------------------------------------
# committed outputs of the reference's torch modules
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", golden_names())
def test_golden_full_step(cuda_device, name):
    ins, refs, T, dtype = load_golden(name)
    ref = {"Y": refs["f_Y"], "Out": refs["f_Out"], "dX": refs["f_dX"], "dWg": refs["f_dWg"], "dWs": refs["f_dWs"]}
    for path in _paths_for(ins):
        for precision in (("strict", "tf32") if dtype == torch.float32 and path == "tensor" else ("strict",)):
            got = gpu_step(ins, cuda_device, path, precision)
            if "integer" in name:
                for k in ref:
                    assert np.array_equal(got[k].float().numpy(), ref[k]), (name, path, precision, k)
            else:
                compare_step(got, ref, tol_for(dtype, precision), keys=tuple(ref), what=f"{name}/{path}/{precision}")


@pytest.mark.parametrize("name", golden_names())
def test_golden_modules_autograd(cuda_device, name):
    """The reference's own test flow (test_all.py:13-77): module forward, loss, backward, compare three tensors."""
    ins, refs, T, dtype = load_golden(name)
    d = to_dev(ins, cuda_device)
    E, I, J = ins["Wg"].shape
    tol = tol_for(dtype, "strict")
    gm = egs.ExpertGather(E, I, J).to(cuda_device)
    gm.W = torch.nn.Parameter(d["Wg"].clone())
    X = d["X"].clone().requires_grad_(True)
    Y = gm(X, d["Ind"].to(torch.int16))
    (Y * d["GY"]).sum().backward()
    sm = egs.ExpertScatter(E, J, I).to(cuda_device)
    sm.W = torch.nn.Parameter(d["Ws"].clone())
    Yin = d["Yin"].clone().requires_grad_(True)
    O = sm(Yin, d["Ind"].to(torch.int32), T)
    (O * d["G"]).sum().backward()
    torch.cuda.synchronize()
    ops.check_status()
    got = {"g_Y": Y, "g_dX": X.grad, "g_dW": gm.W.grad, "s_Out": O, "s_dY": Yin.grad, "s_dW": sm.W.grad}
    for k, v in got.items():
        v = v.detach().float().cpu().numpy()
        if "integer" in name:
            assert np.array_equal(v, refs[k]), (name, k)
        else:
            assert orc.rel_err(v, refs[k]) <= tol, (name, k, orc.rel_err(v, refs[k]))


# ---------------------------------------------------------------------------------------------------------
# the reference's random-shape tests (test_all.py:81-101): six dims drawn from [1,128), int16 ids with
# replacement, loss = output.sum() (so the incoming gradient is a stride-0 expanded scalar)
# ---------------------------------------------------------------------------------------------------------
def _random_dims(seed):
    g = torch.Generator().manual_seed(seed)
    return [int(v) for v in torch.randint(1, 128, (6,), generator=g)]


@pytest.mark.parametrize("seed", range(5))
def test_random_shapes_gather_module(cuda_device, seed):
    B, T, K, E, I, J = _random_dims(100 + seed)
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(B, T, I, generator=g)
    Ind = torch.randint(0, T, (B, E, K), generator=g).to(torch.int16)
    m = egs.ExpertGather(E, I, J).to(cuda_device)
    Xd = X.to(cuda_device).requires_grad_(True)
    Y = m(Xd, Ind.to(cuda_device))
    Y.sum().backward()
    torch.cuda.synchronize()
    ops.check_status()
    ref = orc.torch_gather_module_step(X, m.W.detach().cpu(), Ind, torch.ones(B, E, K, J))
    for got, key in ((Y, "Y"), (Xd.grad, "dX"), (m.W.grad, "dW")):
        got = got.detach().cpu()
        assert orc.rel_err(got, ref[key]) <= 1e-5, (key, orc.rel_err(got, ref[key]))
        assert torch.isclose(got, ref[key], atol=1e-3).all()      # the reference's own criterion (test_all.py:9-11)


@pytest.mark.parametrize("seed", range(5))
def test_random_shapes_scatter_module(cuda_device, seed):
    B, T, K, E, I, J = _random_dims(200 + seed)
    g = torch.Generator().manual_seed(seed)
    Yin = torch.randn(B, E, K, J, generator=g)
    Ind = torch.randint(0, T, (B, E, K), generator=g).to(torch.int16)
    m = egs.ExpertScatter(E, J, I).to(cuda_device)
    Yd = Yin.to(cuda_device).requires_grad_(True)
    O = m(Yd, Ind.to(cuda_device), T)
    O.sum().backward()
    torch.cuda.synchronize()
    ops.check_status()
    ref = orc.torch_scatter_module_step(Yin, m.W.detach().cpu(), Ind, T, torch.ones(B, T, I))
    for got, key in ((O, "Out"), (Yd.grad, "dY"), (m.W.grad, "dW")):
        got = got.detach().cpu()
        assert orc.rel_err(got, ref[key]) <= 1e-5, (key, orc.rel_err(got, ref[key]))
        assert torch.isclose(got, ref[key], atol=1e-3).all()


# ---------------------------------------------------------------------------------------------------------
# bit-exact index handling on both kernel families
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("index", ["distinct", "replace", "zipf"])
def test_integer_valued_inputs_are_bit_exact(cuda_device, dtype, index):
    # ragged sizes: rows per expert (B*K = 222) not a multiple of the 128-row tile, 3 k-stages + tail
    w = Workload("int", 6, 96, 5, 37, 104, 40, dtype, index, 4242)
    ins = workloads.make_inputs(w, integer_valued=True)
    ref = orc.np_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
    for path in ("generic", "tensor"):
        for precision in (("strict", "tf32") if dtype == torch.float32 else ("strict",)):
            if dtype != torch.float32:
                # 16-bit outputs: |values| stay far below 256 only for Y; compare what is exactly representable
                keys = ("Y", "dY")
            else:
                keys = STEP_KEYS
            got = gpu_step(ins, cuda_device, path, precision)
            for k in keys:
                assert np.array_equal(got[k].double().numpy(), ref[k]), (path, precision, k)


def test_identity_weights_return_the_gathered_rows(cuda_device):
    B, T, E, K, I = 3, 50, 4, 20, 64
    g = torch.Generator().manual_seed(5)
    X = torch.randn(B, T, I, generator=g).bfloat16().float()        # bf16-representable: exact in one TF32 product
    W = torch.eye(I).expand(E, I, I).contiguous()
    Ind = torch.randint(0, T, (B, E, K), generator=g)
    rows = torch.gather(X, 1, Ind.reshape(B, E * K, 1).expand(B, E * K, I)).reshape(B, E, K, I)
    for path in ("generic", "tensor"):
        for precision in ("strict", "tf32"):
            Y = ops.gather_gemm(X.to(cuda_device), W.to(cuda_device), Ind.to(cuda_device), path=path, precision=precision)
            assert torch.equal(Y.cpu(), rows), (path, precision)


@pytest.mark.parametrize("idx_dtype", [torch.int16, torch.int32, torch.int64, torch.uint8])
def test_index_dtypes(cuda_device, idx_dtype):
    w = Workload("idx", 2, 100, 3, 9, 32, 16, torch.float32, "replace", 9)
    ins = workloads.make_inputs(w, integer_valued=True)
    ref = orc.np_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
    ins["Ind"] = ins["Ind"].to(idx_dtype)
    for path in ("generic", "tensor"):
        got = gpu_step(ins, cuda_device, path)
        for k in STEP_KEYS:
            assert np.array_equal(got[k].double().numpy(), ref[k]), (path, k)


def test_scatter_output_is_zero_filled_every_call(cuda_device):
    """The reference's forward adds into torch.empty (egs/triton_kernels.py:457); here repeated calls agree."""
    w = Workload("z", 2, 300, 3, 5, 32, 16, torch.float32, "distinct", 3)
    ins = to_dev(workloads.make_inputs(w, integer_valued=True), cuda_device)
    Y = ops.gather_gemm(ins["X"], ins["Wg"], ins["Ind"])
    junk = torch.full((64, 300, 32), 7.0, device=cuda_device)   # dirty the allocator's cache
    del junk
    a = ops.gemm_scatter(Y, ins["Ws"], ins["Ind"], 300).clone()
    for _ in range(3):
        junk = torch.full((2, 300, 32), 9.0, device=cuda_device)
        del junk
        b = ops.gemm_scatter(Y, ins["Ws"], ins["Ind"], 300)
        assert torch.equal(a, b)
    # untouched token rows are exactly zero
    touched = torch.zeros(2, 300, dtype=torch.bool, device=cuda_device)
    touched.scatter_(1, ins["Ind"].reshape(2, -1), True)
    assert float(a[~touched].abs().sum()) == 0.0
    # accumulate-into-given-output mode adds on top
    c = ops.gemm_scatter(Y, ins["Ws"], ins["Ind"], 300, out=a.clone())
    assert torch.equal(c, 2 * a)


def test_out_of_range_index_is_skipped_and_reported(cuda_device):
    w = Workload("oob", 2, 40, 3, 6, 32, 16, torch.float32, "distinct", 11)
    ins = workloads.make_inputs(w, integer_valued=True)
    bad = ins["Ind"].clone()
    bad[1, 2, 3] = 40          # == T
    bad[0, 0, 0] = -1
    good_mask = torch.ones_like(bad, dtype=torch.bool)
    good_mask[1, 2, 3] = False
    good_mask[0, 0, 0] = False
    for path in ("generic", "tensor"):
        ops.reset_status()
        d = to_dev(ins, cuda_device)
        Y = ops.gather_gemm(d["X"], d["Wg"], bad.to(cuda_device), path=path)
        Yref = torch.from_numpy(orc.np_gather(ins["X"], ins["Wg"], ins["Ind"])).float()
        Yref[~good_mask] = 0
        assert torch.equal(Y.cpu(), Yref), path
        Out = ops.gemm_scatter(Y, d["Ws"], bad.to(cuda_device), 40, path=path)
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="outside"):
            ops.check_status()
        ops.check_status()      # the word is cleared by the failed check
        safe = bad.clamp(0, 39)
        ref = orc.np_scatter(Yref, ins["Ws"], safe, 40)
        assert np.array_equal(Out.cpu().double().numpy(), ref), path


# ---------------------------------------------------------------------------------------------------------
# benchmark configurations (full size where the CPU checker finishes in seconds, batch slices otherwise)
# ---------------------------------------------------------------------------------------------------------
CONFIG_CASES = [("cfg0", None), ("cfg1-T256", None), ("cfg1-T1024", None), ("cfg1-T4096", 4), ("cfg1-T16384", 2),
                ("cfg2", 2), ("cfg3", 1), ("cfg4", 2)]


@pytest.mark.parametrize("name,B", CONFIG_CASES)
def test_benchmark_configurations(cuda_device, name, B):
    w = workloads.WORKLOADS[name]
    ins = workloads.make_inputs(w, B=B)
    ref = orc.torch_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
    truth = orc.np_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"]) if w.dtype != torch.float32 else None
    precisions = ("strict", "tf32") if w.dtype == torch.float32 else ("strict",)
    for precision in precisions:
        got = gpu_step(ins, cuda_device, "auto", precision)
        tol = tol_for(w.dtype, precision)
        compare_step(got, ref, tol, what=f"{name}/{precision} vs same-dtype torch path")
        if truth is not None:
            compare_step(got, truth, tol, what=f"{name}/{precision} vs float64 truth")
    gen = gpu_step(ins, cuda_device, "generic", "strict")
    compare_step(gen, ref, tol_for(w.dtype, "strict"), what=f"{name}/generic")


def test_full_size_properties_cfg4_shard(cuda_device):
    """Size-independent checks at the per-GPU size of the multi-GPU configuration (B=64 of cfg4), where the CPU
    checker is too slow: (1) checksum of checksums - column sums of Out per batch element equal the column sums
    of the per-slot products computed by a dense contraction; (2) linearity of the gather in X; (3) dW against a
    dense contraction over a materialised gather, accumulated over batch chunks."""
    w = workloads.WORKLOADS["cfg4"].with_batch(64)
    ins = to_dev(workloads.make_inputs(w), cuda_device)
    X, Wg, Ws, Ind, G = (ins[k] for k in ("X", "Wg", "Ws", "Ind", "G"))
    Y = ops.gather_gemm(X, Wg, Ind)
    Out = ops.gemm_scatter(Y, Ws, Ind, w.T)
    dense = torch.einsum("bekj,eji->bi", Y.float(), Ws.float())
    got = Out.float().sum(1)
    assert float((got - dense).abs().max() / dense.abs().max()) <= 3e-2
    X2 = torch.roll(X, 1, 0)
    Ysum = ops.gather_gemm((X.float() + X2.float()).to(w.dtype), Wg, Ind)
    Y2 = ops.gather_gemm(X2, Wg, Ind)
    lin = (Ysum.float() - (Y.float() + Y2.float())).abs().max() / Ysum.float().abs().max()
    assert float(lin) <= 3e-2
    dY = ops.gather_gemm(G, Ws, Ind, w_layout="nc")
    dWg = ops.dweight(X, dY, Ind)
    dense_dw = torch.zeros(w.E, w.I, w.J, device=cuda_device)
    for b0 in range(0, w.B, 8):
        sl = slice(b0, b0 + 8)
        rows = torch.gather(X[sl], 1, Ind[sl].reshape(8, -1, 1).expand(-1, -1, w.I)).reshape(8, w.E, w.K, w.I)
        dense_dw += torch.einsum("beki,bekj->eij", rows.float(), dY[sl].float())
    assert float((dWg.float() - dense_dw).abs().max() / dense_dw.abs().max()) <= 3e-2
    torch.cuda.synchronize()
    ops.check_status()


def test_no_gathered_intermediate_is_allocated(cuda_device):
    """Peak device memory of a step stays below outputs + dW scratch + a small margin: no [B,E,K,I] block."""
    w = workloads.WORKLOADS["cfg2"].with_batch(4)
    ins = to_dev(workloads.make_inputs(w), cuda_device)
    from expertscattergather_b200.step import train_step
    train_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])      # warm the allocator and the library
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    out = train_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    outputs = sum(v.numel() * v.element_size() for v in out.values())
    scratch = 2 * w.E * w.I * w.J * 4
    gathered_block = w.B * w.E * w.K * w.I * 2
    assert peak <= outputs + scratch + (1 << 20), (peak, outputs, scratch)
    assert gathered_block > (1 << 22)     # the block the reference's torch path materialises would be visible


# ---------------------------------------------------------------------------------------------------------
# ragged shapes that reach the large-problem kernel variants (256-row CTA tiles for G, the persistent
# warp-specialised scatter, direct 16-bit adds) - compared with the generic kernels and the CPU checker
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,precision,T,index", [(torch.bfloat16, "strict", 300, "replace"),
                                                     (torch.float32, "tf32", 300, "replace"),
                                                     (torch.bfloat16, "strict", 3000, "distinct")])
def test_large_variants_on_ragged_shapes(cuda_device, dtype, precision, T, index):
    # M = B*K = 500 rows per expert (not a multiple of 128 or 256), J = 72 (two contraction stages for S, the second
    # partial), I = 1320 (six 256-wide output tiles for S, the last 40 wide; 21 or 42 contraction stages for G).
    # T = 300 with replacement: dozens of contributions per token (16-bit scatter sums in float32 rows);
    # T = 3000 distinct: a few per token (16-bit scatter adds directly, as bulk reductions, ragged last tile included).
    w = Workload("ragged-large", 5, T, 80, 100, 1320, 72, dtype, index, 808)
    ins = workloads.make_inputs(w, integer_valued=True)
    ins["Ind"][2, 7, 5] = T            # out of range: skipped and reported
    ins["Ind"][4, 79, 99] = -3
    ref_ind = ins["Ind"].clamp(0, T - 1)
    d = to_dev(ins, cuda_device)
    res = {}
    for path in ("generic", "tensor"):
        ops.reset_status()
        Y = ops.gather_gemm(d["X"], d["Wg"], d["Ind"], path=path, precision=precision)
        Out = ops.gemm_scatter(Y, d["Ws"], d["Ind"], w.T, path=path, precision=precision)
        dY = ops.gather_gemm(d["G"], d["Ws"], d["Ind"], w_layout="nc", path=path, precision=precision)
        dX = ops.gemm_scatter(dY, d["Wg"], d["Ind"], w.T, w_layout="nc", path=path, precision=precision)
        dWg = ops.dweight(d["X"], dY, d["Ind"], path=path, precision=precision)
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="outside"):
            ops.check_status()
        res[path] = {"Y": Y.cpu(), "Out": Out.cpu(), "dY": dY.cpu(), "dX": dX.cpu(), "dWg": dWg.cpu()}
    # integer-valued inputs: Y and dY are exact in every dtype, so both families must agree bit for bit there
    for k in ("Y", "dY"):
        assert torch.equal(res["generic"][k], res["tensor"][k]), k
    # and with the checker on the rows whose index is valid (masked slots give zero rows / add nothing)
    Yref = orc.np_gather(ins["X"], ins["Wg"], ref_ind)
    bad = torch.zeros_like(ins["Ind"], dtype=torch.bool)
    bad[2, 7, 5] = True
    bad[4, 79, 99] = True
    Yref[bad.numpy()] = 0
    assert np.array_equal(res["tensor"]["Y"].double().numpy(), Yref)
    tol = tol_for(dtype, precision)
    for k in ("Out", "dX", "dWg"):
        assert orc.rel_err(res["tensor"][k], res["generic"][k]) <= tol, (k, orc.rel_err(res["tensor"][k], res["generic"][k]))
    Outref = orc.np_scatter(torch.from_numpy(Yref), ins["Ws"], ref_ind, w.T)
    assert orc.rel_err(res["tensor"]["Out"], Outref) <= tol


@pytest.mark.parametrize("dtype,precision", [(torch.bfloat16, "strict"), (torch.float32, "tf32")])
def test_weight_gradient_two_tile_variant_on_ragged_shapes(cuda_device, dtype, precision):
    """Operator D where the host picks two 128-feature accumulators per CTA (long contraction, grid covering the SMs):
    M = B*K = 1100 contraction rows (last stage partial), FG = 1320 features (five full 256-feature tiles and one of
    40), FD = 72.  Integer-valued inputs make every sum exact in float32, so the tensor-core kernel, the generic
    kernel and the numpy checker must agree bit for bit, in both output layouts."""
    w = Workload("ragged-dw", 11, 400, 30, 100, 1320, 72, dtype, "distinct", 909)
    ins = workloads.make_inputs(w, integer_valued=True)
    ins["Ind"][3, 4, 5] = 400          # out of range: contributes nothing
    ref_ind = ins["Ind"].clone()
    d = to_dev(ins, cuda_device)
    Ycpu = torch.randint(-3, 4, (w.B, w.E, w.K, w.J), generator=torch.Generator().manual_seed(5)).to(dtype)   # slot rows
    Y = Ycpu.to(cuda_device)
    res = {}
    for path in ("generic", "tensor"):
        ops.reset_status()
        dWg = ops.dweight(d["X"], Y, d["Ind"], path=path, precision=precision)                          # [E, I, J]
        dWs = ops.dweight(d["G"], Y, d["Ind"], out_layout="direct_rows", path=path, precision=precision)  # [E, J, I]
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="outside"):
            ops.check_status()
        res[path] = (dWg.cpu(), dWs.cpu())
    assert torch.equal(res["generic"][0], res["tensor"][0])
    assert torch.equal(res["generic"][1], res["tensor"][1])
    # checker: the masked slot adds nothing -> zero its slot row on the checker's side
    Ymask = Ycpu.clone().float()
    Ymask[3, 4, 5] = 0
    ref_ind[3, 4, 5] = 0
    ref_g = torch.from_numpy(orc.np_dweight(ins["X"], Ymask, ref_ind)).to(dtype)
    assert torch.equal(res["tensor"][0], ref_g)
    ref_s = torch.from_numpy(orc.np_dweight(ins["G"], Ymask, ref_ind)).to(dtype).transpose(1, 2).contiguous()
    assert torch.equal(res["tensor"][1], ref_s)


def test_gradients_nobody_asked_for_are_not_computed(cuda_device):
    """needs_input_grad pruning: with a frozen weight or a data input the corresponding kernel is not launched, and
    the gradient that is asked for is unchanged."""
    w = Workload("prune", 3, 64, 4, 16, 64, 32, torch.float32, "distinct", 21)
    ins = workloads.make_inputs(w)
    ref = orc.torch_step(ins["X"], ins["Wg"], ins["Ws"], ins["Ind"], ins["G"])
    d = to_dev(ins, cuda_device)

    def run(x_grad, w_grad):
        g = egs.ExpertGather(w.E, w.I, w.J).to(cuda_device)
        s = egs.ExpertScatter(w.E, w.J, w.I).to(cuda_device)
        with torch.no_grad():
            g.W.copy_(d["Wg"]); s.W.copy_(d["Ws"])
        g.W.requires_grad_(w_grad); s.W.requires_grad_(w_grad)
        x = d["X"].clone().requires_grad_(x_grad)
        out = s(g(x, d["Ind"]), d["Ind"], w.T)
        n0 = ops.launch_count()
        (out * d["G"]).sum().backward()
        torch.cuda.synchronize()
        return ops.launch_count() - n0, x.grad, g.W.grad, s.W.grad

    n_all, dx, dwg, dws = run(True, True)
    n_x, dx_only, none_g, none_s = run(True, False)
    n_w, none_x, dwg_only, dws_only = run(False, True)
    assert none_g is None and none_s is None and none_x is None
    assert n_x < n_all and n_w < n_all
    for a, b in ((dx_only, dx), (dwg_only, dwg), (dws_only, dws)):      # float32 atomics: equal up to summation order
        assert orc.rel_err(a.cpu(), b.cpu()) <= 1e-6
    assert orc.rel_err(dx.cpu(), ref["dX"]) <= 1e-5 and orc.rel_err(dwg.cpu(), ref["dWg"]) <= 1e-5


def test_weight_gradient_into_a_prezeroed_output(cuda_device):
    """egs_dweight_prezeroed: the caller's zero-filled float32 output is accumulated into without a fill of the
    library's own; the result equals the plain call's, and 16-bit tensors are refused (they sum in scratch)."""
    w = Workload("prezero", 4, 96, 6, 24, 64, 32, torch.float32, "distinct", 31)
    ins = workloads.make_inputs(w, integer_valued=True)
    d = to_dev(ins, cuda_device)
    Y = ops.gather_gemm(d["X"], d["Wg"], d["Ind"])
    plain = ops.dweight(d["X"], Y, d["Ind"])
    buf = torch.zeros_like(plain)
    n0 = ops.launch_count()
    got = ops.dweight(d["X"], Y, d["Ind"], zeroed_out=buf)
    assert ops.launch_count() - n0 == 1          # the contraction kernel alone
    assert got is buf and torch.equal(got, plain)
    with pytest.raises(ValueError, match="float32"):
        ops.dweight(d["X"].bfloat16(), Y.bfloat16(), d["Ind"], zeroed_out=buf)


# ---------------------------------------------------------------------------------------------------------
# full benchmark sizes of the tensor-bound configurations: all six outputs, element by element
# ---------------------------------------------------------------------------------------------------------
def _checker_step_on_device(d, chunk):
    """The oracle's torch restatement (oracle.torch_step: gather + einsum + scatter_add_, gradients by autograd) evaluated
    on the GPU in float32 over batch chunks, the weight gradients summed over the chunks in float32.  For these two
    cases only this stands in for the CPU run of the same functions, which needs minutes at these sizes; the inputs are
    the test's 16-bit tensors upcast, so it differs from exact arithmetic by float32 rounding only."""
    X, Wg, Ws, Ind, G = (d[k] for k in ("X", "Wg", "Ws", "Ind", "G"))
    Wg32, Ws32 = Wg.float(), Ws.float()
    outs = {k: [] for k in ("Y", "Out", "dY", "dX")}
    dWg = torch.zeros_like(Wg32)
    dWs = torch.zeros_like(Ws32)
    for b0 in range(0, X.shape[0], chunk):
        sl = slice(b0, b0 + chunk)
        r = orc.torch_step(X[sl].float(), Wg32, Ws32, Ind[sl], G[sl].float())
        for k in outs:
            outs[k].append(r[k])
        dWg += r["dWg"]
        dWs += r["dWs"]
    res = {k: torch.cat(v) for k, v in outs.items()}
    res["dWg"], res["dWs"] = dWg, dWs
    return res


def _rel_err_on_device(a, ref):
    return float((a.float() - ref).abs().max() / ref.abs().max())


@pytest.mark.parametrize("name,B,chunk", [("cfg4", 64, 8), ("cfg3", 8, 2)])
def test_full_size_parity_of_the_tensor_bound_configurations(cuda_device, name, B, chunk):
    """cfg4 at its per-GPU batch (64) and cfg3 at full size through the explicit step: every element of Y, Out, dY, dX, dW_g
    and dW_s against the checker, and the kernel variants the benchmark times at these sizes must be the ones that ran
    (256-row gather CTAs, the persistent scatter with bulk reductions, two-accumulator weight-gradient CTAs)."""
    w = workloads.WORKLOADS[name].with_batch(B)
    plan_g = ops.describe_plan("G", B, w.T, w.E, w.K, w.I, w.J, w.dtype)
    plan_s = ops.describe_plan("S", B, w.T, w.E, w.K, w.J, w.I, w.dtype)
    plan_d = ops.describe_plan("D", B, w.T, w.E, w.K, w.I, w.J, w.dtype)
    assert plan_g["tensor_path"] and plan_g["row_tiles"] == 2, plan_g
    assert plan_d["tensor_path"] and plan_d["row_tiles"] == 2, plan_d
    if name == "cfg4":
        assert plan_s["persistent"] == 1 and plan_s["bulk_epilogue"] == 1 and plan_s["expert_fastest"] == 1, plan_s
    else:
        assert plan_s["tensor_path"] == 1 and plan_s["persistent"] == 0, plan_s
    d = to_dev(workloads.make_inputs(w), cuda_device)
    ops.reset_status()
    got = train_step(d["X"], d["Wg"], d["Ws"], d["Ind"], d["G"])
    torch.cuda.synchronize()
    ops.check_status()
    ref = _checker_step_on_device(d, chunk)
    errs = {k: _rel_err_on_device(got[k], ref[k]) for k in ("Y", "Out", "dY", "dX", "dWg", "dWs")}
    assert all(e <= TOL["bf16"] for e in errs.values()), errs
    # the fused 16-bit pair kernel at the same size (cfg4: middle width 256 fits; cfg3's 512 does not)
    if ops.fused_pair_eligible(w.I, w.J, w.I, w.dtype):
        Y, Out = ops.gather_scatter_pair(d["X"], d["Wg"], d["Ws"], d["Ind"])
        dY, dX = ops.gather_scatter_pair(d["G"], d["Ws"], d["Wg"], d["Ind"], w_layout="nc")
        torch.cuda.synchronize()
        ops.check_status()
        perr = {"Y": _rel_err_on_device(Y, ref["Y"]), "Out": _rel_err_on_device(Out, ref["Out"]),
                "dY": _rel_err_on_device(dY, ref["dY"]), "dX": _rel_err_on_device(dX, ref["dX"])}
        assert all(e <= TOL["bf16"] for e in perr.values()), perr


def test_strict_float32_on_long_contractions(cuda_device):
    """Strict float32 is three TF32 products per element (hi*hi + hi*lo + lo*hi) summed in the tensor core's float32
    accumulator, whose additions truncate: the error grows with the number of accumulation steps (3.3e-5 at a contraction
    of 4096, 1.5e-5 after 8192 rows of D were measured with everything on the tensor cores).  The library therefore
    bounds what one accumulator sees: G / S beyond a contraction of 512 take the FFMA kernels, D splits its rows into
    ranges of at most 1024 whose partial tiles are summed by float32 atomics.  Checked against float64 truth."""
    w = Workload("long", 64, 512, 2, 128, 4096, 64, torch.float32, "distinct", 99)
    ins = workloads.make_inputs(w)
    d = to_dev(ins, cuda_device)
    assert ops.describe_plan("G", w.B, w.T, w.E, w.K, w.I, w.J, w.dtype, precision="strict")["tensor_path"] == 0
    plan_d = ops.describe_plan("D", w.B, w.T, w.E, w.K, w.I, w.J, w.dtype, precision="strict")
    assert plan_d["tensor_path"] == 1 and plan_d["rows_per_split"] <= 1024, plan_d
    ops.reset_status()
    Y = ops.gather_gemm(d["X"], d["Wg"], d["Ind"], precision="strict")
    dWg = ops.dweight(d["X"], Y, d["Ind"], precision="strict")
    torch.cuda.synchronize()
    ops.check_status()
    e_g = orc.rel_err(Y.cpu(), orc.np_gather(ins["X"], ins["Wg"], ins["Ind"]))
    e_d = orc.rel_err(dWg.cpu(), orc.np_dweight(ins["X"], Y.cpu(), ins["Ind"]))
    # the longest contraction that stays on the tensor cores in strict mode
    w2 = Workload("long512", 16, 256, 4, 64, 512, 64, torch.float32, "distinct", 98)
    ins2 = workloads.make_inputs(w2)
    d2 = to_dev(ins2, cuda_device)
    assert ops.describe_plan("G", w2.B, w2.T, w2.E, w2.K, w2.I, w2.J, w2.dtype, precision="strict")["tensor_path"] == 1
    Y2 = ops.gather_gemm(d2["X"], d2["Wg"], d2["Ind"], precision="strict")
    torch.cuda.synchronize()
    e_g2 = orc.rel_err(Y2.cpu(), orc.np_gather(ins2["X"], ins2["Wg"], ins2["Ind"]))
    print(f"strict float32: G C=4096 (FFMA) {e_g:.2e}, G C=512 (tensor cores) {e_g2:.2e}, D 8192 rows in ranges of <=1024 {e_d:.2e}")
    assert e_g <= TOL["fp32"] and e_g2 <= TOL["fp32"] and e_d <= TOL["fp32"], (e_g, e_g2, e_d)
