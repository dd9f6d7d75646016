"""Operator G on pairs of SMs (``path="paired"``: thread-block clusters of two CTAs, tcgen05.mma.cta_group::2) against the
single-CTA tensor path and float64 torch, forward and transposed-weight forms, ragged shapes, bias."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(X, W, Ind, layout, bias=None):
    B, T, C = X.shape
    Wv = W.double() if layout == "cn" else W.double().transpose(1, 2)
    rows = torch.gather(X.double().unsqueeze(1).expand(B, Ind.shape[1], T, C), 2,
                        Ind.long().unsqueeze(-1).expand(-1, -1, -1, C))
    Y = torch.einsum("bekc,ecn->bekn", rows, Wv)
    if bias is not None:
        Y = Y + bias.double().reshape(1, -1, 1, Y.shape[-1])
    return Y


def _case(B, T, E, K, C, N, dt, layout, seed, with_bias=False):
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(seed)
    X = torch.randn(B, T, C, generator=g).to(dev).to(dt)
    W = (torch.randn(E, C, N, generator=g) / C ** 0.5).to(dev).to(dt)
    if layout == "nc":
        W = W.transpose(1, 2).contiguous()
    Ind = torch.stack([torch.stack([torch.randperm(T, generator=g)[:K] for _ in range(E)]) for _ in range(B)]).to(dev).int()
    bias = (torch.randn(E, N, generator=g)).to(dev).to(dt) if with_bias else None
    return X, W, Ind, bias


@pytest.mark.parametrize("shape", [
    (8, 256, 4, 64, 64, 64), (8, 256, 4, 64, 128, 256), (9, 300, 3, 70, 72, 96), (16, 128, 5, 33, 200, 32),
    (8, 1024, 64, 64, 1024, 256), (5, 512, 2, 128, 1024, 224), (1, 64, 2, 8, 64, 64)])
@pytest.mark.parametrize("layout", ["cn", "nc"])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_paired_gather_matches_the_single_cta_kernel(shape, layout, dt):
    from expertscattergather_b200 import ops
    X, W, Ind, _ = _case(*shape, dt, layout, seed=sum(shape))
    Yp = ops.gather_gemm(X, W, Ind, w_layout=layout, path="paired")
    Yt = ops.gather_gemm(X, W, Ind, w_layout=layout, path="tensor")
    ops.check_status()
    # both kernels accumulate the same products in float32 (in a different order) and round once
    r = _ref(X, W, Ind, layout)
    scale = r.abs().max().item()
    assert (Yp.double() - r).abs().max().item() <= 6e-3 * scale
    assert (Yp.double() - Yt.double()).abs().max().item() <= 4e-3 * scale


def test_paired_gather_with_bias_and_out_of_range_indices():
    from expertscattergather_b200 import ops
    X, W, Ind, bias = _case(6, 200, 3, 40, 128, 128, torch.bfloat16, "cn", seed=5, with_bias=True)
    Y = ops.gather_gemm(X, W, Ind, bias=bias, path="paired")
    ops.check_status()
    r = _ref(X, W, Ind, "cn", bias)
    assert (Y.double() - r).abs().max().item() <= 6e-3 * r.abs().max().item()
    bad = Ind.clone()
    bad[1, 2, 3] = 200                                  # one past the last token: the row is written as zeros (+ bias)
    Yb = ops.gather_gemm(X, W, bad, path="paired")
    with pytest.raises(RuntimeError):
        ops.check_status()
    ops.reset_status()
    assert Yb[1, 2, 3].abs().max().item() == 0.0
    keep = torch.ones_like(Yb, dtype=torch.bool)
    keep[1, 2, 3] = False
    Yok = ops.gather_gemm(X, W, Ind, path="paired")
    assert torch.equal(Yb[keep], Yok[keep])


def test_paired_path_refuses_what_it_does_not_take():
    from expertscattergather_b200 import ops
    dev = torch.device("cuda", 0)
    X = torch.randn(2, 32, 64, device=dev)
    W = torch.randn(2, 64, 64, device=dev)
    Ind = torch.zeros(2, 2, 4, dtype=torch.int32, device=dev)
    with pytest.raises(ValueError):                    # float32
        ops.gather_gemm(X, W, Ind, path="paired")
    with pytest.raises(ValueError):                    # N not a multiple of 32
        ops.gather_gemm(X.bfloat16(), torch.randn(2, 64, 48, device=dev).bfloat16(), Ind, path="paired")
    with pytest.raises(ValueError):                    # operator S
        ops.gemm_scatter(torch.randn(2, 2, 4, 64, device=dev).bfloat16(), W.bfloat16(), Ind, 32, path="paired")
    with pytest.raises(ValueError):
        ops.set_path("paired")


def test_paired_gather_at_the_benchmark_shard_size():
    """cfg4 at the per-GPU shard (B=64): 512 tiles over 74 CTA pairs, i.e. the persistent walk, the accumulator hand-over
    between tiles and the expert-fastest tile order are all exercised; element by element against the single-CTA kernel."""
    from expertscattergather_b200 import ops, workloads as wl
    dev = torch.device("cuda", 0)
    w = wl.WORKLOADS["cfg4"]
    d = {k: v.to(dev) for k, v in wl.make_inputs(w, B=64).items()}
    for X, W, layout in ((d["X"], d["Wg"], "cn"), (d["G"], d["Ws"], "nc")):
        Yp = ops.gather_gemm(X, W, d["Ind"], w_layout=layout, path="paired")
        Yt = ops.gather_gemm(X, W, d["Ind"], w_layout=layout, path="tensor")
        ops.check_status()
        scale = Yt.float().abs().max().item()
        assert (Yp.float() - Yt.float()).abs().max().item() <= 8e-3 * scale, layout
        # same products, float32 accumulation in both: most elements agree to the last bit
        assert (Yp == Yt).float().mean().item() > 0.9, layout
