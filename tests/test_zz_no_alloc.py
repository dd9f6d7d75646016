"""The allocation-free weight-gradient entry point (egs_dweight_static_scratch), called through the C ABI.

Some hosts of this library may not allocate device memory at the moment they call it: a runtime that handed its
whole memory budget to its own arena at start-up, a plug-in that only sees the pointers of its inputs and outputs,
a latency-critical loop that must not risk an allocation.  For them the float32 scratch of the weight-gradient
operator is a fixed 16 MiB array inside the library.  These tests call that entry point twice in a row with
different inputs (the second call meets the first call's leftovers in the shared array) and compare each result
with the ordinary entry point, which gets scratch from the caller.  The file name sorts last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

from expertscattergather_b200 import _lib
from expertscattergather_b200.workloads import Workload, make_inputs
from oracle import egs_oracle as orc

TOL_BF16 = 3e-2     # max|a-b| / max|b|, the bf16 tolerance of the parity tests


def _rel(a, b):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    return float((a - b).abs().max() / b.abs().max())


def _call_pair(lib, dev, w, seed_shift, out_layout, watch_allocations=False):
    """Runs both entry points on the same inputs; returns (static-scratch result, caller-scratch result, the float64 result of
    the CPU checker).  With watch_allocations the call of the static-scratch entry point is bracketed by readings of the
    driver's free-memory figure and of torch's allocator counters: none of them may move."""
    ins = make_inputs(Workload(w.name, w.B, w.T, w.E, w.K, w.I, w.J, w.dtype, w.index, w.seed + seed_shift))
    X = ins["X"].to(dev)
    Ind = ins["Ind"].to(dev)
    g = torch.Generator().manual_seed(w.seed + 100 + seed_shift)
    dY = torch.randn(w.B, w.E, w.K, w.J, generator=g).to(w.dtype).to(dev)
    shape = (w.E, w.I, w.J) if out_layout == _lib.DW_GATHERED_ROWS else (w.E, w.J, w.I)
    out_static = torch.full(shape, float("nan"), dtype=w.dtype, device=dev)
    out_plain = torch.full(shape, float("nan"), dtype=w.dtype, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    common = (X.data_ptr(), dY.data_ptr(), Ind.data_ptr())
    dims = (w.B, w.T, w.E, w.K, w.I, w.J, out_layout, _lib.BF16, _lib.I64, _lib.PREC_STRICT, _lib.PATH_AUTO)
    if watch_allocations:
        torch.cuda.synchronize(dev)
        free0 = torch.cuda.mem_get_info(dev)[0]
        stats0 = torch.cuda.memory_stats(dev)
    rc = lib.egs_dweight_static_scratch(*common, out_static.data_ptr(), *dims, status.data_ptr(), stream)
    assert rc == _lib.OK, (rc, lib.egs_last_cuda_error())
    if watch_allocations:
        torch.cuda.synchronize(dev)
        stats1 = torch.cuda.memory_stats(dev)
        assert torch.cuda.mem_get_info(dev)[0] == free0, "the driver's free memory changed across the call"
        for key in ("allocation.all.allocated", "segment.all.allocated", "allocated_bytes.all.allocated", "num_alloc_retries"):
            assert stats1.get(key, 0) == stats0.get(key, 0), key
    ws_bytes = int(lib.egs_dw_workspace_bytes(w.E, w.I, w.J, _lib.BF16))
    ws = torch.empty(ws_bytes // 4, dtype=torch.float32, device=dev)
    rc = lib.egs_dweight(*common, out_plain.data_ptr(), *dims, ws.data_ptr(), ws_bytes, status.data_ptr(), stream)
    assert rc == _lib.OK, (rc, lib.egs_last_cuda_error())
    torch.cuda.synchronize(dev)
    assert int(status.item()) == 0
    truth = torch.from_numpy(orc.np_dweight(ins["X"], dY.cpu(), ins["Ind"]))          # [E, I, J] in float64
    if out_layout == _lib.DW_DIRECT_ROWS:
        truth = truth.transpose(1, 2)
    return out_static, out_plain, truth


@pytest.mark.gpu
def test_static_scratch_matches_caller_scratch_on_two_calls_in_a_row(cuda_device):
    lib = _lib.load()
    # bf16 with few output tiles and many rows per expert: the contraction is split over CTAs, so the float32
    # scratch is really used (partial tiles are added into it, then converted)
    w = Workload("noalloc", 8, 96, 4, 64, 256, 64, torch.bfloat16, "distinct", 321)
    assert w.E * w.I * w.J <= lib.egs_static_scratch_max_elements()
    first = _call_pair(lib, cuda_device, w, 0, _lib.DW_GATHERED_ROWS)
    # other inputs, other layout, same array; this second call (the address look-up is behind us) must not allocate
    second = _call_pair(lib, cuda_device, w, 1, _lib.DW_DIRECT_ROWS, watch_allocations=True)
    for got, want, truth in (first, second):
        assert torch.isfinite(got.float()).all() and torch.isfinite(want.float()).all()
        assert _rel(got, want) <= TOL_BF16, _rel(got, want)
        assert _rel(got, truth) <= TOL_BF16, _rel(got, truth)          # and against the CPU checker
    # the two calls really computed different things
    assert _rel(first[0], second[0].transpose(1, 2)) > 0.1


def test_static_scratch_rejects_oversized_problems():
    """Needs no GPU: the size check comes before anything touches the device."""
    lib = _lib.load()
    cap = lib.egs_static_scratch_max_elements()
    assert cap == 4 * 1024 * 1024
    E, FG, FD = 64, 1024, 256            # 16 Mi elements > 4 Mi
    assert E * FG * FD > cap
    rc = lib.egs_dweight_static_scratch(None, None, None, None, 8, 64, E, 4, FG, FD, 0, _lib.BF16, _lib.I64, 0, 0, None, None)
    assert rc == _lib.ERR_TOO_LARGE
    assert b"exceed the built-in scratch" in lib.egs_last_cuda_error()
    assert lib.egs_dweight_static_scratch(None, None, None, None, 8, 64, -1, 4, 8, 8, 0, _lib.BF16, _lib.I64, 0, 0, None, None) == \
        _lib.ERR_INVALID_ARGUMENT
    # float32 tensors accumulate in the output, never in the scratch: the limit does not apply to them (the call gets past
    # the size check and fails later, here for want of a device / of pointers)
    rc = lib.egs_dweight_static_scratch(None, None, None, None, 8, 64, E, 4, FG, FD, 0, _lib.F32, _lib.I64, 0, 0, None, None)
    assert rc != _lib.ERR_TOO_LARGE
