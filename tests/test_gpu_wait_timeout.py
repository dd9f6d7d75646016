"""Failure detection without a fault: every wait inside the tensor-core kernels is bounded.  The library's self-test
launches one CTA that waits on a barrier nobody completes; the wait gives up after its limit, the kernel returns, the
status word says so, and the context stays usable."""
import ctypes
import time

import pytest
import torch

from expertscattergather_b200 import _lib, ops, workloads
from expertscattergather_b200.workloads import Workload

pytestmark = pytest.mark.gpu


def test_a_wait_that_cannot_be_satisfied_runs_out_and_is_reported(cuda_device):
    lib = _lib.load()
    ops.reset_status()
    w = Workload("timeout", 2, 64, 2, 40, 64, 32, torch.bfloat16, "distinct", 3)
    d = {k: v.to(cuda_device) for k, v in workloads.make_inputs(w, integer_valued=True).items()}
    good = ops.gather_gemm(d["X"], d["Wg"], d["Ind"], path="tensor")
    torch.cuda.synchronize()
    ops.check_status()

    status = ops._status_word(cuda_device)
    out2 = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    limit = 100_000_000                      # SM clocks: about 50 ms
    t0 = time.perf_counter()
    rc = lib.egs_selftest_wait_timeout(status.data_ptr(), out2.data_ptr(), ctypes.c_int64(limit),
                                       torch.cuda.current_stream(cuda_device).cuda_stream)
    _lib.check(rc, "egs_selftest_wait_timeout")
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert out2.tolist() == [1, 1]           # the wait reported failure and raised the CTA's abort flag
    assert 0.01 < elapsed < 2.0              # it cost its limit, not more
    assert int(status.item()) & _lib.STATUS_PIPELINE_TIMEOUT

    # a launch that finds the timeout bit set does no work (a broken pipeline must not cost one limit per wave)
    poisoned = ops.gather_gemm(torch.ones_like(d["X"]), d["Wg"], d["Ind"], path="tensor")
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded wait"):
        ops.check_status()
    del poisoned

    # the failed check cleared the word: the context is usable and results are right again
    again = ops.gather_gemm(d["X"], d["Wg"], d["Ind"], path="tensor")
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(again, good)
