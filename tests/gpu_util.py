"""Helpers shared by the GPU parity tests: run the CUDA path through the tensor-level C-ABI wrappers and
compare with the CPU oracle."""
import torch

from expertscattergather_b200 import ops
from expertscattergather_b200.step import train_step
from oracle import egs_oracle as orc

TOL = {"fp32": 1e-5, "tf32": 2e-2, "bf16": 3e-2, "fp16": 3e-2}
STEP_KEYS = ("Y", "Out", "dY", "dX", "dWg", "dWs")


def tol_for(dtype, precision):
    if dtype == torch.float32:
        return TOL["tf32"] if precision == "tf32" else TOL["fp32"]
    return TOL["bf16"] if dtype == torch.bfloat16 else TOL["fp16"]


def to_dev(d, dev):
    return {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


def gpu_step(ins, dev, path="auto", precision="strict"):
    """Full step through the explicit C-ABI-backed operators; returns CPU tensors."""
    old_path, old_prec = ops.get_path(), ops.get_precision()
    ops.set_path(path)
    ops.set_precision(precision)
    try:
        d = to_dev(ins, dev)
        out = train_step(d["X"], d["Wg"], d["Ws"], d["Ind"], d["G"])
        torch.cuda.synchronize(dev)
        ops.check_status(dev)
        return {k: v.cpu() for k, v in out.items()}
    finally:
        ops.set_path(old_path)
        ops.set_precision(old_prec)


def compare_step(got, ref, tol, keys=STEP_KEYS, what=""):
    errs = {k: orc.rel_err(got[k], ref[k]) for k in keys}
    bad = {k: e for k, e in errs.items() if not e <= tol}
    assert not bad, f"{what}: relative errors above {tol}: {bad} (all: {errs})"
    return errs


def eligible(ins):
    """Whether the tensor-core kernels take this case (row pitches multiples of 16 bytes)."""
    es = ins["X"].element_size()
    I, J = ins["X"].shape[-1], ins["Wg"].shape[-1]
    return (I * es) % 16 == 0 and (J * es) % 16 == 0
