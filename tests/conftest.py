import glob
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")

# parity tolerances, as max|a-ref| / max|ref|
TOL = {"fp32": 1e-5, "tf32": 2e-2, "bf16": 3e-2, "fp16": 3e-2}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def golden_names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load_golden(name):
    """Returns (inputs as torch tensors in the case's dtype, reference outputs as float32 numpy, T, dtype)."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[str(z["dtype"])]
    ins = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in_")}
    for k in list(ins):
        if k != "Ind":
            ins[k] = ins[k].to(dtype)
    refs = {k[4:]: z[k] for k in z.files if k.startswith("ref_")}
    return ins, refs, int(z["T"]), dtype


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
