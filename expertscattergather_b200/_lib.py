"""ctypes binding of libegs_b200.so (the C-ABI library declared in include/egs_b200.h).

There is no CPU fallback: if the library cannot be loaded (and cannot be built because nvcc is absent)
importing the operators raises.
"""
from __future__ import annotations

import ctypes
import os
import threading

from . import build as _build

# enums of include/egs_b200.h
F32, F16, BF16 = 0, 1, 2
I16, I32, I64 = 0, 1, 2
PREC_STRICT, PREC_TF32 = 0, 1
PATH_AUTO, PATH_GENERIC, PATH_TENSOR, PATH_PAIRED = 0, 1, 2, 3
W_CN, W_NC = 0, 1
DW_GATHERED_ROWS, DW_DIRECT_ROWS = 0, 1
OK, ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE, ERR_TOO_LARGE = range(6)
STATUS_INDEX_OUT_OF_RANGE, STATUS_PIPELINE_TIMEOUT, STATUS_INTERNAL = 1, 2, 4

EXPORTS = (
    "egs_version", "egs_status_string", "egs_last_cuda_error", "egs_gather_gemm", "egs_gemm_scatter",
    "egs_dweight", "egs_dweight_static_scratch", "egs_static_scratch_max_elements", "egs_dw_workspace_bytes", "egs_scatter_workspace_bytes", "egs_tensor_path_eligible", "egs_fill_zero", "egs_launch_count",
    "egs_gather_scatter_pair", "egs_fused_pair_eligible", "egs_dweight_prezeroed", "egs_selftest_wait_timeout",
    "egs_describe_plan", "egs_gather_gemm_bias", "egs_gemm_scatter_bias", "egs_route_topk", "egs_index_csr",
    "egs_index_csr_scratch_bytes", "egs_index_compact", "egs_gemm_scatter_prepared", "egs_gemm_scatter_csr",
)


class Dims(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("B", "T", "E", "K", "C", "N")]


class PlanInfo(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("tensor_path", "tile_n", "stages", "row_tiles", "persistent", "bulk_epilogue",
                                            "expert_fastest", "splits", "rows_per_split")]


_lock = threading.Lock()
_lib = None


def _declare(lib: ctypes.CDLL) -> None:
    vp, i, i64, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t
    lib.egs_version.restype = i
    lib.egs_version.argtypes = []
    lib.egs_status_string.restype = ctypes.c_char_p
    lib.egs_status_string.argtypes = [i]
    lib.egs_last_cuda_error.restype = ctypes.c_char_p
    lib.egs_last_cuda_error.argtypes = []
    lib.egs_gather_gemm.restype = i
    lib.egs_gather_gemm.argtypes = [vp, vp, vp, vp, ctypes.POINTER(Dims), i, i, i, i, i, vp, vp]
    lib.egs_gemm_scatter.restype = i
    lib.egs_gemm_scatter.argtypes = [vp, vp, vp, vp, ctypes.POINTER(Dims), i, i, i, i, i, i, vp, sz, vp, vp]
    lib.egs_gather_gemm_bias.restype = i
    lib.egs_gather_gemm_bias.argtypes = [vp, vp, vp, vp, vp, ctypes.POINTER(Dims), i, i, i, i, i, vp, vp]
    lib.egs_gemm_scatter_bias.restype = i
    lib.egs_gemm_scatter_bias.argtypes = [vp, vp, vp, vp, vp, ctypes.POINTER(Dims), i, i, i, i, i, i, vp, sz, vp, vp]
    lib.egs_scatter_workspace_bytes.restype = sz
    lib.egs_scatter_workspace_bytes.argtypes = [i64, i64, i64, i]
    lib.egs_dweight.restype = i
    lib.egs_dweight.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i, i, i, i, i, vp, sz, vp, vp]
    lib.egs_selftest_wait_timeout.restype = i
    lib.egs_selftest_wait_timeout.argtypes = [vp, vp, i64, vp]
    lib.egs_dweight_prezeroed.restype = i
    lib.egs_dweight_prezeroed.argtypes = lib.egs_dweight.argtypes
    lib.egs_dweight_static_scratch.restype = i
    lib.egs_dweight_static_scratch.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i, i, i, i, i, vp, vp]
    lib.egs_static_scratch_max_elements.restype = sz
    lib.egs_static_scratch_max_elements.argtypes = []
    lib.egs_dw_workspace_bytes.restype = sz
    lib.egs_dw_workspace_bytes.argtypes = [i64, i64, i64, i]
    lib.egs_tensor_path_eligible.restype = i
    lib.egs_tensor_path_eligible.argtypes = [i, ctypes.POINTER(Dims), i, ctypes.POINTER(vp), i]
    lib.egs_route_topk.restype = i
    lib.egs_route_topk.argtypes = [vp, vp, i64, i64, i64, i64, i, vp]
    lib.egs_index_csr_scratch_bytes.restype = sz
    lib.egs_index_csr_scratch_bytes.argtypes = [i64, i64]
    lib.egs_index_csr.restype = i
    lib.egs_index_csr.argtypes = [vp, i, i64, i64, i64, i64, vp, vp, vp, vp, vp, sz, vp]
    lib.egs_index_compact.restype = i
    lib.egs_index_compact.argtypes = [vp, i, i64, i64, vp, i, vp, vp]
    lib.egs_gemm_scatter_prepared.restype = i
    lib.egs_gemm_scatter_prepared.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.POINTER(Dims), i, i, i, i, i, i, vp, sz, vp, vp]
    lib.egs_gemm_scatter_csr.restype = i
    lib.egs_gemm_scatter_csr.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.POINTER(Dims), i, i, i, vp]
    lib.egs_describe_plan.restype = i
    lib.egs_describe_plan.argtypes = [i, ctypes.POINTER(Dims), i, i, i, ctypes.POINTER(PlanInfo)]
    lib.egs_fill_zero.restype = i
    lib.egs_fill_zero.argtypes = [vp, sz, vp]
    lib.egs_launch_count.restype = i64
    lib.egs_launch_count.argtypes = []
    lib.egs_gather_scatter_pair.restype = i
    lib.egs_gather_scatter_pair.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i, i, i, i, i, vp, sz, vp, vp]
    lib.egs_fused_pair_eligible.restype = i
    lib.egs_fused_pair_eligible.argtypes = [i64, i64, i64, i, i, i]


def library_path() -> str:
    return os.environ.get("EGS_B200_LIBRARY", _build.LIB_PATH)


def load() -> ctypes.CDLL:
    """Loads (building first when the sources are newer and nvcc is present) and returns the library."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = library_path()
        if path == _build.LIB_PATH:
            try:
                if _build.needs_build():
                    _build.build()
            except Exception as exc:  # nvcc absent or compile error
                if not os.path.exists(path):
                    raise RuntimeError(
                        "libegs_b200.so is not built and could not be built here "
                        f"({exc}); run `python -m expertscattergather_b200.build` where nvcc is available") from exc
        if not os.path.exists(path):
            raise RuntimeError(f"libegs_b200.so not found at {path}")
        lib = ctypes.CDLL(path)
        _declare(lib)
        _lib = lib
        return lib


def check(code: int, what: str) -> None:
    """Turns a non-zero status of the C ABI into a Python exception."""
    if code == OK:
        return
    lib = load()
    text = lib.egs_status_string(code).decode()
    if code == ERR_CUDA:
        text += ": " + lib.egs_last_cuda_error().decode()
    if code in (ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_TOO_LARGE):
        raise ValueError(f"{what}: {text}")
    raise RuntimeError(f"{what}: {text}")
