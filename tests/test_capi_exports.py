"""The C-ABI library loads and exports every function include/egs_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from expertscattergather_b200 import _lib

HEADER = os.path.join(ROOT, "include", "egs_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(egs_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    assert set(_lib.EXPORTS) == set(names), names


@pytest.mark.parametrize("name", declared_functions())
def test_symbol_is_exported(name):
    lib = _lib.load()
    assert getattr(lib, name) is not None


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.egs_version() >= 100
    assert lib.egs_status_string(0) == b"ok"
    for code in range(1, 6):
        assert lib.egs_status_string(code) not in (b"ok", b"unknown status")
    assert lib.egs_status_string(99) == b"unknown status"
    assert lib.egs_launch_count() >= 0


def test_argument_validation_needs_no_gpu():
    lib = _lib.load()
    # null dims / bad enums are rejected before anything touches CUDA
    assert lib.egs_gather_gemm(None, None, None, None, None, 0, 0, 0, 0, 0, None, None) == _lib.ERR_INVALID_ARGUMENT
    d = _lib.Dims(1, 1, 1, 1, 4, 4)
    assert lib.egs_gather_gemm(None, None, None, None, ctypes.byref(d), 7, 0, 0, 0, 0, None, None) == \
        _lib.ERR_INVALID_ARGUMENT
    assert lib.egs_gemm_scatter(None, None, None, None, ctypes.byref(d), 0, 1, 9, 0, 0, 0, None, 0, None, None) == \
        _lib.ERR_INVALID_ARGUMENT
    neg = _lib.Dims(-1, 1, 1, 1, 4, 4)
    assert lib.egs_gather_gemm(None, None, None, None, ctypes.byref(neg), 0, 0, 0, 0, 0, None, None) == \
        _lib.ERR_INVALID_ARGUMENT
    big = _lib.Dims(1 << 20, 1 << 20, 1, 1, 4, 4)
    assert lib.egs_gather_gemm(None, None, None, None, ctypes.byref(big), 0, 0, 0, 0, 0, None, None) == \
        _lib.ERR_TOO_LARGE
    # empty problems succeed without launching
    empty = _lib.Dims(0, 4, 2, 3, 4, 4)
    assert lib.egs_gather_gemm(None, None, None, None, ctypes.byref(empty), 0, 0, 0, 0, 0, None, None) == _lib.OK
    assert lib.egs_dweight(None, None, None, None, 2, 4, 0, 3, 4, 4, 0, 0, 0, 0, 0, None, 0, None, None) == _lib.OK
    assert lib.egs_dweight(None, None, None, None, 2, 4, 2, 3, 4, 4, 5, 0, 0, 0, 0, None, 0, None, None) == \
        _lib.ERR_INVALID_ARGUMENT
    assert lib.egs_fill_zero(None, 0, None) == _lib.OK
    assert lib.egs_fill_zero(None, 16, None) == _lib.ERR_INVALID_ARGUMENT


def test_workspace_size_rule():
    lib = _lib.load()
    assert lib.egs_dw_workspace_bytes(4, 8, 16, _lib.F32) == 0
    assert lib.egs_dw_workspace_bytes(4, 8, 16, _lib.BF16) == 4 * 8 * 16 * 4
    assert lib.egs_dw_workspace_bytes(0, 8, 16, _lib.BF16) == 0
    assert lib.egs_scatter_workspace_bytes(2, 8, 16, _lib.F32) == 0
    assert lib.egs_scatter_workspace_bytes(2, 8, 16, _lib.F16) == 256 + 256 + 2 * 8 * 16 * 4
