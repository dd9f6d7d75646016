"""Tensor-level host API over the C ABI: the three operators G, S, D on torch CUDA tensors.

The functions allocate outputs with torch (so every buffer belongs to torch's caching allocator, as in the
reference's launch wrappers, ``egs/triton_kernels.py:375,408-409,457,491-492``), pass raw pointers, sizes
and the current CUDA stream to ``libegs_b200.so`` and return without synchronising.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

__all__ = ["gather_gemm", "gemm_scatter", "gather_scatter_pair", "fused_pair_eligible", "fused_pair_preferred", "dweight", "fill_zero", "side_stream", "fill_stream", "set_precision", "get_precision", "set_path", "get_path",
           "check_status", "reset_status", "publish_status", "launch_count", "dtype_to_type_id", "tensor_path_eligible", "describe_plan", "route_topk", "build_index_csr", "compact_index", "gemm_scatter_csr", "IndexCSR"]

_PRECISIONS = {"strict": _lib.PREC_STRICT, "fp32": _lib.PREC_STRICT, "tf32": _lib.PREC_TF32}
_PATHS = {"auto": _lib.PATH_AUTO, "generic": _lib.PATH_GENERIC, "tensor": _lib.PATH_TENSOR,
          "paired": _lib.PATH_PAIRED}     # "paired": per-call only, operator G on 16-bit tensors (see gather_gemm)
_SM_COUNT = 148     # B200

_state = {
    "precision": os.environ.get("EGS_B200_PRECISION", "strict").lower(),
    "path": os.environ.get("EGS_B200_PATH", "auto").lower(),
    "debug": os.environ.get("EGS_B200_DEBUG", "0") not in ("0", "", "false"),
}
_status_words: dict[int, torch.Tensor] = {}
_status_mirrors: dict[int, torch.Tensor] = {}     # pinned host copies of the status words (see publish_status)


def set_precision(mode: str) -> None:
    """'strict' (float32 products as accurate as fp32 FMA; the default, matching the reference's
    ``allow_tf32=False``, ``egs/triton_kernels.py:389``) or 'tf32' (single TF32 product)."""
    if mode not in _PRECISIONS:
        raise ValueError(f"unknown precision {mode!r}")
    _state["precision"] = mode


def get_precision() -> str:
    return _state["precision"]


def set_path(path: str) -> None:
    """'auto' (tensor-core kernels when the shape is eligible), 'generic' or 'tensor'."""
    if path not in _PATHS or path == "paired":
        raise ValueError(f"unknown path {path!r}")
    _state["path"] = path


def get_path() -> str:
    return _state["path"]


def dtype_to_type_id(dtype: torch.dtype) -> int:
    """float32 -> 0, float16 -> 1, bfloat16 -> 2; anything else raises ValueError("Unknown dtype"),
    as ``dtype_to_type_id`` in the reference does (``egs/triton_kernels.py:15-23``)."""
    if dtype == torch.float32:
        return _lib.F32
    if dtype == torch.float16:
        return _lib.F16
    if dtype == torch.bfloat16:
        return _lib.BF16
    raise ValueError("Unknown dtype")


def _index_tensor(Ind: torch.Tensor):
    if Ind.dtype == torch.int64:
        return Ind.contiguous(), _lib.I64
    if Ind.dtype == torch.int32:
        return Ind.contiguous(), _lib.I32
    if Ind.dtype == torch.int16:
        return Ind.contiguous(), _lib.I16
    if Ind.dtype in (torch.int8, torch.uint8):
        return Ind.to(torch.int32).contiguous(), _lib.I32
    raise ValueError(f"Ind must be an integer tensor, got {Ind.dtype}")


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = w
    return w


def reset_status(device=None) -> None:
    for idx, w in _status_words.items():
        if device is None or torch.device(device).index in (None, idx):
            w.zero_()
            m = _status_mirrors.get(idx)
            if m is not None:
                m.zero_()


def _status_text(idx: int, v: int) -> str:
    msgs = []
    if v & _lib.STATUS_INDEX_OUT_OF_RANGE:
        msgs.append("an Ind value outside [0, T) was met (slot skipped)")
    if v & _lib.STATUS_PIPELINE_TIMEOUT:
        msgs.append("a bounded wait inside a tensor-core kernel ran out (results invalid)")
    if v & _lib.STATUS_INTERNAL:
        msgs.append("a tensor-core kernel found its shared memory misaligned and did no work (results invalid)")
    return f"egs kernels on cuda:{idx} reported: " + "; ".join(msgs)


def publish_status(device) -> None:
    """Queues, on the current stream, a 4-byte copy of the device status word into a pinned host mirror.  No
    synchronisation: the mirror shows the word as of the last copy that has completed, and every operator call looks
    at it first (see ``_raise_if_flagged``).  The autograd functions and ``train_step`` call this once per backward
    pass / step, so a kernel that flagged a problem (above all a timed-out pipeline wait, after which the kernels skip
    their work) makes the next call raise instead of returning uninitialised memory."""
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    m = _status_mirrors.get(idx)
    if m is None:
        m = torch.zeros(1, dtype=torch.int32).pin_memory()
        _status_mirrors[idx] = m
    m.copy_(_status_word(torch.device("cuda", idx)), non_blocking=True)


def _raise_if_flagged(dev: torch.device) -> None:
    """Host-side look at the pinned mirror (no synchronisation).  Invalid-result bits raise and are cleared on both
    sides; an out-of-range index alone is left for ``check_status`` (the slot was skipped, results are defined)."""
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    m = _status_mirrors.get(idx)
    if m is None:
        return
    v = int(m[0])
    if v & (_lib.STATUS_PIPELINE_TIMEOUT | _lib.STATUS_INTERNAL):
        m.zero_()
        _status_words[idx].zero_()
        raise RuntimeError(_status_text(idx, v))


def check_status(device=None) -> None:
    """Reads the device status word(s) (synchronises) and raises if a kernel flagged a problem."""
    for idx, w in list(_status_words.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        v = int(w.item())
        if v:
            w.zero_()
            m = _status_mirrors.get(idx)
            if m is not None:
                m.zero_()
            raise RuntimeError(_status_text(idx, v))


_side_streams: dict[int, "torch.cuda.Stream"] = {}
_fill_streams: dict[int, "torch.cuda.Stream"] = {}


def side_stream(device) -> "torch.cuda.Stream":
    """A per-device helper stream on which independent work of one step (zero fills, weight gradients) is
    enqueued next to the main chain.  Users fork with ``side.wait_stream(current)`` and join with
    ``current.wait_stream(side)``."""
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    st = _side_streams.get(idx)
    if st is None:
        st = torch.cuda.Stream(torch.device("cuda", idx))
        _side_streams[idx] = st
    return st


def fill_stream(device) -> "torch.cuda.Stream":
    """A second per-device helper stream, for the zero fills of a step's outputs alone: kept apart from
    :func:`side_stream` so that the fills of the next step are not ordered behind the weight-gradient kernels of the
    current one."""
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    st = _fill_streams.get(idx)
    if st is None:
        st = torch.cuda.Stream(torch.device("cuda", idx))
        _fill_streams[idx] = st
    return st


def fill_zero(t: torch.Tensor) -> torch.Tensor:
    """Zero-fills a contiguous CUDA tensor with the library's fill kernel on the current stream."""
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("fill_zero needs a contiguous CUDA tensor")
    with torch.cuda.device(t.device):
        rc = _lib.load().egs_fill_zero(t.data_ptr(), t.numel() * t.element_size(), _stream_ptr(t.device))
    _lib.check(rc, "egs_fill_zero")
    return t


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(_lib.load().egs_launch_count())


def _require_cuda(*tensors) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("expert gather/scatter kernels need CUDA tensors (there is no CPU path)")
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same CUDA device")
    _raise_if_flagged(dev)
    return dev


def _stream_ptr(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _enums(precision, path):
    prec = _PRECISIONS[precision if precision is not None else _state["precision"]]
    pth = _PATHS[path if path is not None else _state["path"]]
    return prec, pth


def _w_dims(W: torch.Tensor, w_layout: str):
    if w_layout == "cn":
        return W.shape[0], W.shape[1], W.shape[2], _lib.W_CN
    if w_layout == "nc":
        return W.shape[0], W.shape[2], W.shape[1], _lib.W_NC
    raise ValueError("w_layout must be 'cn' ([E,C,N]) or 'nc' ([E,N,C])")


def _bias_rows(bias, E, N, dtype, dev):
    """A per-expert bias given as [E, N] or [E, 1, N] -> contiguous [E, N] of the tensors' dtype (None stays None)."""
    if bias is None:
        return None
    if bias.numel() != E * N or bias.shape[0] != E or bias.shape[-1] != N:
        raise ValueError(f"bias must be [E, N] or [E, 1, N] = [{E}, {N}], got {tuple(bias.shape)}")
    if not bias.is_cuda or bias.device != dev:
        raise RuntimeError("bias must be on the tensors' CUDA device")
    return bias.reshape(E, N).to(dtype).contiguous()


def gather_gemm(X, W, Ind, *, w_layout="cn", precision=None, path=None, bias=None):
    """Operator G: ``Y[b,e,k,:] = X[b, Ind[b,e,k], :] @ Wv[e] (+ bias[e])`` with ``Wv = W`` ('cn', W is [E,C,N]) or
    ``W^T`` per expert ('nc', W is [E,N,C]).  X [B,T,C] -> Y [B,E,K,N], dtype of X.  ``bias`` ([E,N] or [E,1,N]) is
    added in the kernel's epilogue.  ``path="paired"`` (16-bit tensors, N a multiple of 32 up to 256) runs the kernel on
    pairs of SMs (``EGS_PATH_PAIRED``); it raises for shapes that kernel does not take."""
    lib = _lib.load()
    if X.dim() != 3 or W.dim() != 3 or Ind.dim() != 3:
        raise ValueError("expected X[B,T,C], W[E,.,.], Ind[B,E,K]")
    dev = _require_cuda(X, W, Ind)
    if W.dtype != X.dtype:
        raise ValueError("X and W must have the same dtype")
    dt = dtype_to_type_id(X.dtype)
    E, C, N, wl = _w_dims(W, w_layout)
    B, T, Cx = X.shape
    Bi, Ei, K = Ind.shape
    if Cx != C or Ei != E or Bi != B:
        raise ValueError(f"shape mismatch: X{tuple(X.shape)} W{tuple(W.shape)} Ind{tuple(Ind.shape)} ({w_layout})")
    Xc, Wc = X.contiguous(), W.contiguous()
    Ic, it = _index_tensor(Ind)
    prec, pth = _enums(precision, path)
    with torch.cuda.device(dev):
        Y = torch.empty((B, E, K, N), device=dev, dtype=X.dtype)
        dims = _lib.Dims(B, T, E, K, C, N)
        bias_c = _bias_rows(bias, E, N, X.dtype, dev)
        if bias_c is None:
            rc = lib.egs_gather_gemm(Xc.data_ptr(), Wc.data_ptr(), Ic.data_ptr(), Y.data_ptr(), ctypes.byref(dims), wl, dt,
                                     it, prec, pth, _status_word(dev).data_ptr(), _stream_ptr(dev))
        else:
            rc = lib.egs_gather_gemm_bias(Xc.data_ptr(), Wc.data_ptr(), bias_c.data_ptr(), Ic.data_ptr(), Y.data_ptr(),
                                          ctypes.byref(dims), wl, dt, it, prec, pth, _status_word(dev).data_ptr(),
                                          _stream_ptr(dev))
    _lib.check(rc, "egs_gather_gemm")
    if _state["debug"]:
        check_status(dev)
    return Y


def gemm_scatter(Y, W, Ind, T, *, w_layout="cn", out=None, precision=None, path=None, bias=None, csr=None):
    """Operator S: ``Out[b, Ind[b,e,k], :] += Y[b,e,k,:] @ Wv[e] (+ bias[e])``; duplicates accumulate.
    Y [B,E,K,C] -> Out [B,T,N].  ``out=None`` allocates and zero-fills; a given ``out`` is added to.  ``bias`` ([E,N] or
    [E,1,N]) is added to every routed slot's product before it is scattered.  ``csr``: an :class:`IndexCSR` of this
    ``Ind`` - the 16-bit scatter then takes its choice between direct additions and float32 rows from it instead of
    counting the contributions per token row again."""
    lib = _lib.load()
    if Y.dim() != 4 or W.dim() != 3 or Ind.dim() != 3:
        raise ValueError("expected Y[B,E,K,C], W[E,.,.], Ind[B,E,K]")
    dev = _require_cuda(Y, W, Ind)
    if W.dtype != Y.dtype:
        raise ValueError("Y and W must have the same dtype")
    dt = dtype_to_type_id(Y.dtype)
    E, C, N, wl = _w_dims(W, w_layout)
    B, Ey, K, Cy = Y.shape
    if Cy != C or Ey != E or tuple(Ind.shape) != (B, E, K):
        raise ValueError(f"shape mismatch: Y{tuple(Y.shape)} W{tuple(W.shape)} Ind{tuple(Ind.shape)} ({w_layout})")
    T = int(T)
    Yc, Wc = Y.contiguous(), W.contiguous()
    Ic, it = _index_tensor(Ind)
    prec, pth = _enums(precision, path)
    with torch.cuda.device(dev):
        zero = 1
        if out is None:
            out = torch.empty((B, T, N), device=dev, dtype=Y.dtype)
        else:
            if tuple(out.shape) != (B, T, N) or out.dtype != Y.dtype or not out.is_contiguous():
                raise ValueError("out must be a contiguous [B,T,N] tensor of Y's dtype")
            zero = 0
        dims = _lib.Dims(B, T, E, K, C, N)
        ws_bytes = int(lib.egs_scatter_workspace_bytes(B, T, N, dt))
        ws = torch.empty(ws_bytes // 4, device=dev, dtype=torch.float32) if ws_bytes else None
        bias_c = _bias_rows(bias, E, N, Y.dtype, dev)
        if csr is not None:
            if (csr.B, csr.T, csr.E, csr.K) != (B, T, E, K):
                raise ValueError("the CSR was built for another Ind shape or T")
            rc = lib.egs_gemm_scatter_prepared(Yc.data_ptr(), Wc.data_ptr(), bias_c.data_ptr() if bias_c is not None else None,
                                               Ic.data_ptr(), csr.info.data_ptr(), out.data_ptr(), ctypes.byref(dims), wl, zero,
                                               dt, it, prec, pth, ws.data_ptr() if ws is not None else None, ws_bytes,
                                               _status_word(dev).data_ptr(), _stream_ptr(dev))
        elif bias_c is None:
            rc = lib.egs_gemm_scatter(Yc.data_ptr(), Wc.data_ptr(), Ic.data_ptr(), out.data_ptr(), ctypes.byref(dims), wl,
                                      zero, dt, it, prec, pth, ws.data_ptr() if ws is not None else None, ws_bytes,
                                      _status_word(dev).data_ptr(), _stream_ptr(dev))
        else:
            rc = lib.egs_gemm_scatter_bias(Yc.data_ptr(), Wc.data_ptr(), bias_c.data_ptr(), Ic.data_ptr(), out.data_ptr(),
                                           ctypes.byref(dims), wl, zero, dt, it, prec, pth,
                                           ws.data_ptr() if ws is not None else None, ws_bytes,
                                           _status_word(dev).data_ptr(), _stream_ptr(dev))
    _lib.check(rc, "egs_gemm_scatter")
    if _state["debug"]:
        check_status(dev)
    return out


def fused_pair_eligible(C1: int, N1: int, N2: int, dtype: torch.dtype, *, w_layout="cn", precision=None) -> bool:
    """True when :func:`gather_scatter_pair` has a kernel for this shape on the current device.  float32: the middle
    width a multiple of 32 and at most 256, the output width within one tile, tiles fitting in shared memory.
    16-bit: the middle width a multiple of 16 and at most 256, the other widths multiples of 8."""
    if dtype not in (torch.float32, torch.bfloat16, torch.float16) or _state["path"] == "generic":
        return False
    lib = _lib.load()
    prec, _ = _enums(precision, None)
    wl = _lib.W_CN if w_layout == "cn" else _lib.W_NC
    return bool(lib.egs_fused_pair_eligible(int(C1), int(N1), int(N2), wl, dtype_to_type_id(dtype), prec))


def fused_pair_preferred(X: torch.Tensor, Wg: torch.Tensor, Ind: torch.Tensor) -> bool:
    """Whether gather -> scatter over these tensors should run as the fused kernel by default.

    float32: a shape the kernel takes in both weight layouts and a grid of at most one wave (one CTA per (expert, 128
    expert rows) and per SM; beyond that the two separate kernels, which fit two CTAs per SM, measured faster).
    16-bit: never by default.  The persistent 16-bit pair kernel is correct and saves the round trip of the middle
    tensor, but both it and the separate kernels are bound by the bytes the SMs pull from L2 per 128-row tile, and
    the separate gather kernel halves those with 256-row tiles: whole steps measured 2 % faster to 14 % slower with
    the fused kernel (B200, bf16 configurations).  ``gather_scatter_pair`` runs it on request."""
    if not X.is_cuda or X.dtype != torch.float32:
        return False
    I, J = X.shape[2], Wg.shape[2]
    pair_ctas = Wg.shape[0] * ((X.shape[0] * Ind.shape[2] + 127) // 128)
    if pair_ctas > _SM_COUNT:
        return False
    return (fused_pair_eligible(I, J, I, X.dtype, w_layout="cn")
            and fused_pair_eligible(I, J, I, X.dtype, w_layout="nc"))


def gather_scatter_pair(Src, W1, W2, Ind, *, w_layout="cn", out=None, precision=None):
    """Operators G and S back to back in one kernel: ``Mid = gather(Src) @ W1v[e]`` (returned, [B,E,K,N1]) and
    ``Dst[b, Ind[b,e,k], :] += Mid[b,e,k,:] @ W2v[e]`` ([B,T,N2]); both weights in the same layout.

    Forward: ``gather_scatter_pair(X, W_g, W_s, Ind)`` -> (Y, Out).  Backward: ``gather_scatter_pair(dOut, W_s, W_g,
    Ind, w_layout="nc")`` -> (dY, dX).  ``out=None`` allocates and zero-fills Dst; a given ``out`` is added to.
    Raises when the shape is not eligible (see :func:`fused_pair_eligible`): callers then use the two operators."""
    lib = _lib.load()
    if Src.dim() != 3 or W1.dim() != 3 or W2.dim() != 3 or Ind.dim() != 3:
        raise ValueError("expected Src[B,T,C1], W1[E,.,.], W2[E,.,.], Ind[B,E,K]")
    dev = _require_cuda(Src, W1, W2, Ind)
    if W1.dtype != Src.dtype or W2.dtype != Src.dtype:
        raise ValueError("Src, W1 and W2 must have the same dtype")
    dt = dtype_to_type_id(Src.dtype)
    E, C1, N1, wl = _w_dims(W1, w_layout)
    E2, N1b, N2, _ = _w_dims(W2, w_layout)
    B, T, Cx = Src.shape
    Bi, Ei, K = Ind.shape
    if Cx != C1 or E2 != E or N1b != N1 or Ei != E or Bi != B:
        raise ValueError(f"shape mismatch: Src{tuple(Src.shape)} W1{tuple(W1.shape)} W2{tuple(W2.shape)} "
                         f"Ind{tuple(Ind.shape)} ({w_layout})")
    Sc, W1c, W2c = Src.contiguous(), W1.contiguous(), W2.contiguous()
    Ic, it = _index_tensor(Ind)
    prec, _ = _enums(precision, None)
    with torch.cuda.device(dev):
        Mid = torch.empty((B, E, K, N1), device=dev, dtype=Src.dtype)
        zero = 1
        if out is None:
            out = torch.empty((B, T, N2), device=dev, dtype=Src.dtype)
        else:
            if tuple(out.shape) != (B, T, N2) or out.dtype != Src.dtype or not out.is_contiguous():
                raise ValueError("out must be a contiguous [B,T,N2] tensor of Src's dtype")
            zero = 0
        ws_bytes = int(lib.egs_scatter_workspace_bytes(B, T, N2, dt))
        ws = torch.empty(ws_bytes // 4, device=dev, dtype=torch.float32) if ws_bytes else None
        rc = lib.egs_gather_scatter_pair(Sc.data_ptr(), W1c.data_ptr(), W2c.data_ptr(), Ic.data_ptr(), Mid.data_ptr(),
                                         out.data_ptr(), B, T, E, K, C1, N1, N2, wl, zero, dt, it, prec,
                                         ws.data_ptr() if ws is not None else None, ws_bytes,
                                         _status_word(dev).data_ptr(), _stream_ptr(dev))
    _lib.check(rc, "egs_gather_scatter_pair")
    if _state["debug"]:
        check_status(dev)
    return Mid, out


def dweight(Xsrc, Ysrc, Ind, *, out_layout="gathered_rows", precision=None, path=None, zeroed_out=None):
    """Operator D: ``P[e,f,g] = sum_{b,k} Xsrc[b, Ind[b,e,k], f] * Ysrc[b,e,k,g]``.
    'gathered_rows' returns P [E,FG,FD]; 'direct_rows' returns P^T [E,FD,FG].
    ``zeroed_out``: an output tensor the caller has already zero-filled (float32 only) - the library then skips its
    own fill, which lets a caller issue the fill early, off the critical path."""
    lib = _lib.load()
    if Xsrc.dim() != 3 or Ysrc.dim() != 4 or Ind.dim() != 3:
        raise ValueError("expected Xsrc[B,T,FG], Ysrc[B,E,K,FD], Ind[B,E,K]")
    dev = _require_cuda(Xsrc, Ysrc, Ind)
    if Xsrc.dtype != Ysrc.dtype:
        raise ValueError("Xsrc and Ysrc must have the same dtype")
    dt = dtype_to_type_id(Xsrc.dtype)
    B, T, FG = Xsrc.shape
    By, E, K, FD = Ysrc.shape
    if By != B or tuple(Ind.shape) != (B, E, K):
        raise ValueError(f"shape mismatch: Xsrc{tuple(Xsrc.shape)} Ysrc{tuple(Ysrc.shape)} Ind{tuple(Ind.shape)}")
    if out_layout == "gathered_rows":
        ol, shape = _lib.DW_GATHERED_ROWS, (E, FG, FD)
    elif out_layout == "direct_rows":
        ol, shape = _lib.DW_DIRECT_ROWS, (E, FD, FG)
    else:
        raise ValueError("out_layout must be 'gathered_rows' or 'direct_rows'")
    Xc, Yc = Xsrc.contiguous(), Ysrc.contiguous()
    Ic, it = _index_tensor(Ind)
    prec, pth = _enums(precision, path)
    with torch.cuda.device(dev):
        fn = lib.egs_dweight
        if zeroed_out is not None:
            if (tuple(zeroed_out.shape) != shape or zeroed_out.dtype != torch.float32 or Xsrc.dtype != torch.float32
                    or not zeroed_out.is_contiguous()):
                raise ValueError("zeroed_out must be a contiguous float32 tensor of the output's shape")
            out, fn = zeroed_out, lib.egs_dweight_prezeroed
        else:
            out = torch.empty(shape, device=dev, dtype=Xsrc.dtype)
        ws_bytes = int(lib.egs_dw_workspace_bytes(E, FG, FD, dt))
        ws = torch.empty(ws_bytes // 4, device=dev, dtype=torch.float32) if ws_bytes else None
        rc = fn(Xc.data_ptr(), Yc.data_ptr(), Ic.data_ptr(), out.data_ptr(), B, T, E, K, FG, FD, ol, dt, it,
                             prec, pth, ws.data_ptr() if ws is not None else None, ws_bytes,
                             _status_word(dev).data_ptr(), _stream_ptr(dev))
    _lib.check(rc, "egs_dweight")
    if _state["debug"]:
        check_status(dev)
    return out


def describe_plan(op: str, B, T, E, K, C, N, dtype, *, w_layout="cn", precision=None) -> dict:
    """The kernel variant 'auto' runs for operator op ('G', 'S' or 'D'; for D pass C = FG, N = FD) at these sizes:
    dict with tensor_path, tile_n, stages, row_tiles, persistent, bulk_epilogue, expert_fastest, splits, rows_per_split."""
    lib = _lib.load()
    dims = _lib.Dims(B, T, E, K, C, N)
    info = _lib.PlanInfo()
    prec, _ = _enums(precision, None)
    rc = lib.egs_describe_plan({"G": 0, "S": 1, "D": 2}[op], ctypes.byref(dims), _lib.W_CN if w_layout == "cn" else _lib.W_NC,
                               dtype_to_type_id(dtype), prec, ctypes.byref(info))
    _lib.check(rc, "egs_describe_plan")
    return {n: int(getattr(info, n)) for n, _ in _lib.PlanInfo._fields_}


_TORCH_INDEX = {torch.int64: _lib.I64, torch.int32: _lib.I32, torch.int16: _lib.I16}


def route_topk(scores: torch.Tensor, K: int, *, index_dtype: torch.dtype = torch.int64) -> torch.Tensor:
    """Expert-choice routing on the device: ``scores`` [B,T,E] -> ``Ind`` [B,E,K], for every (b, e) the K tokens with the
    highest score, best first (equal scores: lower token id first).  K <= min(T, 1024).  The producer of the ``Ind`` the
    gather and scatter modules take; the reference has none (its tests draw Ind at random, ``test_all.py:16``)."""
    lib = _lib.load()
    if scores.dim() != 3:
        raise ValueError("expected scores[B,T,E]")
    dev = _require_cuda(scores)
    if index_dtype not in _TORCH_INDEX:
        raise ValueError("index_dtype must be int64, int32 or int16")
    B, T, E = scores.shape
    sc = scores.float().contiguous()
    with torch.cuda.device(dev):
        Ind = torch.empty((B, E, int(K)), device=dev, dtype=index_dtype)
        rc = lib.egs_route_topk(sc.data_ptr(), Ind.data_ptr(), B, T, E, int(K), _TORCH_INDEX[index_dtype], _stream_ptr(dev))
    _lib.check(rc, "egs_route_topk")
    return Ind


class IndexCSR:
    """Token-major view of an ``Ind`` [B,E,K] built on the device by :func:`build_index_csr`: ``counts`` [B*T] slots per
    token row, ``offsets`` [B*T+1], ``entries`` [B*E*K] slot ids grouped by token row (ascending inside a row), ``info``
    [4] = (heaviest row, rows touched, out-of-range flag, valid slots); all int32 CUDA tensors."""

    def __init__(self, counts, offsets, entries, info, B, T, E, K):
        self.counts, self.offsets, self.entries, self.info = counts, offsets, entries, info
        self.B, self.T, self.E, self.K = B, T, E, K

    def summary(self) -> dict:
        """Reads ``info`` back (synchronises)."""
        v = self.info.tolist()
        return {"max_per_row": v[0], "rows_touched": v[1], "out_of_range": bool(v[2]), "valid_slots": v[3]}


def build_index_csr(Ind: torch.Tensor, T: int) -> IndexCSR:
    """Counting sort of the routed slots by token row (see :class:`IndexCSR`).  Build it once per step: it serves both
    scatters of the step (``gemm_scatter(..., csr=...)`` skips its own counting pass) and :func:`gemm_scatter_csr`."""
    lib = _lib.load()
    if Ind.dim() != 3:
        raise ValueError("expected Ind[B,E,K]")
    dev = _require_cuda(Ind)
    B, E, K = Ind.shape
    T = int(T)
    Ic, it = _index_tensor(Ind)
    with torch.cuda.device(dev):
        counts = torch.empty(B * T, device=dev, dtype=torch.int32)
        offsets = torch.empty(B * T + 1, device=dev, dtype=torch.int32)
        entries = torch.empty(B * E * K, device=dev, dtype=torch.int32)
        info = torch.empty(4, device=dev, dtype=torch.int32)
        sb = int(lib.egs_index_csr_scratch_bytes(B, T))
        scratch = torch.empty((sb + 3) // 4, device=dev, dtype=torch.int32)
        rc = lib.egs_index_csr(Ic.data_ptr(), it, B, T, E, K, counts.data_ptr(), offsets.data_ptr(), entries.data_ptr(),
                               info.data_ptr(), scratch.data_ptr(), sb, _stream_ptr(dev))
    _lib.check(rc, "egs_index_csr")
    return IndexCSR(counts, offsets, entries, info, B, T, E, K)


def compact_index(Ind: torch.Tensor, T: int, dtype: torch.dtype) -> torch.Tensor:
    """``Ind`` in a narrower (or wider) integer type, converted on the device; ids outside [0,T) are reported through the
    status word.  T must fit the target type (int16: T <= 32767)."""
    lib = _lib.load()
    dev = _require_cuda(Ind)
    if dtype not in _TORCH_INDEX:
        raise ValueError("dtype must be int64, int32 or int16")
    Ic, it = _index_tensor(Ind)
    with torch.cuda.device(dev):
        out = torch.empty(Ic.shape, device=dev, dtype=dtype)
        rc = lib.egs_index_compact(Ic.data_ptr(), it, Ic.numel(), int(T), out.data_ptr(), _TORCH_INDEX[dtype],
                                   _status_word(dev).data_ptr(), _stream_ptr(dev))
    _lib.check(rc, "egs_index_compact")
    return out


def gemm_scatter_csr(Y, W, csr: IndexCSR, *, w_layout="cn", out=None, bias=None):
    """Operator S evaluated token-major from a CSR: every token row is summed in a fixed order by one CTA and stored (zeros
    where nothing is routed): no atomics, no zero fill, the same bits on every run.  ``out`` given: added to.  Slower than
    :func:`gemm_scatter` except for small contractions (it re-reads W[e] per contribution); N <= 1024."""
    lib = _lib.load()
    if Y.dim() != 4 or W.dim() != 3:
        raise ValueError("expected Y[B,E,K,C], W[E,.,.]")
    dev = _require_cuda(Y, W, csr.entries)
    if W.dtype != Y.dtype:
        raise ValueError("Y and W must have the same dtype")
    dt = dtype_to_type_id(Y.dtype)
    E, C, N, wl = _w_dims(W, w_layout)
    B, Ey, K, Cy = Y.shape
    if (B, Ey, K) != (csr.B, csr.E, csr.K) or Cy != C or Ey != E:
        raise ValueError("Y, W and the CSR do not describe the same problem")
    Yc, Wc = Y.contiguous(), W.contiguous()
    with torch.cuda.device(dev):
        acc = 0
        if out is None:
            out = torch.empty((B, csr.T, N), device=dev, dtype=Y.dtype)
        else:
            if tuple(out.shape) != (B, csr.T, N) or out.dtype != Y.dtype or not out.is_contiguous():
                raise ValueError("out must be a contiguous [B,T,N] tensor of Y's dtype")
            acc = 1
        bias_c = _bias_rows(bias, E, N, Y.dtype, dev)
        dims = _lib.Dims(B, csr.T, E, K, C, N)
        rc = lib.egs_gemm_scatter_csr(Yc.data_ptr(), Wc.data_ptr(), bias_c.data_ptr() if bias_c is not None else None,
                                      csr.offsets.data_ptr(), csr.entries.data_ptr(), out.data_ptr(), ctypes.byref(dims), wl,
                                      acc, dt, _stream_ptr(dev))
    _lib.check(rc, "egs_gemm_scatter_csr")
    return out


def tensor_path_eligible(op: str, B, T, E, K, C, N, dtype, tensors=()) -> bool:
    """True if 'auto' would run the tcgen05 kernels for operator op ('G', 'S' or 'D') at these sizes."""
    lib = _lib.load()
    dims = _lib.Dims(B, T, E, K, C, N)
    ptrs = (ctypes.c_void_p * max(1, len(tensors)))(*[t.data_ptr() for t in tensors])
    return bool(lib.egs_tensor_path_eligible({"G": 0, "S": 1, "D": 2}[op], ctypes.byref(dims), dtype_to_type_id(dtype),
                                             ptrs, len(tensors)))
