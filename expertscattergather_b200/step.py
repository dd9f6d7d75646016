"""One explicit training step of the path: gather -> scatter -> loss = sum(Out * G) -> backward.

The six operator launches are issued directly (no autograd graph), in the order autograd would run them for
the reference's modules.  ``on_weight_grad(name, tensor)`` is called as soon as each weight gradient has been
enqueued, which is where a data-parallel caller starts that gradient's all-reduce so it overlaps the rest of
the backward pass.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import ops

__all__ = ["train_step", "takes_fused_pairs"]



def _is_capturing(stream: "torch.cuda.Stream") -> bool:
    with torch.cuda.stream(stream):
        return bool(torch.cuda.is_current_stream_capturing())


def _prefilled_outputs(X: torch.Tensor, T: int, n_out: int, main: "torch.cuda.Stream", dw_shapes=()):
    """Allocates Out [B,T,n_out] and dX (like X) and zero-fills them on the fill stream; returns the two tensors, an
    event for "Out is filled", one for "everything is filled", and zero-filled tensors of the shapes in ``dw_shapes``.

    The tensors come from the fill stream's own memory pool: nothing ties the fills to work already queued on the
    main stream or to the weight-gradient kernels on the side stream (the tail of the previous step), so they run
    under it.  The scatters then add into the zeros.  Inside a stream capture the fill stream first joins the capture
    through the main stream."""
    dev = X.device
    fills = ops.fill_stream(dev)
    if _is_capturing(main) and not _is_capturing(fills):
        fills.wait_stream(main)
    with torch.cuda.stream(fills):
        Out = torch.empty((X.shape[0], T, n_out), device=dev, dtype=X.dtype)
        dX = torch.empty_like(X, memory_format=torch.contiguous_format)
        Out.record_stream(main)
        dX.record_stream(main)
        ops.fill_zero(Out)
        out_filled = fills.record_event()
        ops.fill_zero(dX)
        # the weight gradients accumulate into zeros as well: filled here, long before their kernels are due
        dW0 = [ops.fill_zero(torch.empty(shape, device=dev, dtype=X.dtype)) for shape in dw_shapes]
        for t in dW0:
            t.record_stream(ops.side_stream(dev))
    return Out, dX, out_filled, fills.record_event(), dW0


def takes_fused_pairs(X: torch.Tensor, Wg: torch.Tensor, Ind: torch.Tensor) -> bool:
    """Whether :func:`train_step` runs G -> S and dY -> dX as one fused kernel each for these tensors."""
    return ops.fused_pair_preferred(X, Wg, Ind)


def train_step(X: torch.Tensor, Wg: torch.Tensor, Ws: torch.Tensor, Ind: torch.Tensor, G: torch.Tensor,
               on_weight_grad: Optional[Callable[[str, torch.Tensor], None]] = None, overlap: bool = True,
               fused_pairs: bool = True) -> dict:
    """X [B,T,I], Wg [E,I,J], Ws [E,J,I], Ind [B,E,K], G [B,T,I] (the gradient of the loss w.r.t. Out).

    Returns Y, Out, dY, dX, dWg, dWs.  Equivalent to
    ``Y = ExpertGather(X, Ind); Out = ExpertScatter(Y, Ind, T); (Out*G).sum().backward()``.

    With ``overlap`` the work that is off the critical chain G -> S -> dY -> dX runs on helper streams: the zero fills
    of float32 Out and dX on a fill stream (the scatters then add into the zeros; 16-bit outputs are initialised by
    the scatter's own planning step), the two weight-gradient kernels on a side stream, each started as soon as its
    inputs exist.  With ``on_weight_grad`` (the data-parallel case) the operators
    stay on one stream in an order that puts both weight gradients, and with them the start of their reductions,
    before the last scatter; only the fills run beside them.  With ``fused_pairs`` float32 shapes that the fused
    pair kernel takes run G -> S and dY -> dX as one kernel each.
    """
    T = X.shape[1]
    if on_weight_grad is not None:
        # data-parallel order: both weight gradients come before the long dX scatter, so that the reductions the
        # callback starts (dW_s first, then dW_g) run behind the kernels that are still to come
        main = torch.cuda.current_stream(X.device)
        Out = dX = None
        if X.dtype == torch.float32:
            Out, dX, out_filled, fills_done, _ = _prefilled_outputs(X, T, Ws.shape[2], main)
        Y = ops.gather_gemm(X, Wg, Ind, w_layout="cn")
        if Out is not None:
            main.wait_event(out_filled)
        Out = ops.gemm_scatter(Y, Ws, Ind, T, w_layout="cn", out=Out)
        dY = ops.gather_gemm(G, Ws, Ind, w_layout="nc")
        dWs = ops.dweight(G, Y, Ind, out_layout="direct_rows")
        on_weight_grad("Ws", dWs)
        dWg = ops.dweight(X, dY, Ind, out_layout="gathered_rows")
        on_weight_grad("Wg", dWg)
        if dX is not None:
            main.wait_event(fills_done)
        dX = ops.gemm_scatter(dY, Wg, Ind, T, w_layout="nc", out=dX)
        return {"Y": Y, "Out": Out, "dY": dY, "dX": dX, "dWg": dWg, "dWs": dWs}
    if not overlap:
        Y = ops.gather_gemm(X, Wg, Ind, w_layout="cn")                 # gather forward
        Out = ops.gemm_scatter(Y, Ws, Ind, T, w_layout="cn")           # scatter forward
        dY = ops.gather_gemm(G, Ws, Ind, w_layout="nc")                # scatter backward: dY
        dWs = ops.dweight(G, Y, Ind, out_layout="direct_rows")         # scatter backward: dW_s
        dX = ops.gemm_scatter(dY, Wg, Ind, T, w_layout="nc")           # gather backward: dX
        dWg = ops.dweight(X, dY, Ind, out_layout="gathered_rows")      # gather backward: dW_g
        return {"Y": Y, "Out": Out, "dY": dY, "dX": dX, "dWg": dWg, "dWs": dWs}

    dev = X.device
    main = torch.cuda.current_stream(dev)
    side = ops.side_stream(dev)
    # float32 outputs are zero-filled ahead of time on the fill stream; 16-bit outputs are initialised by the scatter's
    # own planning step (prefilling them measured slower where the scatter sums in float32 rows)
    prefill = X.dtype == torch.float32
    fused = fused_pairs and takes_fused_pairs(X, Wg, Ind)
    Out = dX = None
    dWs0 = dWg0 = None
    if prefill:
        Out, dX, out_filled, fills_done, (dWs0, dWg0) = _prefilled_outputs(
            X, T, Ws.shape[2], main, dw_shapes=(tuple(Ws.shape), tuple(Wg.shape)))
    if fused:
        # shapes the fused pair kernels take: two kernels on the critical chain instead of four
        if prefill:
            main.wait_event(out_filled)
        Y, Out = ops.gather_scatter_pair(X, Wg, Ws, Ind, w_layout="cn", out=Out)      # gather + scatter forward
        fwd_done = main.record_event()
        with torch.cuda.stream(side):
            side.wait_event(fwd_done)
            if prefill:
                side.wait_event(fills_done)
            dWs = ops.dweight(G, Y, Ind, out_layout="direct_rows", zeroed_out=dWs0)  # scatter backward: dW_s
            dWs.record_stream(main)
        if prefill:
            main.wait_event(fills_done)
        dY, dX = ops.gather_scatter_pair(G, Ws, Wg, Ind, w_layout="nc", out=dX)       # dY and dX
        dy_ready = main.record_event()
        with torch.cuda.stream(side):
            side.wait_event(dy_ready)
            dWg = ops.dweight(X, dY, Ind, out_layout="gathered_rows", zeroed_out=dWg0)   # gather backward: dW_g
            dWg.record_stream(main)
        main.wait_stream(side)
        return {"Y": Y, "Out": Out, "dY": dY, "dX": dX, "dWg": dWg, "dWs": dWs}
    Y = ops.gather_gemm(X, Wg, Ind, w_layout="cn")                     # gather forward
    if prefill:
        main.wait_event(out_filled)
    Out = ops.gemm_scatter(Y, Ws, Ind, T, w_layout="cn", out=Out)      # scatter forward (adds into zeros)
    fwd_done = main.record_event()
    with torch.cuda.stream(side):                                      # scatter backward: dW_s, next to dY
        side.wait_event(fwd_done)                                      # the backward pass starts after the forward
        if prefill:
            side.wait_event(fills_done)
        dWs = ops.dweight(G, Y, Ind, out_layout="direct_rows", zeroed_out=dWs0)
        dWs.record_stream(main)
    dY = ops.gather_gemm(G, Ws, Ind, w_layout="nc")                    # scatter backward: dY
    dy_ready = main.record_event()
    with torch.cuda.stream(side):                                      # gather backward: dW_g, next to dX
        side.wait_event(dy_ready)
        dWg = ops.dweight(X, dY, Ind, out_layout="gathered_rows", zeroed_out=dWg0)
        dWg.record_stream(main)
    if prefill:
        main.wait_event(fills_done)
    dX = ops.gemm_scatter(dY, Wg, Ind, T, w_layout="nc", out=dX)       # gather backward: dX
    main.wait_stream(side)                                             # join
    return {"Y": Y, "Out": Out, "dY": dY, "dX": dX, "dWg": dWg, "dWs": dWs}
