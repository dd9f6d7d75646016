"""Autograd functions and dispatcher ops of the expert gather / scatter path.

Host-side mirror of the reference's L1 layer (``egs/triton_kernels.py:358-639``): the same four
dispatcher ops in namespace ``mylib`` with the same schemas (``:362,395,444,478``), the same fake
(shape-propagation) registrations for ``torch.compile`` (``:527-567``), the same module-level handles
``expert_{gather,scatter}_{forward,backward}_call`` (``:26-29,569-578``), ``create_kernels()`` and the two
``torch.autograd.Function`` classes (``:581-639``).  The bodies call the sm_100a kernels of
``libegs_b200.so`` instead of Triton; there is no autotuning and no CPU path.

Differences from the reference, on purpose:
* the scatter forward output is zero-filled (the reference allocates it with ``torch.empty`` and only
  adds to it, ``:457``);
* non-contiguous inputs (for example the stride-0 gradient of ``.sum()``) are made contiguous first;
* ``out_dtype`` is accepted and ignored exactly like the reference ignores it: tensors are read in their own
  dtype, accumulated in float32 and written in the input dtype (``:375,457``).
"""
from __future__ import annotations

import torch

from . import ops

__all__ = ["create_kernels", "ExpertGatherFunction", "ExpertScatterFunction", "ExpertGatherScatterFunction",
           "ExpertGatherBiasFunction", "ExpertScatterBiasFunction", "dtype_to_type_id",
           "expert_gather_forward_call", "expert_gather_backward_call", "expert_scatter_forward_call",
           "expert_scatter_backward_call", "OP_NAMESPACE"]

dtype_to_type_id = ops.dtype_to_type_id

expert_gather_forward_call = None
expert_gather_backward_call = None
expert_scatter_forward_call = None
expert_scatter_backward_call = None
OP_NAMESPACE = None


# ---- op bodies ---------------------------------------------------------------------------------------

def _gather_forward(X, W, Ind, out_dtype):
    # Y = gather(X) @ W_g                                      (reference: egs/triton_kernels.py:367-392)
    return ops.gather_gemm(X, W, Ind, w_layout="cn")


def _weight_grad_on_side_stream(Xsrc, Ysrc, Ind, out_layout):
    """Enqueues operator D on the helper stream (it is independent of the dX / dY kernel of the same backward
    call, and the two co-reside on the SMs); the caller joins with ``_join_side``."""
    dev = Xsrc.device
    main = torch.cuda.current_stream(dev)
    side = ops.side_stream(dev)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        grad_W = ops.dweight(Xsrc, Ysrc, Ind, out_layout=out_layout)
        grad_W.record_stream(main)
    return grad_W


def _join_side(t):
    """Joins the helper stream and queues the copy of the status word to its host mirror: once per backward call, after
    its kernels, so that the next operator call raises if one of them reported invalid results."""
    torch.cuda.current_stream(t.device).wait_stream(ops.side_stream(t.device))
    ops.publish_status(t.device)


def _gather_backward(X, W, Ind, grad_output, out_dtype):
    # dX = scatter(dY @ W_g^T), dW_g = gather(X)^T @ dY        (reference: egs/triton_kernels.py:400-441)
    T = X.shape[1]
    grad_output = grad_output.contiguous()
    grad_W = _weight_grad_on_side_stream(X, grad_output, Ind, "gathered_rows")
    grad_X = ops.gemm_scatter(grad_output, W, Ind, T, w_layout="nc")
    _join_side(grad_X)
    return grad_X, grad_W


def _scatter_forward(Y, W, Ind, T, out_dtype):
    # Out = scatter(Y @ W_s)                                   (reference: egs/triton_kernels.py:449-474)
    return ops.gemm_scatter(Y, W, Ind, T, w_layout="cn")


def _scatter_backward(Y, W, Ind, grad_X, out_dtype):
    # dY = gather(dOut) @ W_s^T, dW_s = Y^T @ gather(dOut)     (reference: egs/triton_kernels.py:483-525)
    grad_X = grad_X.contiguous()
    grad_W = _weight_grad_on_side_stream(grad_X, Y, Ind, "direct_rows")
    grad_Y = ops.gather_gemm(grad_X, W, Ind, w_layout="nc")
    _join_side(grad_Y)
    return grad_Y, grad_W


# ---- fake (meta) implementations: shapes and dtypes only --------------------------------------------

def _gather_forward_fake(X, W, Ind, out_dtype):
    return X.new_empty((X.shape[0], W.shape[0], Ind.shape[2], W.shape[2]))


def _gather_backward_fake(X, W, Ind, grad_output, out_dtype):
    return torch.empty_like(X), torch.empty_like(W)


def _scatter_forward_fake(Y, W, Ind, T, out_dtype):
    return Y.new_empty((Y.shape[0], T, W.shape[2]))


def _scatter_backward_fake(Y, W, Ind, grad_X, out_dtype):
    return torch.empty_like(Y), torch.empty_like(W)


_SCHEMAS = {
    "expert_gather_forward_call_fn": ("(Tensor X, Tensor W, Tensor Ind, ScalarType out_dtype) -> Tensor",
                                      _gather_forward, _gather_forward_fake),
    "expert_gather_backward_call_fn": ("(Tensor X, Tensor W, Tensor Ind, Tensor grad_output, ScalarType out_dtype)"
                                       " -> (Tensor, Tensor)", _gather_backward, _gather_backward_fake),
    "expert_scatter_forward_call_fn": ("(Tensor Y, Tensor W, Tensor Ind, int T, ScalarType out_dtype) -> Tensor",
                                       _scatter_forward, _scatter_forward_fake),
    "expert_scatter_backward_call_fn": ("(Tensor Y, Tensor W, Tensor Ind, Tensor grad_X, ScalarType out_dtype)"
                                        " -> (Tensor, Tensor)", _scatter_backward, _scatter_backward_fake),
}


def _define_ops(namespace: str) -> None:
    for name, (schema, impl, fake) in _SCHEMAS.items():
        qual = f"{namespace}::{name}"
        torch.library.define(qual, schema)
        torch.library.impl(qual, "default")(impl)
        torch.library.register_fake(qual)(fake)


def create_kernels() -> None:
    """Defines the four dispatcher ops once per process and binds the module-level call handles.

    Same role and guard as the reference's ``create_kernels`` (``egs/triton_kernels.py:32-36``); here there is
    nothing to JIT, so it only registers the ops.  If another library already owns ``mylib::expert_*`` in this
    process (the reference itself), the ops are registered under ``egs_b200`` instead.
    """
    global expert_gather_forward_call, expert_gather_backward_call
    global expert_scatter_forward_call, expert_scatter_backward_call, OP_NAMESPACE
    if expert_gather_forward_call is not None:
        return
    namespace = "mylib"
    try:
        _define_ops(namespace)
    except RuntimeError:
        namespace = "egs_b200"
        _define_ops(namespace)
    lib = getattr(torch.ops, namespace)
    OP_NAMESPACE = namespace
    expert_gather_forward_call = lib.expert_gather_forward_call_fn
    expert_gather_backward_call = lib.expert_gather_backward_call_fn
    expert_scatter_forward_call = lib.expert_scatter_forward_call_fn
    expert_scatter_backward_call = lib.expert_scatter_backward_call_fn


class ExpertGatherFunction(torch.autograd.Function):
    """``Y[b,e,k,j] = sum_i X[b, Ind[b,e,k], i] * W[e,i,j]`` with X [B,T,I], W [E,I,J], Ind [B,E,K].

    Same call signature and return convention as the reference class (``egs/triton_kernels.py:581-608``):
    ``apply(X, W, Ind, out_type=torch.float32)``; backward returns ``(grad_X, grad_W, None, None)``.  The reference
    always computes both gradients (``:603-608``); here a gradient autograd does not ask for (``needs_input_grad``: a
    frozen weight, an input that is data) is not computed.
    """

    @staticmethod
    def forward(ctx, X, W, Ind, out_type=torch.float32):
        create_kernels()
        ctx.save_for_backward(X, W, Ind)
        ctx.dtype = out_type
        return expert_gather_forward_call(X, W, Ind, out_type)

    @staticmethod
    def backward(ctx, grad_output):
        X, W, Ind = ctx.saved_tensors
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if need_x and need_w:
            grad_X, grad_W = expert_gather_backward_call(X, W, Ind, grad_output, ctx.dtype)
            return grad_X, grad_W, None, None
        grad_output = grad_output.contiguous()
        grad_X = ops.gemm_scatter(grad_output, W, Ind, X.shape[1], w_layout="nc") if need_x else None
        grad_W = ops.dweight(X, grad_output, Ind, out_layout="gathered_rows") if need_w else None
        return grad_X, grad_W, None, None


class ExpertScatterFunction(torch.autograd.Function):
    """``Out[b,t,i] = sum_{e,k: Ind[b,e,k]=t} sum_j Y[b,e,k,j] * W[e,j,i]`` with Y [B,E,K,J], W [E,J,I].

    Same call signature as the reference class (``egs/triton_kernels.py:610-639``):
    ``apply(Y, W, Ind, T, out_type=torch.float32)``; backward returns ``(grad_Y, grad_W, None, None, None)``; a
    gradient autograd does not ask for is not computed (the reference always computes both, ``:634-639``).
    """

    @staticmethod
    def forward(ctx, Y, W, Ind, T, out_type=torch.float32):
        create_kernels()
        ctx.save_for_backward(Y, W, Ind)
        ctx.dtype = out_type
        return expert_scatter_forward_call(Y, W, Ind, int(T), out_type)

    @staticmethod
    def backward(ctx, grad_X):
        Y, W, Ind = ctx.saved_tensors
        need_y, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if need_y and need_w:
            grad_Y, grad_W = expert_scatter_backward_call(Y, W, Ind, grad_X, ctx.dtype)
            return grad_Y, grad_W, None, None, None
        grad_X = grad_X.contiguous()
        grad_Y = ops.gather_gemm(grad_X, W, Ind, w_layout="nc") if need_y else None
        grad_W = ops.dweight(grad_X, Y, Ind, out_layout="direct_rows") if need_w else None
        return grad_Y, grad_W, None, None, None


class ExpertGatherBiasFunction(torch.autograd.Function):
    """``ExpertGatherFunction`` with the per-expert bias of ``ExpertGather(bias=True)`` added in the kernel's epilogue:
    ``Y[b,e,k,:] = X[b, Ind[b,e,k], :] @ W[e] + bias[e]`` with bias [E,1,J] - what the reference computes as
    ``ExpertGatherFunction.apply(...) + self.bias`` (``egs/torch_interface.py:54-56``).  ``apply(X, W, bias, Ind)``;
    backward returns ``(grad_X, grad_W, grad_bias, None)``, grad_bias = the sum of grad_output over batch and slot."""

    @staticmethod
    def forward(ctx, X, W, bias, Ind):
        ctx.save_for_backward(X, W, Ind)
        ctx.bias_shape = tuple(bias.shape)
        return ops.gather_gemm(X, W, Ind, w_layout="cn", bias=bias)

    @staticmethod
    def backward(ctx, grad_output):
        X, W, Ind = ctx.saved_tensors
        need_x, need_w, need_b = ctx.needs_input_grad[:3]
        grad_output = grad_output.contiguous()
        grad_W = _weight_grad_on_side_stream(X, grad_output, Ind, "gathered_rows") if need_w else None
        grad_X = ops.gemm_scatter(grad_output, W, Ind, X.shape[1], w_layout="nc") if need_x else None
        grad_b = grad_output.sum(dim=(0, 2)).reshape(ctx.bias_shape) if need_b else None
        _join_side(grad_output)
        return grad_X, grad_W, grad_b, None


class ExpertScatterBiasFunction(torch.autograd.Function):
    """``ExpertScatterFunction`` with a per-expert bias added to every routed slot's product before it is scattered:
    ``Out[b,t,:] = sum over slots (e,k) routed to t of (Y[b,e,k,:] @ W[e] + bias[e])`` with bias [E,1,I], fused into the
    scatter's epilogue.  ``apply(Y, W, bias, Ind, T)``; backward returns ``(grad_Y, grad_W, grad_bias, None, None)``.
    grad_bias[e] is the sum over the slots of expert e of the gathered rows of grad_Out - operator D against a tensor of
    ones, so no [B,E,K,I] gather is materialised."""

    @staticmethod
    def forward(ctx, Y, W, bias, Ind, T):
        ctx.save_for_backward(Y, W, Ind)
        ctx.bias_shape = tuple(bias.shape)
        return ops.gemm_scatter(Y, W, Ind, int(T), w_layout="cn", bias=bias)

    @staticmethod
    def backward(ctx, grad_X):
        Y, W, Ind = ctx.saved_tensors
        need_y, need_w, need_b = ctx.needs_input_grad[:3]
        grad_X = grad_X.contiguous()
        grad_W = _weight_grad_on_side_stream(grad_X, Y, Ind, "direct_rows") if need_w else None
        grad_Y = ops.gather_gemm(grad_X, W, Ind, w_layout="nc") if need_y else None
        grad_b = None
        if need_b:
            ones = torch.ones(Y.shape[0], Y.shape[1], Y.shape[2], 8, device=Y.device, dtype=Y.dtype)
            grad_b = ops.dweight(grad_X, ones, Ind, out_layout="gathered_rows")[:, :, 0].reshape(ctx.bias_shape)
        _join_side(grad_X)
        return grad_Y, grad_W, grad_b, None, None


class ExpertGatherScatterFunction(torch.autograd.Function):
    """Gather followed by scatter with the same ``Ind`` - the way the two operators are used in a model
    (reference: ``README.md:23-32``) - as one autograd node: ``Out = scatter(gather(X, W_g), W_s)``.

    ``apply(X, W_g, W_s, Ind)`` with X [B,T,I], W_g [E,I,J], W_s [E,J,I], Ind [B,E,K] -> Out [B,T,I].
    Where the fused kernel pays (float32, single-wave grids: ``ops.fused_pair_preferred``) the forward pass is one
    kernel (Y is written once, for the backward pass, and consumed from shared memory) and so is dY -> dX of the
    backward pass; otherwise each pass runs the two separate operators.  The weight gradients are the same two
    contractions as in ``ExpertGatherFunction`` / ``ExpertScatterFunction`` and run next to dY -> dX on the helper
    stream.  backward returns ``(grad_X, grad_W_g, grad_W_s, None)``; gradients autograd does not ask for are skipped.
    """

    @staticmethod
    def forward(ctx, X, Wg, Ws, Ind):
        X, Wg, Ws = X.contiguous(), Wg.contiguous(), Ws.contiguous()
        ctx.fused = ops.fused_pair_preferred(X, Wg, Ind)
        if ctx.fused:
            Y, Out = ops.gather_scatter_pair(X, Wg, Ws, Ind, w_layout="cn")
        else:
            Y = ops.gather_gemm(X, Wg, Ind, w_layout="cn")
            Out = ops.gemm_scatter(Y, Ws, Ind, X.shape[1], w_layout="cn")
        ctx.save_for_backward(X, Wg, Ws, Ind, Y)
        return Out

    @staticmethod
    def backward(ctx, grad_out):
        X, Wg, Ws, Ind, Y = ctx.saved_tensors
        need_x, need_wg, need_ws = ctx.needs_input_grad[:3]
        grad_out = grad_out.contiguous()
        grad_X = grad_Wg = grad_Ws = dY = None
        if need_ws:
            grad_Ws = _weight_grad_on_side_stream(grad_out, Y, Ind, "direct_rows")   # needs only dOut and Y
        if need_x and ctx.fused:
            dY, grad_X = ops.gather_scatter_pair(grad_out, Ws, Wg, Ind, w_layout="nc")
        elif need_x or need_wg:
            dY = ops.gather_gemm(grad_out, Ws, Ind, w_layout="nc")
        if need_wg:
            grad_Wg = _weight_grad_on_side_stream(X, dY, Ind, "gathered_rows")
        if need_x and grad_X is None:
            grad_X = ops.gemm_scatter(dY, Wg, Ind, X.shape[1], w_layout="nc")
        if need_ws or need_wg:
            _join_side(grad_out)
        return grad_X, grad_Wg, grad_Ws, None
