"""Linear layers on the tcgen05 GEMM with hand-written backward passes.

* ``linear(x, weight, bias, residual)``: ``y = x W^T + b (+ residual)``.
* ``mlp(x, w1, b1, w2, b2, act, residual)``: ``act(x W1^T + b1) W2^T + b2 (+ residual)``.  The
  activation is one memory-speed pass between the GEMMs, and in the backward pass one pass applies
  its derivative and sums the bias gradient of the first GEMM.  (The GEMM can apply both in its
  epilogue, ``FUSE_ACT_IN_GEMM``; at K = 1024 that made the epilogue warps the bottleneck:
  0.218 + 0.196 ms fused against 0.116 + 0.045 and 0.103 + 0.06 ms for 16384 x 4096 x 1024.)

Weight gradients are produced by transposed-operand GEMMs straight from the row-major
activations (no transposes are materialised).  When a parameter carries an fp32 ``main_grad``
buffer (set up by the optimizer), the gradient is accumulated into it by the GEMM epilogue and
autograd sees ``None`` - the "gradient accumulation fusion" that replaces the reference's
flatten/cast/accumulate pass (Merak/core/merak_engine.py:552-574).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib, flop_counter
from . import gemm as G
from .elementwise import act_backward, act_forward, colsum
from .norm import _param_grad


FUSE_ACT_IN_GEMM = False


def _as2d(x, K):
    x2 = x.reshape(-1, K)
    if x2.stride(1) != 1 or x2.stride(0) % 8 != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    return x2


def _weight_grad(dy2, x2, weight, mg=None):
    """dW[N,K] = dy2^T x2, accumulated into ``weight.main_grad`` (or ``mg``) when present."""
    mg = mg if mg is not None else getattr(weight, "main_grad", None)
    if mg is not None:
        G.gemm(dy2, x2, a_mn=True, b_mn=True, out=mg.view(weight.shape), accumulate=True)
        return None
    dw, _ = G.gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
    return dw


def _bias_grad(dy2, bias):
    if bias is None or not bias.requires_grad:
        return None
    mg = getattr(bias, "main_grad", None)
    if mg is not None:
        colsum(dy2, mg.view(-1))
        return None
    return colsum(dy2).to(bias.dtype)


class _Linear(torch.autograd.Function):
    """``fork=True`` also returns the input (as an alias): a caller that feeds ``x`` both into this
    layer and into a residual connection takes the residual from the second output, and the sum of
    the two gradients of ``x`` then happens in the epilogue of the data-gradient GEMM instead of in
    a separate elementwise kernel."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, fork=False):
        N, K = weight.shape
        x2 = _as2d(x, K)
        r2 = _as2d(residual, N) if residual is not None else None
        y, _ = G.gemm(x2, weight, bias=bias, aux_in=r2, aux_mode=G.AUX_ADD if r2 is not None else G.AUX_NONE)
        ctx.save_for_backward(x2, weight, bias)
        ctx.in_shape = x.shape
        ctx.has_res = residual is not None
        ctx.main_grad = getattr(weight, "main_grad", None)     # slices of stacked weights carry their own view
        ctx.fork = fork
        if fork:
            ctx.set_materialize_grads(False)
            return y.view(*x.shape[:-1], N), x.view_as(x)
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy, dx_extra=None):
        x2, weight, bias = ctx.saved_tensors
        N, K = weight.shape
        if dy is None:           # fork: only the pass-through output was used
            return dx_extra, None, None, None, None
        dy2 = _as2d(dy, N)
        dx = None
        if ctx.needs_input_grad[0]:
            e2 = _as2d(dx_extra, K) if dx_extra is not None else None
            dx2, _ = G.gemm(dy2, weight, b_mn=True, aux_in=e2, aux_mode=G.AUX_ADD if e2 is not None else G.AUX_NONE)
            dx = dx2.view(ctx.in_shape)
        dw = _weight_grad(dy2, x2, weight, ctx.main_grad) if weight.requires_grad else None
        db = _bias_grad(dy2, bias)
        return dx, dw, db, (dy if ctx.has_res else None), None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not _lib.use_kernels(x, weight) or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        _lib.note_library_fallback("linear", x)
        y = F.linear(x, weight, bias)
        return y + residual if residual is not None else y
    if flop_counter.enabled():          # the kernel's work is invisible to the ATen-level counter
        flop_counter.add(2 * (x.numel() // x.shape[-1]) * weight.shape[0] * weight.shape[1])
    return _Linear.apply(x, weight, bias, residual, False)


def linear_fork(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """``(x W^T + b, x)``: use the second result wherever ``x`` is needed again (residual), see
    :class:`_Linear`."""
    if not _lib.use_kernels(x, weight) or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return linear(x, weight, bias), x
    return _Linear.apply(x, weight, bias, None, True)


class _MLP(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, act, residual, fork=False):
        F1, K = w1.shape
        N = w2.shape[0]
        x2 = _as2d(x, K)
        r2 = _as2d(residual, N) if residual is not None else None
        if FUSE_ACT_IN_GEMM or act == G.ACT_NONE:
            a, h = G.gemm(x2, w1, bias=b1, act=act, want_preact=True)
        else:
            h, _ = G.gemm(x2, w1, bias=b1)
            a = act_forward(act, h)
        y, _ = G.gemm(a, w2, bias=b2, aux_in=r2, aux_mode=G.AUX_ADD if r2 is not None else G.AUX_NONE)
        ctx.save_for_backward(x2, w1, b1, w2, b2, h, a)
        ctx.act, ctx.in_shape, ctx.has_res = act, x.shape, residual is not None
        ctx.fork = fork
        if fork:
            ctx.set_materialize_grads(False)
            return y.view(*x.shape[:-1], N), x.view_as(x)
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy, dx_extra=None):
        x2, w1, b1, w2, b2, h, a = ctx.saved_tensors
        N = w2.shape[0]
        if dy is None:
            return dx_extra, None, None, None, None, None, None, None
        dy2 = _as2d(dy, N)
        # dh = (dy W2) * act'(h): derivative applied in the GEMM epilogue
        db1_done = False
        if FUSE_ACT_IN_GEMM or ctx.act == G.ACT_NONE:
            dh, _ = G.gemm(dy2, w2, b_mn=True, act=ctx.act, aux_in=h, aux_mode=G.AUX_DACT)
        else:
            dh, _ = G.gemm(dy2, w2, b_mn=True)
            mg1 = getattr(b1, "main_grad", None) if (b1 is not None and b1.requires_grad) else None
            dh = act_backward(ctx.act, dh, h, mg1.view(-1) if mg1 is not None else None)
            db1_done = mg1 is not None
        dw2 = _weight_grad(dy2, a, w2) if w2.requires_grad else None
        db2 = _bias_grad(dy2, b2)
        dx = None
        if ctx.needs_input_grad[0]:
            e2 = _as2d(dx_extra, w1.shape[1]) if dx_extra is not None else None
            dx2, _ = G.gemm(dh, w1, b_mn=True, aux_in=e2, aux_mode=G.AUX_ADD if e2 is not None else G.AUX_NONE)
            dx = dx2.view(ctx.in_shape)
        dw1 = _weight_grad(dh, x2, w1) if w1.requires_grad else None
        db1 = None if db1_done else _bias_grad(dh, b1)
        return dx, dw1, db1, dw2, db2, None, (dy if ctx.has_res else None), None


def mlp(x, w1, b1, w2, b2, act: int = G.ACT_GELU_ERF, residual=None):
    """``act(x w1^T + b1) w2^T + b2 (+ residual)``."""
    if not _lib.use_kernels(x, w1, w2) or x.dtype != torch.bfloat16:
        _lib.note_library_fallback("mlp", x)
        hdn = G.act_forward(act, F.linear(x, w1, b1))
        y = F.linear(hdn, w2, b2)
        return y + residual if residual is not None else y
    if flop_counter.enabled():
        flop_counter.add(2 * (x.numel() // x.shape[-1]) * (w1.numel() + w2.numel()))
    return _MLP.apply(x, w1, b1, w2, b2, act, residual, False)


def mlp_fork(x, w1, b1, w2, b2, act: int = G.ACT_GELU_ERF):
    """``(mlp(x), x)``: the second result carries ``x`` to the residual connection, see :class:`_Linear`."""
    if not _lib.use_kernels(x, w1, w2) or x.dtype != torch.bfloat16:
        return mlp(x, w1, b1, w2, b2, act), x
    return _MLP.apply(x, w1, b1, w2, b2, act, None, True)
