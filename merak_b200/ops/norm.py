"""Fused (dropout +) residual-add + LayerNorm / RMSNorm with a hand-written backward.

``fused_norm`` computes ``z = dropout(x) + residual`` and ``y = norm(z)`` in one pass and returns
``(y, z)``; ``z`` is the updated residual stream of a pre-norm block or simply the saved input of
a post-norm block.  CUDA tensors run ``csrc/norm.cu``; CPU tensors run the PyTorch formula below
(without dropout randomness parity: the CPU path uses ``torch.nn.functional.dropout``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib
from .rng import dropout_state


def norm_reference(x, residual, weight, bias, eps, rms, p_drop=0.0, training=True):
    z = x.float()
    if p_drop > 0.0 and training:
        z = dropout_state().host_dropout(z, p_drop)
    if residual is not None:
        z = z + residual.float()
    z = z.to(x.dtype)
    zf = z.float()
    if rms:
        y = zf * torch.rsqrt(zf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    else:
        y = F.layer_norm(zf, (zf.shape[-1],), weight.float(), None if bias is None else bias.float(), eps)
    return y.to(x.dtype), z


class _FusedNorm(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, residual, weight, bias, eps, rms, p_drop):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, H)
            if not r2.is_contiguous():
                r2 = r2.contiguous()
        M = x2.shape[0]
        y = torch.empty_like(x2)
        need_z = (r2 is not None) or p_drop > 0.0
        z = torch.empty_like(x2) if need_z else x2
        mean = None if rms else torch.empty(M, dtype=torch.float32, device=x.device)
        rstd = torch.empty(M, dtype=torch.float32, device=x.device)
        rng = None
        call_id = 0
        if p_drop > 0.0:
            st = dropout_state()
            rng = st.tensor(x.device)
            call_id = st.next_call_id()
        params_f32 = weight.dtype == torch.float32
        assert bias is None or bias.dtype == weight.dtype
        rc = _lib.kernels().mrk_norm_fwd(
            x2.data_ptr(), _lib.ptr(r2), weight.data_ptr(), _lib.ptr(bias), y.data_ptr(),
            z.data_ptr() if need_z else 0, _lib.ptr(mean), rstd.data_ptr(), _lib.ptr(rng), call_id,
            float(p_drop), float(eps), M, H, int(rms), int(params_f32), _lib.stream_ptr())
        _lib.check(rc, "mrk_norm_fwd")
        ctx.save_for_backward(z, weight, mean, rstd, rng)
        # an unused output must not cost a zero-filled gradient tensor (and a pass over it in the kernel)
        ctx.set_materialize_grads(False)
        ctx.meta = (rms, p_drop, call_id, bias is not None, residual is not None, x.shape, params_f32)
        ctx.need_z = need_z
        if need_z:
            return y.view(x.shape), z.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dz_extra=None):
        z, weight, mean, rstd, rng = ctx.saved_tensors
        rms, p_drop, call_id, has_bias, has_res, shape, params_f32 = ctx.meta
        H = shape[-1]
        if dy is None:          # only the pre-norm sum was used downstream
            if dz_extra is None:
                return None, None, None, None, None, None, None
            dy = torch.zeros_like(dz_extra)
        dy2 = dy.reshape(-1, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        M = dy2.shape[0]
        e2 = None
        if dz_extra is not None:
            e2 = dz_extra.reshape(-1, H)
            if not e2.is_contiguous():
                e2 = e2.contiguous()
        dres = torch.empty_like(dy2)
        dx = torch.empty_like(dy2) if p_drop > 0.0 else dres
        dgamma = torch.empty(H, dtype=torch.float32, device=dy.device)
        dbeta = torch.empty(H, dtype=torch.float32, device=dy.device) if has_bias else None
        lib = _lib.kernels()
        ws = _workspace(dy.device, H, lib)
        rc = lib.mrk_norm_bwd(
            dy2.data_ptr(), z.data_ptr(), _lib.ptr(e2), weight.data_ptr(), _lib.ptr(mean), rstd.data_ptr(),
            dres.data_ptr(), dx.data_ptr(), dgamma.data_ptr(), _lib.ptr(dbeta), ws.data_ptr(), _lib.ptr(rng), call_id,
            float(p_drop), M, H, int(rms), int(params_f32), _lib.stream_ptr())
        _lib.check(rc, "mrk_norm_bwd")
        dw = _param_grad(weight, dgamma)
        db = _param_grad(weight, dbeta) if has_bias else None
        return dx.view(shape), (dres.view(shape) if has_res else None), dw, db, None, None, None


def _param_grad(param, grad_f32):
    """Routes an fp32 parameter gradient: accumulate into ``param.main_grad`` when the optimizer
    owns an fp32 gradient buffer, else hand a tensor of the parameter's dtype back to autograd."""
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        mg.add_(grad_f32.view(mg.shape))
        return None
    return grad_f32.to(param.dtype)


_WORKSPACES = {}


def _workspace(device, H, lib):
    """Accumulator rows for the weight / bias gradient partial sums: zero on creation, and every
    backward call leaves them zero again, so one buffer per (device, hidden size) serves all calls
    issued in stream order."""
    key = (device.index, H, torch.cuda.current_stream(device).cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = _WORKSPACES[key] = torch.zeros((lib.mrk_norm_bwd_workspace_rows(), 2, H), dtype=torch.float32, device=device)
    return ws


def fused_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
               residual: Optional[torch.Tensor] = None, eps: float = 1e-5, rms: bool = False,
               p_drop: float = 0.0, training: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(norm(z), z)`` with ``z = dropout(x, p_drop) + residual``."""
    if not training:
        p_drop = 0.0
    H = x.shape[-1]
    if not _lib.use_kernels(x) or x.dtype != torch.bfloat16 or H % 8 != 0 or H > 8192:
        return norm_reference(x, residual, weight, bias, eps, rms, p_drop, training)
    if residual is None and p_drop == 0.0:
        # z is x itself: keep it out of the autograd node so no output aliases an input
        return _FusedNorm.apply(x, None, weight, bias, eps, rms, 0.0), x
    return _FusedNorm.apply(x, residual, weight, bias, eps, rms, p_drop)
