"""Autograd wrappers of the small memory-bound kernels: embedding, rotary embedding, SwiGLU,
dropout and bias-gradient column sums.  CPU tensors take the PyTorch formulas (the test oracle)."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from . import _lib
from .norm import _param_grad
from .rng import dropout_state


# ---------------------------------------------------------------------------------------------
# column sums (bias gradients)
# ---------------------------------------------------------------------------------------------
def colsum(x2: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 column sums of a 2-D bf16 tensor, added into ``out`` when given."""
    M, N = x2.shape
    if not _lib.use_kernels(x2) or x2.dtype != torch.bfloat16 or N % 2 or x2.stride(1) != 1 or x2.stride(0) % 2:
        s = x2.float().sum(0)
        if out is None:
            return s
        out.add_(s)
        return out
    if out is None:
        out = torch.zeros(N, dtype=torch.float32, device=x2.device)
    _lib.check(_lib.kernels().mrk_colsum(x2.data_ptr(), out.data_ptr(), M, N, x2.stride(0), _lib.stream_ptr()),
               "mrk_colsum")
    return out


# ---------------------------------------------------------------------------------------------
# activation between the two GEMMs of an MLP
# ---------------------------------------------------------------------------------------------
def _act_kernel_ok(*ts) -> bool:
    return all(t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) == ts[0].stride(0)
               and t.stride(0) % 8 == 0 and t.shape[1] % 8 == 0 and t.data_ptr() % 16 == 0 for t in ts)


def act_forward(act: int, h: torch.Tensor) -> torch.Tensor:
    """``act(h)`` for a 2-D bf16 tensor (one pass at memory speed)."""
    from . import gemm as G
    if not _lib.use_kernels(h) or not _act_kernel_ok(h) or not h.is_contiguous():
        return G.act_forward(act, h.float()).to(h.dtype)
    out = torch.empty_like(h)
    _lib.check(_lib.kernels().mrk_act_fwd(h.data_ptr(), out.data_ptr(), h.numel(), act, _lib.stream_ptr()), "mrk_act_fwd")
    return out


def act_backward(act: int, d: torch.Tensor, h: torch.Tensor, colsum_out: Optional[torch.Tensor] = None):
    """``d * act'(h)`` written over ``d`` (2-D bf16).  With ``colsum_out`` (fp32 ``[N]``) the column sums of the
    result are added into it in the same pass: the bias gradient of the GEMM that produced ``h``."""
    from . import gemm as G
    if not _lib.use_kernels(d, h) or not _act_kernel_ok(d, h):
        out = (d.float() * G.act_grad(act, h)).to(d.dtype)
        if colsum_out is not None:
            colsum_out.add_(out.float().sum(0))
        return out
    M, N = d.shape
    _lib.check(_lib.kernels().mrk_act_bwd(d.data_ptr(), h.data_ptr(), d.data_ptr(),
                                          colsum_out.data_ptr() if colsum_out is not None else None, M, N, d.stride(0),
                                          act, _lib.stream_ptr()), "mrk_act_bwd")
    return d


# ---------------------------------------------------------------------------------------------
# embedding (sum of up to three lookups, vocab-parallel aware)
# ---------------------------------------------------------------------------------------------
class _Embedding(torch.autograd.Function):

    @staticmethod
    def forward(ctx, ids_list, starts, *tables):
        n = len(tables)
        H = tables[0].shape[1]
        shape = ids_list[0].shape
        idx = [i.reshape(-1).to(torch.int64).contiguous() for i in ids_list]
        T = idx[0].numel()
        out = torch.empty((T, H), dtype=tables[0].dtype, device=tables[0].device)
        P = ctypes.c_void_p
        tarr = (P * 3)(*[t.data_ptr() for t in tables] + [0] * (3 - n))
        iarr = (P * 3)(*[i.data_ptr() for i in idx] + [0] * (3 - n))
        rows = (ctypes.c_int * 3)(*[t.shape[0] for t in tables] + [0] * (3 - n))
        st = (ctypes.c_int * 3)(*list(starts) + [0] * (3 - n))
        _lib.check(_lib.kernels().mrk_embedding_fwd(ctypes.cast(tarr, P), ctypes.cast(iarr, P), ctypes.cast(rows, P),
                                                    ctypes.cast(st, P), n, out.data_ptr(), T, H, _lib.stream_ptr()),
                   "mrk_embedding_fwd")
        ctx.idx, ctx.starts, ctx.tables = idx, list(starts), tables
        return out.view(*shape, H)

    @staticmethod
    def backward(ctx, dout):
        H = dout.shape[-1]
        d2 = dout.reshape(-1, H)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        T = d2.shape[0]
        grads = []
        for table, idx, start in zip(ctx.tables, ctx.idx, ctx.starts):
            if not table.requires_grad:
                grads.append(None)
                continue
            mg = getattr(table, "main_grad", None)
            if mg is not None:
                _lib.check(_lib.kernels().mrk_embedding_bwd(d2.data_ptr(), idx.data_ptr(), mg.data_ptr(), T, H,
                                                            table.shape[0], start, 1, _lib.stream_ptr()),
                           "mrk_embedding_bwd")
                grads.append(None)
            else:
                g = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
                _lib.check(_lib.kernels().mrk_embedding_bwd(d2.data_ptr(), idx.data_ptr(), g.data_ptr(), T, H,
                                                            table.shape[0], start, 1, _lib.stream_ptr()),
                           "mrk_embedding_bwd")
                grads.append(g.to(table.dtype))
        return (None, None, *grads)


def embedding_sum(ids_list: Sequence[torch.Tensor], tables: Sequence[torch.Tensor],
                  starts: Optional[Sequence[int]] = None) -> torch.Tensor:
    """``sum_k tables[k][ids_list[k] - starts[k]]`` with out-of-range ids contributing zero."""
    starts = list(starts) if starts is not None else [0] * len(tables)
    t0 = tables[0]
    H = t0.shape[1]
    if (not _lib.use_kernels(t0) or t0.dtype != torch.bfloat16 or H % 8 != 0 or len(tables) > 3
            or any(t.dtype != t0.dtype or not t.is_contiguous() for t in tables)):
        out = None
        for ids, table, start in zip(ids_list, tables, starts):
            local = ids - start
            ok = (local >= 0) & (local < table.shape[0])
            e = F.embedding(local.clamp(0, table.shape[0] - 1), table)
            e = e * ok.unsqueeze(-1).to(e.dtype)
            out = e if out is None else out + e
        return out
    ids_list = [i.expand(ids_list[0].shape) if i.shape != ids_list[0].shape else i for i in ids_list]
    return _Embedding.apply(tuple(ids_list), tuple(starts), *tables)


# ---------------------------------------------------------------------------------------------
# rotary position embedding on [B, L, H, D]
# ---------------------------------------------------------------------------------------------
def rope_tables(max_len: int, dim: int, theta: float = 10000.0, device=None):
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    ang = torch.outer(torch.arange(max_len, dtype=torch.float32, device=device), inv)
    return ang.cos().contiguous(), ang.sin().contiguous()


def rope_reference(x, cos, sin, positions=None, inverse=False):
    B, L, H, D = x.shape
    if positions is None:
        c, s = cos[:L][None, :, None, :], sin[:L][None, :, None, :]
    else:
        c, s = cos[positions][:, :, None, :], sin[positions][:, :, None, :]
    if inverse:
        s = -s
    xf = x.float()
    lo, hi = xf[..., : D // 2], xf[..., D // 2:]
    return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1).to(x.dtype)


def _rope_launch(x, cos, sin, positions, inverse):
    B, L, H, D = x.shape
    if x.stride(3) != 1:
        x = x.contiguous()
    y = torch.empty((B, L, H, D), dtype=x.dtype, device=x.device)
    pos = positions.to(torch.int64).contiguous() if positions is not None else None
    _lib.check(_lib.kernels().mrk_rope(x.data_ptr(), y.data_ptr(), cos.data_ptr(), sin.data_ptr(), _lib.ptr(pos),
                                       B, L, H, D, x.stride(0), x.stride(1), x.stride(2), y.stride(0), y.stride(1),
                                       y.stride(2), int(inverse), _lib.stream_ptr()), "mrk_rope")
    return y


class _Rope(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, cos, sin, positions):
        ctx.save_for_backward(cos, sin, positions)
        return _rope_launch(x, cos, sin, positions, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin, positions = ctx.saved_tensors
        return _rope_launch(dy, cos, sin, positions, True), None, None, None


def apply_rope(x, cos, sin, positions=None):
    """Rotate-half rotary embedding; ``cos``/``sin`` are fp32 ``[max_len, D/2]`` tables."""
    if not _lib.use_kernels(x) or x.dtype != torch.bfloat16 or x.shape[-1] % 4 != 0:
        return rope_reference(x, cos, sin, positions)
    return _Rope.apply(x, cos, sin, positions)


# ---------------------------------------------------------------------------------------------
# SwiGLU on a fused gate|up tensor
# ---------------------------------------------------------------------------------------------
class _SwiGLU(torch.autograd.Function):

    @staticmethod
    def forward(ctx, gu):
        F2 = gu.shape[-1]
        g2 = gu.reshape(-1, F2)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        M, Fh = g2.shape[0], F2 // 2
        out = torch.empty((M, Fh), dtype=gu.dtype, device=gu.device)
        _lib.check(_lib.kernels().mrk_swiglu_fwd(g2.data_ptr(), out.data_ptr(), M, Fh, F2, _lib.stream_ptr()),
                   "mrk_swiglu_fwd")
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], Fh)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        M, F2 = g2.shape
        d2 = dout.reshape(M, F2 // 2)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dgu = torch.empty_like(g2)
        _lib.check(_lib.kernels().mrk_swiglu_bwd(g2.data_ptr(), d2.data_ptr(), dgu.data_ptr(), M, F2 // 2, F2,
                                                 _lib.stream_ptr()), "mrk_swiglu_bwd")
        return dgu.view(ctx.shape)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` where ``gate_up = cat([gate, up], -1)``."""
    Fh = gate_up.shape[-1] // 2
    if not _lib.use_kernels(gate_up) or gate_up.dtype != torch.bfloat16 or Fh % 8 != 0:
        g, u = gate_up[..., :Fh], gate_up[..., Fh:]
        return (F.silu(g.float()) * u.float()).to(gate_up.dtype)
    return _SwiGLU.apply(gate_up)


# ---------------------------------------------------------------------------------------------
# dropout
# ---------------------------------------------------------------------------------------------
class _Dropout(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, p):
        st = dropout_state()
        rng = st.tensor(x.device)
        call_id = st.next_call_id()
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _lib.check(_lib.kernels().mrk_dropout(xc.data_ptr(), y.data_ptr(), xc.numel(), float(p), rng.data_ptr(),
                                              call_id, _lib.stream_ptr()), "mrk_dropout")
        ctx.rng, ctx.call_id, ctx.p = rng, call_id, p
        return y

    @staticmethod
    def backward(ctx, dy):
        dc = dy.contiguous()
        dx = torch.empty_like(dc)
        _lib.check(_lib.kernels().mrk_dropout(dc.data_ptr(), dx.data_ptr(), dc.numel(), float(ctx.p),
                                              ctx.rng.data_ptr(), ctx.call_id, _lib.stream_ptr()), "mrk_dropout")
        return dx, None


def dropout(x: torch.Tensor, p: float, training: bool = True) -> torch.Tensor:
    if p <= 0.0 or not training:
        return x
    if not _lib.use_kernels(x) or x.dtype != torch.bfloat16 or x.numel() % 8 != 0:
        return dropout_state().host_dropout(x, p)
    return _Dropout.apply(x, p)
