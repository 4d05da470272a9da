"""Fused scaled-dot-product attention (flash attention) with a hand-written backward.

Tensors use the ``[batch, seq, heads, head_dim]`` layout so that Q/K/V can be strided views of a
fused QKV projection and the output feeds the next GEMM without a transpose.  On CUDA the
tcgen05 kernels in ``csrc/attention_{fwd,bwd}.cu`` run; on CPU the same math is evaluated with
PyTorch (fp32), which is also the oracle of the GPU tests.

Stands in for the eager ``matmul -> softmax -> dropout -> matmul`` attention of the models the
reference trains (examples/models/gpt2/config.py:28) and for the SDPA / FlashAttention-2 branch
of Merak/core/sequence_parallel/modeling/llama.py:24-160.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib, flop_counter
from .rng import dropout_state

def _declare():
    _lib.kernels()


def attention_reference(q, k, v, key_bias=None, causal=False, scale=None):
    """fp32 evaluation of softmax(scale * q k^T + bias + causal mask) v on [B, L, H, D] tensors."""
    B, Lq, H, D = q.shape
    Lk, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    if Hkv != H:
        kf = kf.repeat_interleave(H // Hkv, dim=1)
        vf = vf.repeat_interleave(H // Hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if key_bias is not None:
        s = s + key_bias.float()[:, None, None, :]
    if causal:
        keep = torch.ones(Lq, Lk, dtype=torch.bool, device=q.device).tril(Lk - Lq)
        s = s.masked_fill(~keep, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)


def _mix32(x: torch.Tensor) -> torch.Tensor:
    m = 0xFFFFFFFF
    x = x ^ (x >> 16)
    x = (x * 0x85EBCA6B) & m
    x = x ^ (x >> 13)
    x = (x * 0xC2B2AE35) & m
    return x ^ (x >> 16)


def dropout_keep_mask(seed: int, stream: int, B: int, H: int, Lq: int, Lk: int, p: float, device) -> torch.Tensor:
    """The keep mask ``[B, H, Lq, Lk]`` (bool) the flash kernels use for dropout probability ``p`` and generator
    state ``(seed, stream = offset + call id)``: the same stateless hash as ``csrc/attention_dropout.cuh``,
    evaluated with int64 tensors.  For tests and for reproducing a run's masks."""
    m = 0xFFFFFFFF
    t = lambda v: torch.tensor(int(v) & m, dtype=torch.int64, device=device)
    base = _mix32(t(seed) ^ _mix32((t(seed >> 32) + 0x9E3779B9) & m)
                  ^ _mix32(((t(stream) * 0x9E3779B1) + t(stream >> 32)) & m))
    bh = torch.arange(B * H, dtype=torch.int64, device=device).view(B, H, 1, 1)
    q = torch.arange(Lq, dtype=torch.int64, device=device).view(1, 1, Lq, 1)
    k = torch.arange(Lk, dtype=torch.int64, device=device).view(1, 1, 1, Lk)
    rowkey = _mix32((_mix32(base ^ ((bh * 0x85EBCA6B) & m)) + q * 0xC2B2AE35) & m)
    thresh = min(int(float(torch.tensor(p, dtype=torch.float32).item()) * 4294967296.0), m)
    return _mix32(rowkey ^ ((k * 0x9E3779B1) & m)) >= thresh


def attention_with_dropout(q, k, v, key_bias, causal, scale, dropout_p):
    """Attention with dropout on the probabilities (the eager ``matmul -> softmax -> dropout -> matmul``
    of the reference's models) for the cases the flash kernels do not take (CPU, dtypes other than bf16, head
    dims other than 64 / 128): PyTorch's ``scaled_dot_product_attention``, announced once through
    ``note_library_fallback`` on CUDA; tensors are ``[B, L, H, D]`` as everywhere in this module."""
    _lib.note_library_fallback("attention with dropout on the probabilities", q)
    B, Lq, H, D = q.shape
    Hkv = k.shape[2]
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    if Hkv != H:
        kh = kh.repeat_interleave(H // Hkv, dim=1)
        vh = vh.repeat_interleave(H // Hkv, dim=1)
    mask = None
    if key_bias is not None:
        mask = key_bias.to(q.dtype)[:, None, None, :].expand(B, 1, Lq, k.shape[1])
        if causal:
            keep = torch.ones(Lq, k.shape[1], dtype=torch.bool, device=q.device).tril(k.shape[1] - Lq)
            mask = mask.masked_fill(~keep, float("-inf"))
    out = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, dropout_p=float(dropout_p),
                                         is_causal=bool(causal and mask is None), scale=scale)
    return out.permute(0, 2, 1, 3)


def _strides3(t):
    return (t.stride(0), t.stride(1), t.stride(2))


def _tma_ok(t) -> bool:
    return (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all((s * t.element_size()) % 16 == 0
                                                                  for s in _strides3(t)))


def _dropout_args(dropout_p: float, device):
    """(generator state tensor or None, call id) of one attention call; the backward pass reuses both."""
    if dropout_p <= 0.0:
        return None, 0
    st = dropout_state()
    # heads are what tensor parallelism shards: the rank-dependent generator, so that two ranks' local head
    # 0 do not share a mask (with one rank per replica the two generators coincide)
    return st.tensor(device, sharded=True), st.next_call_id()


class _FlashAttention(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, key_bias, causal, scale, dropout_p=0.0):
        _declare()
        B, Lq, H, D = q.shape
        Lk, Hkv = k.shape[1], k.shape[2]
        q, k, v = (t if _tma_ok(t) else t.contiguous() for t in (q, k, v))
        out = torch.empty((B, Lq, H, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        kb = key_bias.float().contiguous() if key_bias is not None else None
        rng, call_id = _dropout_args(dropout_p, q.device)
        rc = _lib.kernels().mrk_attn_fwd_drop(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), _lib.ptr(kb),
            B, H, Hkv, Lq, Lk, D, *_strides3(q), *_strides3(k), *_strides3(v), *_strides3(out),
            int(causal), float(scale), float(dropout_p), _lib.ptr(rng), call_id, _lib.stream_ptr())
        _lib.check(rc, "mrk_attn_fwd")
        ctx.save_for_backward(q, k, v, out, lse, kb, rng)
        ctx.causal, ctx.scale, ctx.drop = causal, scale, (float(dropout_p), call_id)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, kb, rng = ctx.saved_tensors
        B, Lq, H, D = q.shape
        Lk, Hkv = k.shape[1], k.shape[2]
        if not _tma_ok(dout):
            dout = dout.contiguous()
        dq = torch.empty((B, Lq, H, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((B, Lk, Hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((B, Lk, Hkv, D), dtype=q.dtype, device=q.device)
        delta = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        dq_acc = torch.empty((B, Lq, H, D), dtype=torch.float32, device=q.device)
        strides = []
        for t in (q, k, v, out, dout, dq, dk, dv):
            strides.extend(_strides3(t))
        arr = (ctypes.c_longlong * 24)(*strides)
        rc = _lib.kernels().mrk_attn_bwd_drop(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            delta.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _lib.ptr(kb),
            B, H, Hkv, Lq, Lk, D, ctypes.cast(arr, ctypes.c_void_p), int(ctx.causal), float(ctx.scale),
            ctx.drop[0], _lib.ptr(rng), ctx.drop[1], _lib.stream_ptr())
        _lib.check(rc, "mrk_attn_bwd")
        return dq, dk, dv, None, None, None, None


class _FlashAttentionPacked(torch.autograd.Function):
    """Attention on a packed projection output ``[B, L, Hq + 2*Hkv, D]`` (query heads first, then key
    heads, then value heads).  The backward writes dQ, dK and dV straight into one packed gradient
    tensor, so no per-slice gradient tensors are materialised and summed."""

    @staticmethod
    def forward(ctx, qkv, hq, hkv, key_bias, causal, scale, dropout_p=0.0):
        if not _tma_ok(qkv):
            qkv = qkv.contiguous()
        B, L, _, D = qkv.shape
        q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
        out = torch.empty((B, L, hq, D), dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty((B, hq, L), dtype=torch.float32, device=qkv.device)
        kb = key_bias.float().contiguous() if key_bias is not None else None
        rng, call_id = _dropout_args(dropout_p, qkv.device)
        rc = _lib.kernels().mrk_attn_fwd_drop(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), _lib.ptr(kb),
            B, hq, hkv, L, L, D, *_strides3(q), *_strides3(k), *_strides3(v), *_strides3(out),
            int(causal), float(scale), float(dropout_p), _lib.ptr(rng), call_id, _lib.stream_ptr())
        _lib.check(rc, "mrk_attn_fwd")
        ctx.save_for_backward(qkv, out, lse, kb, rng)
        ctx.meta = (hq, hkv, causal, scale, float(dropout_p), call_id)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, kb, rng = ctx.saved_tensors
        hq, hkv, causal, scale, p_drop, call_id = ctx.meta
        B, L, _, D = qkv.shape
        if not _tma_ok(dout):
            dout = dout.contiguous()
        q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, :, :hq], dqkv[:, :, hq:hq + hkv], dqkv[:, :, hq + hkv:]
        delta = torch.empty((B, hq, L), dtype=torch.float32, device=qkv.device)
        dq_acc = torch.empty((B, L, hq, D), dtype=torch.float32, device=qkv.device)
        strides = []
        for t in (q, k, v, out, dout, dq, dk, dv):
            strides.extend(_strides3(t))
        arr = (ctypes.c_longlong * 24)(*strides)
        rc = _lib.kernels().mrk_attn_bwd_drop(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            delta.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _lib.ptr(kb),
            B, hq, hkv, L, L, D, ctypes.cast(arr, ctypes.c_void_p), int(causal), float(scale), p_drop, _lib.ptr(rng),
            call_id, _lib.stream_ptr())
        _lib.check(rc, "mrk_attn_bwd")
        return dqkv, None, None, None, None, None, None


def flash_attention_packed(qkv: torch.Tensor, num_q_heads: int, num_kv_heads: int,
                           key_bias: Optional[torch.Tensor] = None, causal: bool = False,
                           scale: Optional[float] = None, dropout_p: float = 0.0) -> torch.Tensor:
    """Self-attention on ``qkv`` of shape ``[B, L, Hq + 2*Hkv, D]``; returns ``[B, L, Hq, D]``.
    ``dropout_p`` > 0 (pass it in training mode only) drops attention probabilities."""
    D = qkv.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not _lib.use_kernels(qkv) or qkv.dtype != torch.bfloat16 or D not in (64, 128):
        q, k, v = (qkv[:, :, :num_q_heads], qkv[:, :, num_q_heads:num_q_heads + num_kv_heads],
                   qkv[:, :, num_q_heads + num_kv_heads:])
        if dropout_p > 0.0:
            return attention_with_dropout(q, k, v, key_bias, causal, scale, dropout_p)
        _lib.note_library_fallback("attention", qkv)
        return attention_reference(q, k, v, key_bias, causal, scale)
    if flop_counter.enabled():
        flop_counter.add(4 * qkv.shape[0] * num_q_heads * qkv.shape[1] * qkv.shape[1] * D // (2 if causal else 1))
    return _FlashAttentionPacked.apply(qkv, num_q_heads, num_kv_heads, key_bias, causal, scale, float(dropout_p))


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    key_bias: Optional[torch.Tensor] = None, causal: bool = False,
                    scale: Optional[float] = None, dropout_p: float = 0.0) -> torch.Tensor:
    """``softmax(scale * q k^T + key_bias + causal mask) v``.

    q ``[B, Lq, H, D]``; k, v ``[B, Lk, Hkv, D]`` with ``H % Hkv == 0`` (grouped-query attention);
    ``key_bias`` ``[B, Lk]`` additive (0 / large negative for padding).  ``D`` is 64 or 128 on CUDA.
    """
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not _lib.use_kernels(q, k, v) or q.dtype != torch.bfloat16 or D not in (64, 128):
        if dropout_p > 0.0:
            return attention_with_dropout(q, k, v, key_bias, causal, scale, dropout_p)
        if _lib.use_kernels(q, k, v):
            _lib.note_library_fallback("attention", q)
        return attention_reference(q, k, v, key_bias, causal, scale)
    if flop_counter.enabled():
        flop_counter.add(4 * q.shape[0] * q.shape[2] * q.shape[1] * k.shape[1] * D // (2 if causal else 1))
    return _FlashAttention.apply(q, k, v, key_bias, causal, scale, float(dropout_p))
