"""bf16 GEMM with fused epilogues (bias, activation, residual add, activation derivative).

``gemm`` is the raw operator: on CUDA tensors it launches the tcgen05 kernel
(``csrc/gemm_tcgen05.cu``); on CPU tensors it evaluates the same formula in PyTorch, which is
also the oracle the GPU tests compare against.

Replaces the ``F.linear`` / ``torch.matmul`` call sites of the reference
(Merak/core/mpu/layers.py:252,354; Merak/core/tensor_parallel/mp_layers.py:249,319) and the
elementwise passes that follow them.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib, flop_counter

ACT_NONE, ACT_GELU_ERF, ACT_GELU_TANH, ACT_RELU, ACT_SILU = 0, 1, 2, 3, 4
AUX_NONE, AUX_ADD, AUX_DACT = 0, 1, 2
_F_OUT_F32, _F_ACC, _F_BIAS_F32, _F_A_MN, _F_B_MN = 1, 2, 4, 8, 16

ACT_BY_NAME = {None: ACT_NONE, "none": ACT_NONE, "gelu": ACT_GELU_ERF, "gelu_erf": ACT_GELU_ERF,
               "gelu_new": ACT_GELU_TANH, "gelu_tanh": ACT_GELU_TANH, "gelu_pytorch_tanh": ACT_GELU_TANH,
               "relu": ACT_RELU, "silu": ACT_SILU, "swish": ACT_SILU}


def act_forward(act: int, x: torch.Tensor) -> torch.Tensor:
    if act == ACT_GELU_ERF:
        return F.gelu(x)
    if act == ACT_GELU_TANH:
        return F.gelu(x, approximate="tanh")
    if act == ACT_RELU:
        return F.relu(x)
    if act == ACT_SILU:
        return F.silu(x)
    return x


def act_grad(act: int, x: torch.Tensor) -> torch.Tensor:
    """d act(x) / dx evaluated in fp32."""
    x = x.float()
    if act == ACT_GELU_ERF:
        cdf = 0.5 * (1.0 + torch.erf(x * (1.0 / math.sqrt(2.0))))
        pdf = torch.exp(-0.5 * x * x) * (1.0 / math.sqrt(2.0 * math.pi))
        return cdf + x * pdf
    if act == ACT_GELU_TANH:
        c = math.sqrt(2.0 / math.pi)
        u = c * (x + 0.044715 * x ** 3)
        t = torch.tanh(u)
        du = c * (1.0 + 3 * 0.044715 * x * x)
        return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * du
    if act == ACT_RELU:
        return (x > 0).float()
    if act == ACT_SILU:
        s = torch.sigmoid(x)
        return s * (1 + x * (1 - s))
    return torch.ones_like(x)


def _reference(a, b, a_mn, b_mn, bias, act, aux_in, aux_mode, alpha, out, accumulate, out_dtype,
               want_preact):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    v = (A @ B) * alpha
    if bias is not None:
        v = v + bias.float()
    pre = v.to(torch.bfloat16) if want_preact else None
    if act != ACT_NONE and aux_mode != AUX_DACT:
        v = act_forward(act, v)
    if aux_mode == AUX_ADD:
        v = v + aux_in.float()
    elif aux_mode == AUX_DACT:
        v = v * act_grad(act, aux_in)
    if out is not None:
        if accumulate:
            out.add_(v.to(out.dtype))
        else:
            out.copy_(v.to(out.dtype))
    else:
        out = v.to(out_dtype)
    return out, pre


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         bias: Optional[torch.Tensor] = None, act: int = ACT_NONE,
         aux_in: Optional[torch.Tensor] = None, aux_mode: int = AUX_NONE, alpha: float = 1.0,
         out: Optional[torch.Tensor] = None, accumulate: bool = False,
         out_dtype: torch.dtype = torch.bfloat16, want_preact: bool = False, block_n: int = 0):
    """``C[M,N] = epilogue(alpha * op(a) @ op(b)^T)``.

    * ``a`` is ``[M,K]`` (``a_mn=False``) or ``[K,M]`` (``a_mn=True``); ``b`` is ``[N,K]`` or ``[K,N]``.
      Both are bf16 with unit stride in the last dimension.
    * ``bias`` ``[N]`` bf16 or fp32; ``act`` one of the ``ACT_*`` codes.
    * ``aux_mode=AUX_ADD`` adds ``aux_in`` ``[M,N]`` after the activation (residual);
      ``aux_mode=AUX_DACT`` multiplies by ``act'(aux_in)`` instead of applying ``act``.
    * ``out`` (bf16 or fp32) is written, or accumulated into when ``accumulate=True``.
    * ``want_preact`` additionally returns ``alpha*a@b^T + bias`` in bf16 (saved for backward).

    Returns ``(C, preact_or_None)``.
    """
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, "inner dimensions differ: %d vs %d" % (K, Kb)
    if not _lib.use_kernels(a, b):
        return _reference(a, b, a_mn, b_mn, bias, act, aux_in, aux_mode, alpha, out, accumulate,
                          out.dtype if out is not None else out_dtype, want_preact)
    if flop_counter.enabled():
        flop_counter.add(2 * M * N * K)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "tcgen05 GEMM takes bf16 operands"
    if a.stride(1) != 1 or (a.stride(0) * 2) % 16 != 0 or a.data_ptr() % 16 != 0:
        a = a.contiguous()
    if b.stride(1) != 1 or (b.stride(0) * 2) % 16 != 0 or b.data_ptr() % 16 != 0:
        b = b.contiguous()
    if (a.stride(0) % 8) != 0 or (b.stride(0) % 8) != 0:
        # row pitch not a multiple of 16 bytes: TMA cannot address it; pad the pitch.
        a = _pad_pitch(a)
        b = _pad_pitch(b)
    if out is None:
        assert not accumulate
        if N % 8 != 0:      # keep rows 16-byte aligned so the epilogue can use vector stores
            out = torch.empty((M, (N + 7) // 8 * 8), dtype=out_dtype, device=a.device)[:, :N]
        else:
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    else:
        assert out.shape == (M, N) and out.stride(1) == 1
    assert out.dtype in (torch.bfloat16, torch.float32)
    flags = 0
    if out.dtype == torch.float32:
        flags |= _F_OUT_F32
    if accumulate:
        flags |= _F_ACC
    if bias is not None:
        assert bias.numel() == N and bias.is_contiguous()
        if bias.dtype == torch.float32:
            flags |= _F_BIAS_F32
        else:
            assert bias.dtype == torch.bfloat16
    if a_mn:
        flags |= _F_A_MN
    if b_mn:
        flags |= _F_B_MN
    pre = None
    if want_preact:
        pre = torch.empty((M, (N + 7) // 8 * 8), dtype=torch.bfloat16, device=a.device)[:, :N]
    if aux_mode != AUX_NONE:
        assert aux_in is not None and aux_in.shape == (M, N) and aux_in.dtype == torch.bfloat16
        assert aux_in.stride(1) == 1
    rc = _lib.kernels().mrk_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        _lib.ptr(bias), _lib.ptr(aux_in), aux_in.stride(0) if aux_in is not None else 0,
        _lib.ptr(pre), pre.stride(0) if pre is not None else 0, act, aux_mode, flags, float(alpha),
        block_n, _lib.stream_ptr())
    _lib.check(rc, "mrk_gemm_bf16")
    return out, pre


def _pad_pitch(t: torch.Tensor) -> torch.Tensor:
    rows, cols = t.shape
    if t.stride(0) % 8 == 0 and t.stride(1) == 1:
        return t
    pitch = (cols + 7) // 8 * 8
    buf = torch.zeros((rows, pitch), dtype=t.dtype, device=t.device)
    buf[:, :cols].copy_(t)
    return buf[:, :cols]
