"""Vocab-parallel softmax cross entropy.

``vocab_parallel_cross_entropy(logits_shard, target)`` returns the per-token loss for logits whose
last dimension is split over the tensor-parallel group, like the reference function of the same
name (Merak/core/mpu/cross_entropy.py:26-118).  CUDA bf16/fp32 logits go through the fused
kernels with a single exchange of ``(max, sum-exp, target-logit)`` triples; this module holds the
PyTorch formulation used on CPU (three small all-reduces) which is also the test oracle.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import mpu


class _VocabParallelCrossEntropyTorch(torch.autograd.Function):

    @staticmethod
    def forward(ctx, logits, target, vocab_start, group):
        n = dist.get_world_size(group) if group is not None else 1
        lf = logits.float()
        lmax = lf.max(dim=-1).values
        if n > 1:
            dist.all_reduce(lmax, op=dist.ReduceOp.MAX, group=group)
        lf = lf - lmax.unsqueeze(-1)
        V = logits.shape[-1]
        local = target - vocab_start
        in_range = (local >= 0) & (local < V)
        idx = local.clamp(0, V - 1)
        tgt = lf.gather(-1, idx.unsqueeze(-1)).squeeze(-1) * in_range
        ex = lf.exp()
        sumexp = ex.sum(-1)
        if n > 1:
            dist.all_reduce(tgt, group=group)
            dist.all_reduce(sumexp, group=group)
        loss = sumexp.log() - tgt
        ctx.save_for_backward(ex / sumexp.unsqueeze(-1), in_range, idx)
        ctx.in_dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, g):
        softmax, in_range, idx = ctx.saved_tensors
        grad = softmax.clone()
        grad.scatter_add_(-1, idx.unsqueeze(-1), -in_range.unsqueeze(-1).to(grad.dtype))
        grad = grad * g.unsqueeze(-1)
        return grad.to(ctx.in_dtype), None, None, None


def vocab_parallel_cross_entropy(vocab_parallel_logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Per-token loss (same shape as ``target``) from vocabulary-sharded logits."""
    tp, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
    start = rank * vocab_parallel_logits.shape[-1]
    return _VocabParallelCrossEntropyTorch.apply(vocab_parallel_logits, target, start,
                                                 mpu.get_model_parallel_group() if tp > 1 else None)


def vocab_parallel_cross_entropy_torch(logits, labels, vocab_start, group, ignore_index=-100):
    """Mean over non-ignored targets (PyTorch path of ``ops.cross_entropy.softmax_cross_entropy``)."""
    flat_logits = logits.reshape(-1, logits.shape[-1])
    flat_labels = labels.reshape(-1)
    valid = flat_labels != ignore_index
    safe = torch.where(valid, flat_labels, torch.zeros_like(flat_labels))
    per_tok = _VocabParallelCrossEntropyTorch.apply(flat_logits, safe, vocab_start, group)
    per_tok = per_tok * valid
    return per_tok.sum() / valid.sum().clamp(min=1)
