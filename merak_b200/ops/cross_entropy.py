"""Softmax cross entropy over (optionally vocabulary-sharded) logits.

Forward makes one pass over the logits producing per-row ``(max, sum-exp, target logit)``; with a
tensor-parallel group the triples of all ranks are exchanged in ONE all-gather (the reference
issues three all-reduces: Merak/core/mpu/cross_entropy.py:33,64,72) and merged on device.  The
gradient ``(softmax - onehot) * scale`` is written by a second kernel that reads the still
L2-resident rows.  Mean reduction over non-ignored targets, like ``nn.CrossEntropyLoss``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib


def cross_entropy_reference(logits, labels, ignore_index=-100):
    return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), labels.reshape(-1),
                           ignore_index=ignore_index)


class _SoftmaxCrossEntropy(torch.autograd.Function):

    @staticmethod
    def forward(ctx, logits, labels, ignore_index, vocab_start, tp_group, loss_scale):
        V = logits.shape[-1]
        lg = logits.reshape(-1, V)
        if lg.stride(1) != 1 or lg.stride(0) % 8 != 0:
            pitch = (V + 7) // 8 * 8
            buf = torch.empty((lg.shape[0], pitch), dtype=lg.dtype, device=lg.device)
            buf[:, :V].copy_(lg)
            lg = buf[:, :V]
        lab = labels.reshape(-1).to(torch.int64).contiguous()
        M = lg.shape[0]
        lib = _lib.kernels()
        stream = _lib.stream_ptr()
        f32 = int(lg.dtype == torch.float32)
        tp = 1
        if tp_group is not None:
            import torch.distributed as dist
            tp = dist.get_world_size(tp_group)
        stats = torch.empty((M, 3), dtype=torch.float32, device=lg.device)
        _lib.check(lib.mrk_ce_stats(lg.data_ptr(), lab.data_ptr(), stats.data_ptr(), M, V, lg.stride(0),
                                    int(vocab_start), int(ignore_index), f32, stream), "mrk_ce_stats")
        if tp > 1:
            import torch.distributed as dist
            allstats = torch.empty((tp * M, 3), dtype=torch.float32, device=lg.device)
            dist.all_gather_into_tensor(allstats, stats, group=tp_group)
        else:
            allstats = stats
        lse = torch.empty(M, dtype=torch.float32, device=lg.device)
        sums = torch.zeros(2, dtype=torch.float32, device=lg.device)   # [loss_sum, valid_count]
        _lib.check(lib.mrk_ce_finalize(allstats.data_ptr(), tp, M * 3, lab.data_ptr(), lse.data_ptr(), 0,
                                       sums.data_ptr(), sums.data_ptr() + 4, M, int(ignore_index), stream),
                   "mrk_ce_finalize")
        denom = sums[1].clamp(min=1.0)
        loss = sums[0] / denom
        ctx.save_for_backward(lg, lab, lse, denom)
        ctx.meta = (ignore_index, vocab_start, logits.shape, f32, loss_scale)
        return loss * loss_scale if loss_scale != 1.0 else loss

    @staticmethod
    def backward(ctx, dloss):
        lg, lab, lse, denom = ctx.saved_tensors
        ignore_index, vocab_start, shape, f32, loss_scale = ctx.meta
        M, V = lg.shape
        gscale = (dloss.float() * loss_scale / denom).reshape(1).contiguous()
        pitch = (V + 7) // 8 * 8
        dl = torch.empty((M, pitch), dtype=lg.dtype, device=lg.device)
        _lib.check(_lib.kernels().mrk_ce_grad(lg.data_ptr(), lab.data_ptr(), lse.data_ptr(), gscale.data_ptr(),
                                              dl.data_ptr(), M, V, lg.stride(0), pitch, int(vocab_start),
                                              int(ignore_index), f32, _lib.stream_ptr()), "mrk_ce_grad")
        return dl[:, :V].unflatten(0, shape[:-1]), None, None, None, None, None


def softmax_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                          vocab_start: int = 0, tp_group=None, loss_scale: float = 1.0) -> torch.Tensor:
    """Mean cross entropy.  With ``tp_group`` the last dimension of ``logits`` is this rank's
    vocabulary slice starting at ``vocab_start`` and ``labels`` hold global ids."""
    if not _lib.use_kernels(logits) or logits.dtype not in (torch.bfloat16, torch.float32):
        from ..parallel import cross_entropy as vp
        if tp_group is not None:
            return vp.vocab_parallel_cross_entropy_torch(logits, labels, vocab_start, tp_group,
                                                         ignore_index) * loss_scale
        return cross_entropy_reference(logits, labels, ignore_index) * loss_scale
    return _SoftmaxCrossEntropy.apply(logits, labels, ignore_index, vocab_start, tp_group, loss_scale)
