"""Sub-pipelined tensor model parallelism: hide tensor-parallel all-reduces behind GEMMs by
splitting a micro-batch into chunks (``args.tp_overlapping_level``).

* level 1 - inside one linear layer (Merak/core/tensor_parallel/mp_layers.py:187-497): the input is
  cut in two along dim 0; a row-parallel layer launches the all-reduce of chunk 1 asynchronously
  while the GEMM of chunk 2 runs; a column-parallel layer does the same for the data-gradient
  all-reduce in its backward pass.
* level 2 / 3 - across a transformer block (Merak/core/tensor_parallel/transformer_blocks.py:99-777):
  the block processes 2 (level 2) or 4 (level 3) batch chunks in a software pipeline, so that the
  attention-output all-reduce of chunk *i* overlaps the MLP of chunk *i-1*.  Here this is expressed
  generically for any block built from ``ColPara`` / ``RowPara`` layers, not for GPT-2 only.

These paths use ``torch.distributed`` asynchronous collectives (``comm_mode='nccl'``).  With
``comm_mode='fused'`` the GEMM+collective kernels overlap at tile granularity and chunking is not
needed; ``apply_tp_overlap`` is then a no-op.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import gemm as G
from ..ops.linear import _bias_grad, _weight_grad, linear as k_linear
from . import mpu
from .tp_transform import ColPara, RowPara

ASYNC_OP: List = []      # outstanding work handles (drained by sync_comm)


def sync_comm():
    while ASYNC_OP:
        ASYNC_OP.pop(0).wait()


class _AsyncReduce(torch.autograd.Function):
    """All-reduce launched asynchronously in forward; identity backward."""

    @staticmethod
    def forward(ctx, x):
        if mpu.get_model_parallel_world_size() > 1:
            x = x.contiguous()
            ASYNC_OP.append(dist.all_reduce(x, group=mpu.get_model_parallel_group(), async_op=True))
        return x

    @staticmethod
    def backward(ctx, g):
        return g


class _PipedColumnLinear(torch.autograd.Function):
    """Column-parallel linear whose backward pipelines chunks: the data-gradient all-reduce of one
    chunk is in flight while the gradient GEMMs of the next chunk run."""

    @staticmethod
    def forward(ctx, x, weight, bias, chunks):
        ctx.save_for_backward(x, weight, bias)
        ctx.chunks = chunks
        y, _ = G.gemm(x.reshape(-1, x.shape[-1]), weight, bias=bias, out_dtype=x.dtype)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias = ctx.saved_tensors
        n = ctx.chunks if x.shape[0] >= ctx.chunks else 1
        group, tp = mpu.get_model_parallel_group(), mpu.get_model_parallel_world_size()
        dxs, works = [], []
        dw_total, db_total = None, None
        for dy_c, x_c in reversed(list(zip(dy.chunk(n, 0), x.chunk(n, 0)))):
            dy2 = dy_c.reshape(-1, dy_c.shape[-1])
            x2 = x_c.reshape(-1, x_c.shape[-1])
            dx, _ = G.gemm(dy2, weight, b_mn=True, out_dtype=x.dtype)
            dx = dx.contiguous()
            if tp > 1:
                works.append(dist.all_reduce(dx, group=group, async_op=True))
            dxs.insert(0, dx.view(x_c.shape))
            dw = _weight_grad(dy2, x2, weight) if weight.requires_grad else None
            db = _bias_grad(dy2, bias) if bias is not None else None
            if dw is not None:
                dw_total = dw if dw_total is None else dw_total + dw
            if db is not None:
                db_total = db if db_total is None else db_total + db
        for w in works:
            w.wait()
        return torch.cat(dxs, 0), dw_total, db_total, None


class _WaitAll(torch.autograd.Function):
    """Forward: wait for outstanding collectives.  Backward: same (placed so that the gradient
    all-reduce of a later chunk is complete before an earlier chunk's gradient is consumed)."""

    @staticmethod
    def forward(ctx, x):
        sync_comm()
        return x

    @staticmethod
    def backward(ctx, g):
        sync_comm()
        return g


class PipedRowParallelLinear(nn.Module):
    """Level 1 row-parallel layer: GEMM(chunk 1) -> async all-reduce ∥ GEMM(chunk 2) -> all-reduce."""

    def __init__(self, inner: RowPara, chunks: int = 2):
        super().__init__()
        self.row_linear = inner.row_linear
        self.chunks = chunks

    def forward(self, x, residual=None):
        lin = self.row_linear
        parts = x.chunk(self.chunks, dim=0) if x.shape[0] >= self.chunks else (x,)
        outs = []
        for p in parts:
            outs.append(_AsyncReduce.apply(k_linear(p, lin.weight, None)))   # reduce of chunk i runs under GEMM i+1
        outs = [_WaitAll.apply(o) for o in outs]                              # results are read only after the wait
        y = torch.cat(outs, dim=0)
        if lin.bias is not None:
            y = y + lin.bias
        return y if residual is None else y + residual


class PipedColumnParallelLinear(nn.Module):
    """Level 1 column-parallel layer: the data-gradient all-reduce of chunk 2 runs while chunk 1's
    gradient GEMMs execute."""

    def __init__(self, inner: ColPara, chunks: int = 2):
        super().__init__()
        self.col_linear = inner.col_linear
        self.chunks = chunks

    def forward(self, x, residual=None):
        lin = self.col_linear
        y = _PipedColumnLinear.apply(x, lin.weight, lin.bias, self.chunks)
        return y if residual is None else y + residual


class ChunkPipelinedBlock(nn.Module):
    """Levels 2/3: runs ``block`` on 2 or 4 batch chunks.  Because every chunk's row-parallel
    all-reduce is asynchronous (level-1 layers inside), the collective of chunk *i* overlaps the
    GEMMs of chunk *i+1*."""

    def __init__(self, block: nn.Module, chunks: int):
        super().__init__()
        self.block, self.chunks = block, chunks

    def forward(self, hidden_states, *args, **kwargs):
        if hidden_states.shape[0] < self.chunks:
            return self.block(hidden_states, *args, **kwargs)
        outs = [self.block(h, *args, **kwargs) for h in hidden_states.chunk(self.chunks, dim=0)]
        return torch.cat(outs, dim=0)


def apply_tp_overlap(model: nn.Module, level: int, comm_mode: str = "nccl", block_classes=()):
    """Rewrites tensor-parallel layers for the requested overlap level; returns how many were changed."""
    if level <= 0 or mpu.get_model_parallel_world_size() == 1 or comm_mode == "fused":
        return 0
    changed = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, RowPara) and not child.row_linear.sequence_parallel:
                setattr(parent, name, PipedRowParallelLinear(child))
                changed += 1
            elif isinstance(child, ColPara) and not child.col_linear.sequence_parallel and \
                    not child.col_linear.gather_output:
                setattr(parent, name, PipedColumnParallelLinear(child))
                changed += 1
    if level >= 2 and block_classes:
        chunks = 2 if level == 2 else 4
        for parent in list(model.modules()):
            for name, child in list(parent.named_children()):
                if isinstance(child, tuple(block_classes)) and not isinstance(parent, ChunkPipelinedBlock):
                    setattr(parent, name, ChunkPipelinedBlock(child, chunks))
    return changed
