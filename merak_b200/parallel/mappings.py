"""Autograd-aware communication primitives between parallel "regions".

Tensor-parallel family (Merak/core/mpu/mappings.py:308-402): identity/all-reduce pairs for
column- and row-parallel linears, last-dim scatter/gather.  Megatron-style sequence parallelism
(absent from the reference, required by Llama tp+sp training): all-gather / reduce-scatter along
the *sequence* dimension inside the tensor-parallel group.  Ulysses family
(Merak/core/mpu/mappings.py:180-267, 405-476): head<->sequence all-to-all and sequence
split/gather on the dedicated sequence axis.

Every primitive is a no-op when its group has one rank, so single-process code paths need no
``torch.distributed`` initialisation.
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist

from . import mpu


def _size(group_getter_size) -> int:
    return group_getter_size()


# ---------------------------------------------------------------------------------------------
# raw collectives on the tensor-parallel group
# ---------------------------------------------------------------------------------------------
def _tp():
    return mpu.get_model_parallel_group(), mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()


_SHAPE_ONLY = [False]


@contextlib.contextmanager
def shape_only_collectives():
    """While a model is being exported to a graph only output shapes matter: every collective of
    this module becomes a local operation with the same output shape (all-reduce: identity;
    all-gather: the local tensor repeated; reduce-scatter: the first chunk).  The folded graph calls
    the real wrappers afterwards (``fx.export_trace``)."""
    prev, _SHAPE_ONLY[0] = _SHAPE_ONLY[0], True
    try:
        yield
    finally:
        _SHAPE_ONLY[0] = prev


def _reduce(x):
    group, n, _ = _tp()
    if n == 1 or _SHAPE_ONLY[0]:
        return x
    x = x.contiguous()
    dist.all_reduce(x, group=group)
    return x


def _all_gather_stacked(x, group, n):
    """All-gather into a ``[n, *x.shape]`` tensor (allocated as the flat concatenation every
    backend accepts)."""
    x = x.contiguous()
    if _SHAPE_ONLY[0]:
        return x.unsqueeze(0).expand((n,) + tuple(x.shape)).contiguous()
    flat = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(flat, x, group=group)
    return flat.view((n,) + tuple(x.shape))


def _split_last(x):
    _, n, r = _tp()
    if n == 1:
        return x
    assert x.shape[-1] % n == 0
    return x.chunk(n, dim=-1)[r].contiguous()


def _gather_last(x):
    group, n, _ = _tp()
    if n == 1:
        return x
    out = _all_gather_stacked(x, group, n)
    return torch.cat(list(out.unbind(0)), dim=-1)


def _gather_dim(x, dim, group, n):
    if n == 1:
        return x
    out = _all_gather_stacked(x, group, n)
    if dim == 0:
        return out.view((n * x.shape[0],) + tuple(x.shape[1:]))
    return torch.cat(list(out.unbind(0)), dim=dim)


def _split_dim(x, dim, n, r):
    if n == 1:
        return x
    assert x.shape[dim] % n == 0, "dimension %d of size %d not divisible by %d" % (dim, x.shape[dim], n)
    return x.chunk(n, dim=dim)[r].contiguous()


def _reduce_scatter_dim(x, dim, group, n):
    if n == 1:
        return x
    assert x.shape[dim] % n == 0
    if _SHAPE_ONLY[0]:
        return x.chunk(n, dim=dim)[0].contiguous()
    parts = torch.cat([c.contiguous() for c in x.chunk(n, dim=dim)], 0)     # [n*chunk0, ...]
    out = torch.empty((parts.shape[0] // n,) + tuple(parts.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, parts, group=group)
    return out


# ---------------------------------------------------------------------------------------------
# tensor-parallel regions
# ---------------------------------------------------------------------------------------------
class _CopyToModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        return _reduce(g)


class _ReduceFromModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _reduce(x)

    @staticmethod
    def backward(ctx, g):
        return g


class _ScatterToModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _split_last(x)

    @staticmethod
    def backward(ctx, g):
        return _gather_last(g)


class _GatherFromModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _gather_last(x)

    @staticmethod
    def backward(ctx, g):
        return _split_last(g)


class _ReduceScatterToSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        group, n, _ = _tp()
        return _reduce_scatter_dim(x, dim, group, n)

    @staticmethod
    def backward(ctx, g):
        group, n, _ = _tp()
        return _gather_dim(g, ctx.dim, group, n), None


class _GatherFromSequenceParallelRegion(torch.autograd.Function):
    """All-gather along the sequence dim; backward reduce-scatters (the input feeds a
    column-parallel GEMM whose data gradient is partial on every rank)."""

    @staticmethod
    def forward(ctx, x, dim, reduce_scatter_grad):
        ctx.dim, ctx.rs = dim, reduce_scatter_grad
        group, n, _ = _tp()
        return _gather_dim(x, dim, group, n)

    @staticmethod
    def backward(ctx, g):
        group, n, r = _tp()
        if ctx.rs:
            return _reduce_scatter_dim(g, ctx.dim, group, n), None, None
        return _split_dim(g, ctx.dim, n, r), None, None


class _ScatterToSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        _, n, r = _tp()
        return _split_dim(x, dim, n, r)

    @staticmethod
    def backward(ctx, g):
        group, n, _ = _tp()
        return _gather_dim(g, ctx.dim, group, n), None


def copy_to_model_parallel_region(x):
    return x if mpu.get_model_parallel_world_size() == 1 else _CopyToModelParallelRegion.apply(x)


def reduce_from_model_parallel_region(x):
    return x if mpu.get_model_parallel_world_size() == 1 else _ReduceFromModelParallelRegion.apply(x)


def scatter_to_model_parallel_region(x):
    return x if mpu.get_model_parallel_world_size() == 1 else _ScatterToModelParallelRegion.apply(x)


def gather_from_model_parallel_region(x):
    return x if mpu.get_model_parallel_world_size() == 1 else _GatherFromModelParallelRegion.apply(x)


def reduce_scatter_to_sequence_parallel_region(x, dim=1):
    return x if mpu.get_model_parallel_world_size() == 1 else _ReduceScatterToSequenceParallelRegion.apply(x, dim)


def gather_from_sequence_parallel_region(x, dim=1, reduce_scatter_grad=True):
    if mpu.get_model_parallel_world_size() == 1:
        return x
    return _GatherFromSequenceParallelRegion.apply(x, dim, reduce_scatter_grad)


def scatter_to_sequence_parallel_region(x, dim=1):
    return x if mpu.get_model_parallel_world_size() == 1 else _ScatterToSequenceParallelRegion.apply(x, dim)


# ---------------------------------------------------------------------------------------------
# Ulysses (dedicated sequence axis): all-to-all and split/gather
# ---------------------------------------------------------------------------------------------
def _sp():
    return (mpu.get_sequence_parallel_group(), mpu.get_sequence_parallel_world_size(),
            mpu.get_sequence_parallel_rank())


def _all_to_all(x, scatter_dim, gather_dim, group, n):
    if n == 1:
        return x
    parts = [c.contiguous() for c in x.chunk(n, dim=scatter_dim)]
    send = torch.cat(parts, 0)
    recv = None
    if send.is_cuda:
        # peer-mapped group: every rank stores its blocks straight into the destinations' buffers
        # (the push all-to-all kernel of the expert-parallel path) instead of a library collective
        from . import expert
        comm = expert.get_ep_comm(group, send.device)
        per = parts[0].shape[0]
        flat = send.reshape(n * per, -1)
        if comm is not None and (flat.shape[1] * flat.element_size()) % 16 == 0:
            begin = [k * per for k in range(n + 1)]
            recv = comm.push(flat, begin, [comm.rank * per] * n, n * per, worst_rows=n * per).view_as(send)
    if recv is None:
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
    return torch.cat(list(recv.chunk(n, dim=0)), dim=gather_dim)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scatter_dim, gather_dim):
        ctx.dims = (scatter_dim, gather_dim)
        group, n, _ = _sp()
        return _all_to_all(x, scatter_dim, gather_dim, group, n)

    @staticmethod
    def backward(ctx, g):
        group, n, _ = _sp()
        return _all_to_all(g, ctx.dims[1], ctx.dims[0], group, n), None, None


class _SplitForwardGatherBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        _, n, r = _sp()
        return _split_dim(x, dim, n, r)

    @staticmethod
    def backward(ctx, g):
        group, n, _ = _sp()
        return _gather_dim(g, ctx.dim, group, n), None


class _GatherForwardSplitBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        group, n, _ = _sp()
        return _gather_dim(x, dim, group, n)

    @staticmethod
    def backward(ctx, g):
        _, n, r = _sp()
        return _split_dim(g, ctx.dim, n, r), None


def all_to_all_sequence_parallel_region(x, scatter_dim=2, gather_dim=1):
    return x if mpu.get_sequence_parallel_world_size() == 1 else _AllToAll.apply(x, scatter_dim, gather_dim)


def split_for_sequence_parallel_region(x, dim=1):
    return x if mpu.get_sequence_parallel_world_size() == 1 else _SplitForwardGatherBackward.apply(x, dim)


def gather_for_sequence_parallel_region(x, dim=1):
    return x if mpu.get_sequence_parallel_world_size() == 1 else _GatherForwardSplitBackward.apply(x, dim)
