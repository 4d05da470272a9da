"""Sub-pipelined tensor model parallelism: hide tensor-parallel all-reduces behind GEMMs by
splitting a micro-batch into chunks (``args.tp_overlapping_level``).

* level 1 - inside one linear layer (Merak/core/tensor_parallel/mp_layers.py:187-497): the input is
  cut in two along dim 0; a row-parallel layer launches the all-reduce of chunk 1 asynchronously
  while the GEMM of chunk 2 runs; a column-parallel layer does the same for the data-gradient
  all-reduce in its backward pass.
* level 2 / 3 - across a transformer block (Merak/core/tensor_parallel/transformer_blocks.py:99-777):
  the block is cut into five stages at its communication points and runs as a software pipeline
  over 2 (level 2) or 4 (level 3) batch chunks, forward and backward, with hand-chosen stage
  order in both directions (``_StagedBlock``): each all-reduce is in flight while another chunk's
  stage computes.  The reference's level 3 instead carries the last all-reduce of a layer into
  the next layer; with four chunks in flight that reduce is hidden behind three other chunks'
  stages inside the layer, and the interface between layers stays one tensor.

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
from . import mappings as M
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


# ---------------------------------------------------------------------------------------------
# levels 2 / 3: a transformer block as a software pipeline over batch chunks
# ---------------------------------------------------------------------------------------------
def _row_partial(row: nn.Module, x):
    """The un-reduced product of a row-parallel layer; the pipeline launches its all-reduce when the
    stage returns and the next stage adds the bias."""
    return k_linear(x, row.row_linear.weight, None)


def _col_local(col: nn.Module, x):
    """A column-parallel layer without its communication: the pipeline launches the all-reduce of
    the input gradient itself when the stage's backward has produced it."""
    lin = col.col_linear
    return k_linear(x, lin.weight, lin.bias)


def _row_bias(row: nn.Module):
    return row.row_linear.bias


def block_stages(block: nn.Module):
    """Cuts a transformer block into five stages at its communication points (reference:
    ``PipedTPFunction``'s fp1..fp6, Merak/core/tensor_parallel/transformer_blocks.py:359-491).
    A stage never uses a tensor whose all-reduce it launched itself:

    ====  ==========================================================  =========================
    P1    first norm                                                  backward starts by waiting
    P2    column-parallel QKV, attention, row-parallel GEMM          ends by launching a reduce
    P3    (wait) bias + dropout + residual, second norm
    P4    column-parallel FC, activation, row-parallel GEMM           ends by launching a reduce
    P5    (wait) bias + dropout + residual
    ====  ==========================================================  =========================

    In the backward pass the column-parallel layers at the head of P2 / P4 launch the all-reduce
    of their input gradient, which P1 / P3 of the same chunk consume."""
    name = type(block).__name__
    if name == "GPT2Block":
        from ..ops.attention import flash_attention_packed
        from ..ops.elementwise import dropout
        attn, mlp = block.attn, block.mlp
        if not (isinstance(attn.c_proj, RowPara) and isinstance(mlp.c_proj, RowPara) and
                isinstance(attn.c_attn, ColPara) and isinstance(mlp.c_fc, ColPara)):
            return None

        def p1(h):
            return h, block.ln_1(h)

        def p2(h, x):
            qkv = _col_local(attn.c_attn, x)
            B, L = qkv.shape[0], qkv.shape[1]
            local = qkv.shape[-1] // 3
            heads = local // attn.head_dim
            ctx = flash_attention_packed(qkv.view(B, L, 3 * heads, attn.head_dim), heads, heads, causal=True)
            return h, _row_partial(attn.c_proj, ctx.reshape(B, L, local))

        def p3(h, part):
            bias = _row_bias(attn.c_proj)
            a = h + dropout(part if bias is None else part + bias, attn.resid_pdrop, block.training)
            return a, block.ln_2(a)

        def p4(a, y):
            return a, _row_partial(mlp.c_proj, G.act_forward(mlp.act, _col_local(mlp.c_fc, y)))

        def p5(a, part):
            bias = _row_bias(mlp.c_proj)
            return a + dropout(part if bias is None else part + bias, mlp.resid_pdrop, block.training)

        return [p1, p2, p3, p4, p5]
    return None


STAGE_GROUPS = ((0, 1), (2, 3), (4,))       # stages run back to back for one chunk before the next chunk's turn
REDUCED_OUTPUT = {1: 1, 3: 1}                # stage -> index of the output that is a row-parallel partial sum
REDUCED_INPUT_GRAD = {1: 1, 3: 1}            # stage -> index of the input feeding a column-parallel layer


def _launch_reduce(t: torch.Tensor, handles: list):
    handles.append(dist.all_reduce(t, group=mpu.get_model_parallel_group(), async_op=True))


class _StagedBlock(torch.autograd.Function):
    """Runs the stages of ``block_stages`` over several batch chunks in an interleaved order, in
    the forward AND in the backward pass: while the all-reduce a stage launched for one chunk is in
    flight, a stage of another chunk computes.  Each (chunk, stage) is its own autograd sub-graph on
    detached inputs, so the backward order is chosen here rather than by the autograd engine
    (reference: the hand-staged ``bp1..bp6``, Merak/core/tensor_parallel/transformer_blocks.py:
    425-491)."""

    @staticmethod
    def forward(ctx, stages, n_chunks, *chunks):
        handles = [[] for _ in range(n_chunks)]
        state = [(c,) for c in chunks]
        records = {}
        with torch.enable_grad():
            for group in STAGE_GROUPS:
                for c in range(n_chunks):
                    _wait(handles[c])
                    for k in group:
                        ins = tuple(t.detach().requires_grad_(t.is_floating_point()) for t in state[c])
                        outs = stages[k](*ins)
                        outs = outs if isinstance(outs, tuple) else (outs,)
                        records[(c, k)] = (ins, outs)
                        state[c] = outs
                        if k in REDUCED_OUTPUT:        # the group's last stage: the sum travels while others compute
                            _launch_reduce(outs[REDUCED_OUTPUT[k]].detach(), handles[c])
        for h in handles:
            _wait(h)
        ctx.records, ctx.n_chunks, ctx.n_stages = records, n_chunks, len(stages)
        return tuple(state[c][0].detach() for c in range(n_chunks))

    @staticmethod
    def backward(ctx, *gouts):
        n, records = ctx.n_chunks, ctx.records
        handles = [[] for _ in range(n)]
        grads = [(g,) for g in gouts]
        for group in reversed(STAGE_GROUPS):
            for c in reversed(range(n)):
                for k in reversed(group):
                    _wait(handles[c])                  # the input gradient the previous stage left in flight
                    ins, outs = records.pop((c, k))
                    pairs = [(o, g) for o, g in zip(outs, grads[c]) if g is not None and o.requires_grad]
                    torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
                    grads[c] = tuple(i.grad for i in ins)
                    if k in REDUCED_INPUT_GRAD and grads[c][REDUCED_INPUT_GRAD[k]] is not None:
                        # every rank holds a partial input gradient of its column shard: sum them while
                        # the other chunks' stages run
                        _launch_reduce(grads[c][REDUCED_INPUT_GRAD[k]], handles[c])
        for h in handles:
            _wait(h)
        return (None, None) + tuple(g[0] for g in grads)


def _wait(handles: list):
    while handles:
        handles.pop(0).wait()


class ChunkPipelinedBlock(nn.Module):
    """Levels 2 / 3: the block runs as a software pipeline over 2 (level 2) or 4 (level 3) batch
    chunks, stage by stage (``_StagedBlock``), so that every tensor-parallel all-reduce of a chunk,
    forward and backward, is in flight while another chunk computes.  Blocks ``block_stages`` does
    not know how to cut fall back to running the chunks one after the other."""

    def __init__(self, block: nn.Module, chunks: int):
        super().__init__()
        self.block, self.chunks = block, chunks

    def forward(self, hidden_states, *args, **kwargs):
        if hidden_states.shape[0] < self.chunks:
            return self.block(hidden_states, *args, **kwargs)
        parts = hidden_states.chunk(self.chunks, dim=0)
        stages = block_stages(self.block) if not args and not kwargs else None
        if stages is None or mpu.get_model_parallel_world_size() == 1:
            return torch.cat([self.block(h, *args, **kwargs) for h in parts], dim=0)
        outs = _StagedBlock.apply(stages, len(parts), *parts)
        return torch.cat(outs, dim=0)


def apply_tp_overlap(model: nn.Module, level: int, comm_mode: str = "nccl", block_classes=()):
    """Rewrites tensor-parallel layers for the requested overlap level; returns how many were changed."""
    if level <= 0 or mpu.get_model_parallel_world_size() == 1 or comm_mode == "fused":
        return 0
    changed = 0
    staged = set()
    if level >= 2 and block_classes:
        # whole blocks become chunk pipelines; the layers inside keep their plain form (the pipeline
        # defers their all-reduces itself)
        chunks = 2 if level == 2 else 4
        for parent in list(model.modules()):
            for name, child in list(parent.named_children()):
                if isinstance(child, tuple(block_classes)) and not isinstance(parent, ChunkPipelinedBlock) and \
                        block_stages(child) is not None:
                    setattr(parent, name, ChunkPipelinedBlock(child, chunks))
                    staged.update(id(m) for m in child.modules())
                    changed += 1
    for parent in list(model.modules()):
        if id(parent) in staged:
            continue
        for name, child in list(parent.named_children()):
            if isinstance(child, RowPara) and not child.row_linear.sequence_parallel:
                setattr(parent, name, PipedRowParallelLinear(child))
                changed += 1
            elif isinstance(child, ColPara) and not child.col_linear.sequence_parallel and \
                    not child.col_linear.gather_output:
                setattr(parent, name, PipedColumnParallelLinear(child))
                changed += 1
    return changed
