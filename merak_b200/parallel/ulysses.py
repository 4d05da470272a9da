"""Ulysses-style sequence parallelism on the dedicated ``sequence`` axis of the grid
(Merak/core/sequence_parallel/operation.py:43-90, modeling/llama.py:162-334).

Between attention blocks every rank holds ``[B, L/sp, H]``.  Inside attention, after the q/k/v
projection, an all-to-all trades the sequence shard for a head shard (``[B, L, heads/sp, D]``), the
rotary embedding and flash attention run on the full sequence with the local heads, and a second
all-to-all restores ``[B, L/sp, heads, D]`` before the output projection.  The sequence is split
once after the token embedding and gathered once after the final norm, so the language-model head
and the loss see the full sequence, as in the reference.

Supported model family: Llama-style decoders (the reference registry covers the same family only).
Head counts (query and key/value) must be divisible by ``sp * tp``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..models import llama as L
from ..ops.attention import flash_attention
from ..ops.elementwise import apply_rope
from . import mappings as M
from . import mpu


class LlamaAttentionSP(L.LlamaAttention):
    """Same parameters as ``LlamaAttention``; forward exchanges sequence shards for head shards."""

    def forward(self, x, residual=None, position_ids=None):
        qkv = self.qkv_proj(x)
        B, Ls = qkv.shape[0], qkv.shape[1]
        ratio = self.num_heads // self.num_key_value_heads
        kv_local = qkv.shape[-1] // ((ratio + 2) * self.head_dim)
        q_local = kv_local * ratio
        sp = mpu.get_sequence_parallel_world_size()
        if q_local % sp or kv_local % sp:
            raise ValueError("heads (%d query, %d kv) are not divisible by the sequence-parallel degree %d" %
                             (q_local, kv_local, sp))
        qkv = qkv.view(B, Ls, q_local + 2 * kv_local, self.head_dim)
        q, k, v = qkv[:, :, :q_local], qkv[:, :, q_local:q_local + kv_local], qkv[:, :, q_local + kv_local:]
        # [B, L/sp, h, D] -> [B, L, h/sp, D]
        q = M.all_to_all_sequence_parallel_region(q.contiguous(), scatter_dim=2, gather_dim=1)
        k = M.all_to_all_sequence_parallel_region(k.contiguous(), scatter_dim=2, gather_dim=1)
        v = M.all_to_all_sequence_parallel_region(v.contiguous(), scatter_dim=2, gather_dim=1)
        cos, sin = self._tables(x.device)
        q, k = apply_rope(q, cos, sin, position_ids), apply_rope(k, cos, sin, position_ids)
        ctx = flash_attention(q, k, v, causal=True)
        # [B, L, h/sp, D] -> [B, L/sp, h, D]
        ctx = M.all_to_all_sequence_parallel_region(ctx.contiguous(), scatter_dim=1, gather_dim=2)
        ctx = ctx.reshape(B, Ls, q_local * self.head_dim)
        y = self.o_proj(ctx)
        return y if residual is None else y + residual


class SplitSequence(nn.Module):
    """Wraps the module that starts the sequence-parallel region (the token embedding)."""

    def __init__(self, inner: nn.Module, dim: int = 1):
        super().__init__()
        self.inner, self.dim = inner, dim

    @property
    def weight(self):
        return self.inner.weight

    def forward(self, *a, **k):
        return M.split_for_sequence_parallel_region(self.inner(*a, **k), self.dim)


class GatherSequence(nn.Module):
    """Wraps the module that ends the sequence-parallel region (the final norm)."""

    def __init__(self, inner: nn.Module, dim: int = 1):
        super().__init__()
        self.inner, self.dim = inner, dim

    def forward(self, *a, **k):
        return M.gather_for_sequence_parallel_region(self.inner(*a, **k), self.dim)


MODELS_SP_CONFIG = {"llama": {L.LlamaAttention: LlamaAttentionSP}}


def get_leaf_modules_for_sp(model):
    """Classes the tracer must treat as leaves when sequence parallelism is on."""
    return (L.LlamaDecoderLayer, SplitSequence, GatherSequence)


def replace_to_sp_module(model: nn.Module, args=None):
    mt = getattr(getattr(model, "config", None), "model_type", None)
    table = MODELS_SP_CONFIG.get(mt)
    if table is None:
        raise ValueError("sequence parallelism supports %s models, got %r" % (sorted(MODELS_SP_CONFIG), mt))
    dim = getattr(args, "sequence_dim", 1) if args is not None else 1
    for m in model.modules():
        for src, dst in table.items():
            if type(m) is src:
                m.__class__ = dst
    inner = model.model
    if not isinstance(inner.embed_tokens, SplitSequence):
        inner.embed_tokens = SplitSequence(inner.embed_tokens, dim)
    if not isinstance(inner.norm, GatherSequence):
        inner.norm = GatherSequence(inner.norm, dim)
    # parameters of the blocks see only this rank's tokens: their gradients are summed over the
    # sequence group by the engine
    for name, p in model.named_parameters():
        p.ulysses_parallel = True
    # the output projection runs after the gather, on the full sequence, on every rank: its
    # gradient is already complete (and identical) everywhere
    # and so is the embedding's: the backward of the split gathers the gradient slices of all ranks
    head = getattr(model, "lm_head", None)
    for mod in (head, inner.embed_tokens):
        if mod is not None:
            for p in mod.parameters():
                p.ulysses_replicated = True
    return model
