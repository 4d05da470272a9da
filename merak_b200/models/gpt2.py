"""GPT-2 decoder with Hugging Face parameter names (``transformer.h.{i}.attn.c_attn`` ...), built
on the framework's kernels: fused QKV GEMM -> flash attention -> projection GEMM with residual
epilogue, fused residual+LayerNorm, MLP (GEMM, activation pass at memory speed, GEMM).

The module tree and names follow ``transformers``' ``GPT2LMHeadModel`` so the reference's GPT-2
feature dict (Merak/core/tensor_parallel/mp_mapping.py:21-29: c_attn/c_fc column-parallel,
c_proj row-parallel), its ``layer_split`` cut points (Merak/core/fx/graph_shard/layer_config.py)
and checkpoint keys apply unchanged.  Weights use the ``nn.Linear`` ``[out, in]`` layout (HF's
``Conv1D`` stores the transpose; the conversion tools transpose on import/export).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from ..ops import gemm as G
from ..ops.attention import flash_attention, flash_attention_packed
from ..ops.cross_entropy import softmax_cross_entropy
from ..ops.elementwise import dropout, embedding_sum
from ..ops.linear import linear as k_linear, mlp as k_mlp
from ..ops.modules import Dropout, Embedding, LayerNorm, Linear


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    n_inner: Optional[int] = None
    activation_function: str = "gelu_new"
    resid_pdrop: float = 0.1
    embd_pdrop: float = 0.1
    attn_pdrop: float = 0.1
    layer_norm_epsilon: float = 1e-5
    initializer_range: float = 0.02
    tie_word_embeddings: bool = True
    model_type: str = "gpt2"
    use_cache: bool = False

    @property
    def hidden_size(self):
        return self.n_embd

    @property
    def num_hidden_layers(self):
        return self.n_layer

    @property
    def num_attention_heads(self):
        return self.n_head

    @property
    def max_position_embeddings(self):
        return self.n_positions


class GPT2Attention(nn.Module):
    def __init__(self, config: GPT2Config):
        super().__init__()
        self.embed_dim = config.n_embd
        self.num_heads = config.n_head
        self.head_dim = self.embed_dim // self.num_heads
        self.split_size = self.embed_dim
        self.c_attn = Linear(self.embed_dim, 3 * self.embed_dim)
        self.c_attn.fused_parts = 3          # rows are [q; k; v]: shard each part separately under TP
        self.c_proj = Linear(self.embed_dim, self.embed_dim)
        self.c_attn.tp_unit = self.c_proj.tp_unit = self.head_dim     # heads are never split between ranks
        self.resid_pdrop = config.resid_pdrop
        self.attn_pdrop = float(config.attn_pdrop or 0.0)

    def forward(self, x, residual=None):
        qkv = self.c_attn(x)
        B, L = qkv.shape[0], qkv.shape[1]     # the projection may have gathered the sequence
        local = qkv.shape[-1] // 3
        heads = local // self.head_dim
        ctx = flash_attention_packed(qkv.view(B, L, 3 * heads, self.head_dim), heads, heads, causal=True,
                                     dropout_p=self.attn_pdrop if self.training else 0.0)
        ctx = ctx.reshape(B, L, local)
        if residual is not None and not (self.training and self.resid_pdrop > 0):
            return self.c_proj(ctx, residual)
        out = dropout(self.c_proj(ctx), self.resid_pdrop, self.training)
        return out if residual is None else out + residual


class GPT2MLP(nn.Module):
    def __init__(self, config: GPT2Config):
        super().__init__()
        inner = config.n_inner or 4 * config.n_embd
        self.c_fc = Linear(config.n_embd, inner)
        self.c_proj = Linear(inner, config.n_embd)
        self.act = G.ACT_BY_NAME[config.activation_function]
        self.resid_pdrop = config.resid_pdrop

    def forward(self, x, residual=None):
        fused_res = residual is not None and not (self.training and self.resid_pdrop > 0)
        if type(self.c_fc) is Linear and type(self.c_proj) is Linear:
            y = k_mlp(x, self.c_fc.weight, self.c_fc.bias, self.c_proj.weight, self.c_proj.bias, self.act,
                      residual if fused_res else None)
        else:   # tensor-parallel wrappers: column -> activation -> row
            h = G.act_forward(self.act, self.c_fc(x))
            y = self.c_proj(h)
            if fused_res:
                y = y + residual
        if fused_res:
            return y
        y = dropout(y, self.resid_pdrop, self.training)
        return y if residual is None else y + residual


class GPT2Block(nn.Module):
    def __init__(self, config: GPT2Config):
        super().__init__()
        self.ln_1 = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.attn = GPT2Attention(config)
        self.ln_2 = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.mlp = GPT2MLP(config)

    def forward(self, hidden_states):
        a = self.attn(self.ln_1(hidden_states), hidden_states)
        return self.mlp(self.ln_2(a), a)


class GPT2Model(nn.Module):
    def __init__(self, config: GPT2Config):
        super().__init__()
        self.config = config
        self.wte = Embedding(config.vocab_size, config.n_embd)
        self.wpe = Embedding(config.n_positions, config.n_embd)
        self.drop = Dropout(config.embd_pdrop)
        self.h = nn.ModuleList([GPT2Block(config) for _ in range(config.n_layer)])
        self.ln_f = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)

    def forward(self, input_ids):
        pos = torch.arange(input_ids.size(1), device=input_ids.device).unsqueeze(0)
        h = self.drop(self.wte(input_ids) + self.wpe(pos))
        for blk in self.h:
            h = blk(h)
        return self.ln_f(h)


class GPT2LMHeadModel(nn.Module):
    """Returns logits, or ``(loss, logits)`` when ``labels`` are given (next-token shift inside)."""

    def __init__(self, config: GPT2Config):
        super().__init__()
        self.config = config
        self.transformer = GPT2Model(config)
        self.lm_head = Linear(config.n_embd, config.vocab_size, bias=False)
        self.apply(self._init_weights)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.transformer.wte.weight
        for name, p in self.named_parameters():
            if name.endswith("c_proj.weight"):
                nn.init.normal_(p, mean=0.0, std=config.initializer_range / (2 * config.n_layer) ** 0.5)

    def _init_weights(self, m):
        std = self.config.initializer_range
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, mean=0.0, std=std)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=std)
        elif isinstance(m, nn.LayerNorm):
            nn.init.ones_(m.weight)
            nn.init.zeros_(m.bias)

    def get_input_embeddings(self):
        return self.transformer.wte

    def get_output_embeddings(self):
        return self.lm_head

    def forward(self, input_ids, labels=None):
        h = self.transformer(input_ids)
        logits = self.lm_head(h)
        if labels is None:
            return logits
        loss = softmax_cross_entropy(logits[:, :-1, :], labels[:, 1:])
        return loss, logits


def gpt2_config(name: str = "gpt2", **overrides) -> GPT2Config:
    presets = {
        "gpt2": dict(n_embd=768, n_layer=12, n_head=12),
        "gpt2-medium": dict(n_embd=1024, n_layer=24, n_head=16),
        "gpt2-large": dict(n_embd=1280, n_layer=36, n_head=20),
        "gpt2-xl": dict(n_embd=1600, n_layer=48, n_head=25),
        "gpt2-tiny": dict(n_embd=256, n_layer=4, n_head=4, n_positions=128),
    }
    cfg = dict(presets[name])
    cfg.update(overrides)
    return GPT2Config(**cfg)
