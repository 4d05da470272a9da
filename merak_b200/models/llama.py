"""Llama-family decoder (RMSNorm, rotary embeddings, grouped-query attention, SwiGLU) on the
framework's kernels, with Hugging Face parameter names for the surrounding modules
(``model.layers.{i}.self_attn`` / ``mlp`` / ``input_layernorm`` ...).

q/k/v and gate/up are fused projections (``qkv_proj``, ``gate_up_proj``) so each is one GEMM; their
state-dict entries appear under the HF names ``q_proj/k_proj/v_proj`` and ``gate_proj/up_proj``.
This is the model of the reference's Llama example (examples/models/llama/run_llama.py:46-93)
and the only family its Ulysses sequence-parallel layers cover
(Merak/core/sequence_parallel/modeling/llama.py:162-334).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from ..ops.attention import flash_attention
from ..ops.cross_entropy import softmax_cross_entropy
from ..ops.elementwise import apply_rope, rope_tables, swiglu
from ..ops.modules import Embedding, Linear, RMSNorm, expose_fused_projection


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    initializer_range: float = 0.02
    tie_word_embeddings: bool = False
    attention_dropout: float = 0.0
    model_type: str = "llama"

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads


class LlamaAttention(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config
        self.num_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.head_dim = config.hidden_size // config.num_attention_heads
        qkv_out = (self.num_heads + 2 * self.num_key_value_heads) * self.head_dim
        self.qkv_proj = Linear(config.hidden_size, qkv_out, bias=False)
        self.qkv_proj.fused_sizes = [self.num_heads * self.head_dim, self.num_key_value_heads * self.head_dim,
                                     self.num_key_value_heads * self.head_dim]
        self.o_proj = Linear(self.num_heads * self.head_dim, config.hidden_size, bias=False)
        self._rope = None
        expose_fused_projection(self, "qkv_proj", ("q_proj", "k_proj", "v_proj"), self.qkv_proj.fused_sizes)

    def _tables(self, device):
        if self._rope is None or self._rope[0].device != device:
            self._rope = rope_tables(self.config.max_position_embeddings, self.head_dim, self.config.rope_theta, device)
        return self._rope

    def forward(self, x, residual=None, position_ids=None):
        qkv = self.qkv_proj(x)
        B, L = qkv.shape[0], qkv.shape[1]     # the projection may have gathered the sequence
        ratio = self.num_heads // self.num_key_value_heads
        kv_local = qkv.shape[-1] // ((ratio + 2) * self.head_dim)      # local kv heads under TP
        q_local = kv_local * ratio
        qkv = qkv.view(B, L, q_local + 2 * kv_local, self.head_dim)
        q, k, v = qkv[:, :, :q_local], qkv[:, :, q_local:q_local + kv_local], qkv[:, :, q_local + kv_local:]
        cos, sin = self._tables(x.device)
        q, k = apply_rope(q, cos, sin, position_ids), apply_rope(k, cos, sin, position_ids)
        ctx = flash_attention(q, k, v, causal=True).reshape(B, L, q_local * self.head_dim)
        return self.o_proj(ctx, residual) if type(self.o_proj) is Linear else (
            self.o_proj(ctx) if residual is None else self.o_proj(ctx) + residual)


class LlamaMLP(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.intermediate_size = config.intermediate_size
        self.gate_up_proj = Linear(config.hidden_size, 2 * config.intermediate_size, bias=False)
        self.gate_up_proj.fused_parts = 2
        self.down_proj = Linear(config.intermediate_size, config.hidden_size, bias=False)
        expose_fused_projection(self, "gate_up_proj", ("gate_proj", "up_proj"))

    def forward(self, x, residual=None):
        h = swiglu(self.gate_up_proj(x))
        if type(self.down_proj) is Linear:
            return self.down_proj(h, residual)
        y = self.down_proj(h)
        return y if residual is None else y + residual


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.self_attn = LlamaAttention(config)
        self.mlp = LlamaMLP(config)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, hidden_states, position_ids=None):
        a = self.self_attn(self.input_layernorm(hidden_states), hidden_states, position_ids)
        return self.mlp(self.post_attention_layernorm(a), a)


class LlamaModel(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config
        self.embed_tokens = Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([LlamaDecoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, input_ids, position_ids=None):
        h = self.embed_tokens(input_ids)
        for l in self.layers:
            h = l(h, position_ids)
        return self.norm(h)


class LlamaForCausalLM(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config
        self.model = LlamaModel(config)
        self.lm_head = Linear(config.hidden_size, config.vocab_size, bias=False)
        std = config.initializer_range
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, mean=0.0, std=std)
            elif isinstance(m, nn.Embedding):
                nn.init.normal_(m.weight, mean=0.0, std=std)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    def forward(self, input_ids, labels=None, position_ids=None):
        h = self.model(input_ids, position_ids)
        logits = self.lm_head(h)
        if labels is None:
            return logits
        return softmax_cross_entropy(logits[:, :-1, :], labels[:, 1:]), logits


def llama_config(name: str = "llama-7b", **overrides) -> LlamaConfig:
    presets = {
        "llama-7b": dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32),
        "llama-13b": dict(hidden_size=5120, intermediate_size=13824, num_hidden_layers=40, num_attention_heads=40),
        "llama-tiny": dict(hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, vocab_size=1024, max_position_embeddings=256),
    }
    cfg = dict(presets[name])
    cfg.update(overrides)
    return LlamaConfig(**cfg)
