"""DeepSeek-V2-Lite-shape mixture-of-experts decoder: multi-head latent attention (compressed KV with
a decoupled rotary part), a dense SwiGLU MLP in the first layer(s) and routed + shared experts in the
others, with Hugging Face module names (``model.layers.{i}.self_attn.{q_proj, kv_a_proj_with_mqa,
kv_a_layernorm, kv_b_proj, o_proj}``, ``mlp.gate``, ``mlp.experts``, ``mlp.shared_experts``).

The routed experts of a layer are stored stacked (``mlp.experts.gate_up_proj [E_local, 2F, H]``,
``mlp.experts.down_proj [E_local, H, F]``) and split over the expert-parallel group
(``merak_b200.parallel.expert``).  The reference has no MoE model; this family covers the
expert-parallel workload (27 layers, d_model 2048, 16 heads, kv_lora_rank 512, 64 routed + 2 shared
experts, top-6, expert d_ff 1408, vocab 102400).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.attention import flash_attention
from ..ops.cross_entropy import softmax_cross_entropy
from ..ops.elementwise import apply_rope, rope_tables, swiglu
from ..ops.modules import Embedding, Linear, RMSNorm, expose_fused_projection
from ..parallel.expert import MoELayer


@dataclass
class DeepseekV2Config:
    vocab_size: int = 102400
    hidden_size: int = 2048
    intermediate_size: int = 10944
    moe_intermediate_size: int = 1408
    num_hidden_layers: int = 27
    num_attention_heads: int = 16
    kv_lora_rank: int = 512
    q_lora_rank: Optional[int] = None
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    n_routed_experts: int = 64
    n_shared_experts: int = 2
    num_experts_per_tok: int = 6
    first_k_dense_replace: int = 1
    moe_layer_freq: int = 1
    routed_scaling_factor: float = 1.0
    norm_topk_prob: bool = False
    aux_loss_alpha: float = 0.001
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    initializer_range: float = 0.006
    tie_word_embeddings: bool = False
    model_type: str = "deepseek_v2"


class DeepseekV2Attention(nn.Module):
    """Multi-head latent attention.  K and V are expanded from a shared ``kv_lora_rank`` latent; every
    head's key is ``[k_nope (128) | k_rope (64, one per token, shared by the heads)]``."""

    def __init__(self, config: DeepseekV2Config):
        super().__init__()
        c = config
        self.config = c
        self.num_heads = c.num_attention_heads
        self.q_head_dim = c.qk_nope_head_dim + c.qk_rope_head_dim
        self.q_proj = Linear(c.hidden_size, self.num_heads * self.q_head_dim, bias=False)
        self.kv_a_proj_with_mqa = Linear(c.hidden_size, c.kv_lora_rank + c.qk_rope_head_dim, bias=False)
        self.kv_a_layernorm = RMSNorm(c.kv_lora_rank, eps=c.rms_norm_eps)
        self.kv_b_proj = Linear(c.kv_lora_rank, self.num_heads * (c.qk_nope_head_dim + c.v_head_dim), bias=False)
        self.o_proj = Linear(self.num_heads * c.v_head_dim, c.hidden_size, bias=False)
        self.scale = self.q_head_dim ** -0.5
        self._rope = None

    def _tables(self, device):
        if self._rope is None or self._rope[0].device != device:
            self._rope = rope_tables(self.config.max_position_embeddings, self.config.qk_rope_head_dim,
                                     self.config.rope_theta, device)
        return self._rope

    def forward(self, x, residual=None, position_ids=None):
        c = self.config
        B, L, _ = x.shape
        Hh, dn, dr, dv = self.num_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim
        q = self.q_proj(x).view(B, L, Hh, dn + dr)
        ckv = self.kv_a_proj_with_mqa(x)
        latent, k_rope = ckv[..., :c.kv_lora_rank], ckv[..., c.kv_lora_rank:]
        kv = self.kv_b_proj(self.kv_a_layernorm(latent.contiguous())).view(B, L, Hh, dn + dv)
        cos, sin = self._tables(x.device)
        q_rope = apply_rope(q[..., dn:].contiguous(), cos, sin, position_ids)
        k_rope = apply_rope(k_rope.reshape(B, L, 1, dr).contiguous(), cos, sin, position_ids)
        qf = torch.cat([q[..., :dn], q_rope], dim=-1)
        kf = torch.cat([kv[..., :dn], k_rope.expand(B, L, Hh, dr)], dim=-1)
        v = kv[..., dn:]
        ctx = _mla_attention(qf, kf, v, self.scale)
        ctx = ctx.reshape(B, L, Hh * dv)
        return self.o_proj(ctx, residual) if type(self.o_proj) is Linear else (
            self.o_proj(ctx) if residual is None else self.o_proj(ctx) + residual)


def _mla_attention(q, k, v, scale):
    """Causal attention with a 192-wide query/key and a 128-wide value.  Head dims the flash kernel
    supports (q, k, v all 64 or 128 wide) go to it; the 192/128 shape uses the library SDPA call
    until the kernel grows a split-key variant."""
    if q.shape[-1] == v.shape[-1] and q.shape[-1] in (64, 128):
        return flash_attention(q, k, v, causal=True, scale=scale)
    from ..ops import _lib
    _lib.note_library_fallback("attention with a 192-wide key", q)
    out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                         scale=scale)
    return out.transpose(1, 2)


class DeepseekV2MLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__()
        self.gate_up_proj = Linear(hidden_size, 2 * intermediate_size, bias=False)
        self.gate_up_proj.fused_parts = 2
        self.down_proj = Linear(intermediate_size, hidden_size, bias=False)
        expose_fused_projection(self, "gate_up_proj", ("gate_proj", "up_proj"))

    def forward(self, x, residual=None):
        h = swiglu(self.gate_up_proj(x))
        if type(self.down_proj) is Linear:
            return self.down_proj(h, residual)
        y = self.down_proj(h)
        return y if residual is None else y + residual


class MoEDecoderLayer(nn.Module):
    def __init__(self, config: DeepseekV2Config, layer_idx: int):
        super().__init__()
        c = config
        self.self_attn = DeepseekV2Attention(c)
        self.is_moe = (c.n_routed_experts > 0 and layer_idx >= c.first_k_dense_replace
                       and layer_idx % c.moe_layer_freq == 0)
        if self.is_moe:
            self.mlp = MoELayer(c.hidden_size, c.moe_intermediate_size, c.n_routed_experts, c.num_experts_per_tok,
                                num_shared=c.n_shared_experts, scaling=c.routed_scaling_factor,
                                norm_topk_prob=c.norm_topk_prob, aux_loss_alpha=c.aux_loss_alpha,
                                std=c.initializer_range, seed=1000 + layer_idx)
        else:
            self.mlp = DeepseekV2MLP(c.hidden_size, c.intermediate_size)
        self.input_layernorm = RMSNorm(c.hidden_size, eps=c.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(c.hidden_size, eps=c.rms_norm_eps)

    def forward(self, hidden_states, position_ids=None):
        a = self.self_attn(self.input_layernorm(hidden_states), hidden_states, position_ids)
        h = self.post_attention_layernorm(a)
        if self.is_moe:
            return a + self.mlp(h)
        return self.mlp(h, a)


class DeepseekV2Model(nn.Module):
    def __init__(self, config: DeepseekV2Config):
        super().__init__()
        self.config = config
        self.embed_tokens = Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([MoEDecoderLayer(config, i) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, input_ids, position_ids=None):
        h = self.embed_tokens(input_ids)
        for l in self.layers:
            h = l(h, position_ids)
        return self.norm(h)


class DeepseekV2ForCausalLM(nn.Module):
    """``forward(input_ids, labels)`` -> logits or ``(loss, logits)``; the router auxiliary losses of
    the layers are added to the loss."""

    def __init__(self, config: DeepseekV2Config):
        super().__init__()
        self.config = config
        self.model = DeepseekV2Model(config)
        self.lm_head = Linear(config.hidden_size, config.vocab_size, bias=False)
        std = config.initializer_range
        for m in self.modules():
            if isinstance(m, nn.Linear) or isinstance(m, nn.Embedding):
                nn.init.normal_(m.weight, mean=0.0, std=std)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    def aux_loss(self):
        total = None
        for l in self.model.layers:
            a = getattr(l.mlp, "aux_loss", None)
            if a is not None:
                total = a if total is None else total + a
        return total

    def forward(self, input_ids, labels=None, position_ids=None):
        h = self.model(input_ids, position_ids)
        logits = self.lm_head(h)
        if labels is None:
            return logits
        loss = softmax_cross_entropy(logits[:, :-1, :], labels[:, 1:])
        aux = self.aux_loss()
        if aux is not None:
            loss = loss + aux.to(loss.dtype)
        return loss, logits


def deepseek_v2_config(name: str = "deepseek-v2-lite", **overrides) -> DeepseekV2Config:
    presets = {
        "deepseek-v2-lite": dict(),
        "deepseek-tiny": dict(vocab_size=512, hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
                              num_hidden_layers=3, num_attention_heads=4, kv_lora_rank=32, qk_nope_head_dim=32,
                              qk_rope_head_dim=16, v_head_dim=32, n_routed_experts=8, n_shared_experts=1,
                              num_experts_per_tok=2, max_position_embeddings=128, initializer_range=0.02),
    }
    cfg = dict(presets[name])
    cfg.update(overrides)
    return DeepseekV2Config(**cfg)
