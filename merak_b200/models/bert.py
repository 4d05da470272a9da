"""BERT encoder for masked-language-model pre-training on the framework's kernels.

Module names follow ``transformers``' ``BertForMaskedLM`` / ``BertForPreTraining``
(``bert.encoder.layer.{i}.attention.output.dense`` ...), the model family of the reference's
headline example (examples/bert_pretraining/run_bert.py:61-117) and of its BERT feature dict
(Merak/core/tensor_parallel/mp_mapping.py:38-44).  Query/key/value are one fused projection
(``attention.self.qkv``); its state-dict entries are exposed under the Hugging Face names
``query/key/value`` so checkpoints interchange.

Per layer: fused QKV GEMM -> flash attention (bidirectional, optional key-padding bias) ->
output GEMM -> fused dropout+residual+LayerNorm -> MLP (GEMM, GELU pass, GEMM) -> fused
dropout+residual+LayerNorm.
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
from ..ops.linear import linear as k_linear, linear_fork, mlp as k_mlp, mlp_fork as k_mlp_fork
from ..ops.modules import LayerNorm, Linear, expose_fused_projection
from ..ops.norm import fused_norm


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    hidden_act: str = "gelu"
    hidden_dropout_prob: float = 0.1
    attention_probs_dropout_prob: float = 0.1
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-12
    tie_word_embeddings: bool = True
    model_type: str = "bert"


class BertEmbeddings(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.word_embeddings = nn.Embedding(config.vocab_size, config.hidden_size)
        self.position_embeddings = nn.Embedding(config.max_position_embeddings, config.hidden_size)
        self.token_type_embeddings = nn.Embedding(config.type_vocab_size, config.hidden_size)
        self.LayerNorm = LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.p = config.hidden_dropout_prob

    def forward(self, input_ids, token_type_ids=None):
        pos = torch.arange(input_ids.shape[1], device=input_ids.device).unsqueeze(0).expand_as(input_ids)
        if token_type_ids is None:
            token_type_ids = torch.zeros_like(input_ids)
        e = embedding_sum([input_ids, pos, token_type_ids],
                          [self.word_embeddings.weight, self.position_embeddings.weight,
                           self.token_type_embeddings.weight])
        return dropout(self.LayerNorm(e), self.p, self.training)


class BertSelfAttention(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.num_attention_heads = config.num_attention_heads
        self.attention_head_size = config.hidden_size // config.num_attention_heads
        self.all_head_size = config.hidden_size
        self.p_attn = float(config.attention_probs_dropout_prob or 0.0)
        self.qkv = Linear(config.hidden_size, 3 * config.hidden_size)
        self.qkv.fused_parts = 3
        expose_fused_projection(self, "qkv", ("query", "key", "value"))

    def forward(self, x, key_bias=None, fork: bool = False):
        """``fork=True`` also returns ``x`` for the residual connection (its gradient is then summed in
        the QKV data-gradient GEMM, see ``ops.linear.linear_fork``)."""
        x_res = x
        if fork and type(self.qkv) is Linear:
            qkv, x_res = linear_fork(x, self.qkv.weight, self.qkv.bias)
        else:
            qkv = self.qkv(x)
        B, L = qkv.shape[0], qkv.shape[1]     # the projection may have gathered the sequence
        local = qkv.shape[-1] // 3
        heads = local // self.attention_head_size
        qkv = qkv.view(B, L, 3 * heads, self.attention_head_size)
        ctx = flash_attention_packed(qkv, heads, heads, key_bias=key_bias, causal=False,
                                     dropout_p=self.p_attn if self.training else 0.0)
        ctx = ctx.reshape(B, L, local)
        return (ctx, x_res) if fork else ctx


class BertSelfOutput(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.dense = Linear(config.hidden_size, config.hidden_size)
        self.LayerNorm = LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.p = config.hidden_dropout_prob

    def forward(self, hidden_states, input_tensor):
        return self.LayerNorm(self.dense(hidden_states), residual=input_tensor, p_drop=self.p)


class BertAttention(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.self = BertSelfAttention(config)
        self.output = BertSelfOutput(config)

    def forward(self, x, key_bias=None):
        ctx, x_res = self.self(x, key_bias, fork=True)
        return self.output(ctx, x_res)


class BertIntermediate(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.dense = Linear(config.hidden_size, config.intermediate_size)
        self.act = G.ACT_BY_NAME[config.hidden_act]


class BertOutput(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.dense = Linear(config.intermediate_size, config.hidden_size)
        self.LayerNorm = LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.p = config.hidden_dropout_prob


class BertLayer(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.attention = BertAttention(config)
        self.intermediate = BertIntermediate(config)
        self.output = BertOutput(config)

    def forward(self, hidden_states, key_bias=None):
        a = self.attention(hidden_states, key_bias)
        fc1, fc2 = self.intermediate.dense, self.output.dense
        if type(fc1) is Linear and type(fc2) is Linear:
            ff, a = k_mlp_fork(a, fc1.weight, fc1.bias, fc2.weight, fc2.bias, self.intermediate.act)
        else:
            ff = fc2(G.act_forward(self.intermediate.act, fc1(a)))
        return self.output.LayerNorm(ff, residual=a, p_drop=self.output.p)


class BertEncoder(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.layer = nn.ModuleList([BertLayer(config) for _ in range(config.num_hidden_layers)])

    def forward(self, h, key_bias=None):
        for l in self.layer:
            h = l(h, key_bias)
        return h


class BertModel(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.config = config
        self.embeddings = BertEmbeddings(config)
        self.encoder = BertEncoder(config)

    def forward(self, input_ids, token_type_ids=None, attention_mask=None):
        key_bias = None
        if attention_mask is not None:
            key_bias = (1.0 - attention_mask.float()) * -30000.0
        return self.encoder(self.embeddings(input_ids, token_type_ids), key_bias)


class BertPredictionHeadTransform(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.dense = Linear(config.hidden_size, config.hidden_size)
        self.act = G.ACT_BY_NAME[config.hidden_act]
        self.LayerNorm = LayerNorm(config.hidden_size, eps=config.layer_norm_eps)

    def forward(self, x):
        return self.LayerNorm(G.act_forward(self.act, self.dense(x)))


class BertLMPredictionHead(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.transform = BertPredictionHeadTransform(config)
        self.decoder = Linear(config.hidden_size, config.vocab_size, bias=True)
        self.bias = self.decoder.bias

    def forward(self, x):
        return self.decoder(self.transform(x))


class BertOnlyMLMHead(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.predictions = BertLMPredictionHead(config)

    def forward(self, x):
        return self.predictions(x)


class BertForMaskedLM(nn.Module):
    """``forward(input_ids, token_type_ids, attention_mask, labels)`` -> logits or ``(loss, logits)``;
    ``labels`` are -100 outside the masked positions."""

    def __init__(self, config: BertConfig):
        super().__init__()
        self.config = config
        self.bert = BertModel(config)
        self.cls = BertOnlyMLMHead(config)
        self.apply(self._init_weights)
        if config.tie_word_embeddings:
            self.cls.predictions.decoder.weight = self.bert.embeddings.word_embeddings.weight

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
        return self.bert.embeddings.word_embeddings

    def get_output_embeddings(self):
        return self.cls.predictions.decoder

    def forward(self, input_ids, token_type_ids=None, attention_mask=None, labels=None):
        h = self.bert(input_ids, token_type_ids, attention_mask)
        logits = self.cls(h)
        if labels is None:
            return logits
        return softmax_cross_entropy(logits, labels), logits


def bert_config(name: str = "bert-base", **overrides) -> BertConfig:
    presets = {
        "bert-base": dict(hidden_size=768, num_hidden_layers=12, num_attention_heads=12, intermediate_size=3072),
        "bert-large": dict(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096),
        "bert-tiny": dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=512,
                          max_position_embeddings=128),
    }
    cfg = dict(presets[name])
    cfg.update(overrides)
    return BertConfig(**cfg)
