"""LoRA adapter layers (Merak/core/finetuning/lora/layer.py:119-712): ``Linear``, ``Embedding`` and
``Conv2d`` wrappers holding named adapters (``lora_A`` / ``lora_B`` per adapter), with
merge / unmerge / get_delta_weight.  The low-rank products run on the same GEMM op as the base
layer; the base weight stays frozen."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.linear import linear as k_linear


class LoraLayer:
    """Mixin state shared by all adapter-carrying layers."""

    def _init_lora_state(self):
        self.r: Dict[str, int] = {}
        self.lora_alpha: Dict[str, int] = {}
        self.scaling: Dict[str, float] = {}
        self.lora_dropout = nn.ModuleDict()
        self.lora_A = nn.ModuleDict()
        self.lora_B = nn.ModuleDict()
        self.lora_embedding_A = nn.ParameterDict()
        self.lora_embedding_B = nn.ParameterDict()
        self.merged_adapters = []
        self.active_adapter = "default"
        self.disable_adapters = False

    @property
    def merged(self) -> bool:
        return bool(self.merged_adapters)

    def set_adapter(self, name: str):
        self.active_adapter = name

    def scale_layer(self, factor: float):
        for k in self.scaling:
            self.scaling[k] *= factor


class Linear(nn.Module, LoraLayer):
    def __init__(self, base: nn.Linear, adapter_name: str = "default", r: int = 8, lora_alpha: int = 8,
                 lora_dropout: float = 0.0, fan_in_fan_out: bool = False, init_lora_weights: bool = True):
        super().__init__()
        self._init_lora_state()
        self.base_layer = base
        self.in_features, self.out_features = base.in_features, base.out_features
        self.fan_in_fan_out = fan_in_fan_out
        for p in base.parameters():
            p.requires_grad = False
        self.update_layer(adapter_name, r, lora_alpha, lora_dropout, init_lora_weights)
        self.active_adapter = adapter_name

    @property
    def weight(self):
        return self.base_layer.weight

    @property
    def bias(self):
        return self.base_layer.bias

    def update_layer(self, name, r, lora_alpha, lora_dropout, init_lora_weights=True):
        if r <= 0:
            raise ValueError("r must be positive")
        w = self.base_layer.weight
        self.r[name], self.lora_alpha[name] = r, lora_alpha
        self.lora_dropout[name] = nn.Dropout(lora_dropout) if lora_dropout > 0 else nn.Identity()
        self.lora_A[name] = nn.Linear(self.in_features, r, bias=False, device=w.device, dtype=w.dtype)
        self.lora_B[name] = nn.Linear(r, self.out_features, bias=False, device=w.device, dtype=w.dtype)
        self.scaling[name] = lora_alpha / r
        if init_lora_weights:
            nn.init.kaiming_uniform_(self.lora_A[name].weight, a=math.sqrt(5))
            nn.init.zeros_(self.lora_B[name].weight)

    def get_delta_weight(self, name: str) -> torch.Tensor:
        d = self.lora_B[name].weight.float() @ self.lora_A[name].weight.float() * self.scaling[name]
        return (d.t() if self.fan_in_fan_out else d).to(self.base_layer.weight.dtype)

    def merge(self):
        for name in self.lora_A:
            if name not in self.merged_adapters:
                self.base_layer.weight.data += self.get_delta_weight(name)
                self.merged_adapters.append(name)

    def unmerge(self):
        while self.merged_adapters:
            name = self.merged_adapters.pop()
            self.base_layer.weight.data -= self.get_delta_weight(name)

    def forward(self, x, residual=None):
        try:
            y = self.base_layer(x, residual) if residual is not None else self.base_layer(x)
        except TypeError:
            y = self.base_layer(x)
            y = y if residual is None else y + residual
        if self.disable_adapters or self.merged:
            return y
        name = self.active_adapter
        if name in self.lora_A:
            a = k_linear(self.lora_dropout[name](x), self.lora_A[name].weight)
            y = y + k_linear(a, self.lora_B[name].weight) * self.scaling[name]
        return y


class Embedding(nn.Module, LoraLayer):
    def __init__(self, base: nn.Embedding, adapter_name: str = "default", r: int = 8, lora_alpha: int = 8,
                 lora_dropout: float = 0.0, init_lora_weights: bool = True):
        super().__init__()
        self._init_lora_state()
        self.base_layer = base
        for p in base.parameters():
            p.requires_grad = False
        w = base.weight
        self.r[adapter_name], self.lora_alpha[adapter_name] = r, lora_alpha
        self.scaling[adapter_name] = lora_alpha / r
        self.lora_embedding_A[adapter_name] = nn.Parameter(torch.zeros(r, base.num_embeddings, device=w.device, dtype=w.dtype))
        self.lora_embedding_B[adapter_name] = nn.Parameter(torch.randn(base.embedding_dim, r, device=w.device, dtype=w.dtype))
        self.active_adapter = adapter_name

    @property
    def weight(self):
        return self.base_layer.weight

    def get_delta_weight(self, name):
        return (self.lora_embedding_B[name].float() @ self.lora_embedding_A[name].float()).t().to(
            self.base_layer.weight.dtype) * self.scaling[name]

    def merge(self):
        for name in self.lora_embedding_A:
            if name not in self.merged_adapters:
                self.base_layer.weight.data += self.get_delta_weight(name)
                self.merged_adapters.append(name)

    def unmerge(self):
        while self.merged_adapters:
            self.base_layer.weight.data -= self.get_delta_weight(self.merged_adapters.pop())

    def forward(self, ids):
        y = self.base_layer(ids)
        if self.disable_adapters or self.merged:
            return y
        name = self.active_adapter
        if name in self.lora_embedding_A:
            after_a = F.embedding(ids, self.lora_embedding_A[name].t())
            y = y + (after_a @ self.lora_embedding_B[name].t()) * self.scaling[name]
        return y


class Conv2d(nn.Module, LoraLayer):
    def __init__(self, base: nn.Conv2d, adapter_name: str = "default", r: int = 8, lora_alpha: int = 8,
                 lora_dropout: float = 0.0, init_lora_weights: bool = True):
        super().__init__()
        self._init_lora_state()
        self.base_layer = base
        for p in base.parameters():
            p.requires_grad = False
        w = base.weight
        self.r[adapter_name], self.lora_alpha[adapter_name] = r, lora_alpha
        self.scaling[adapter_name] = lora_alpha / r
        self.lora_dropout[adapter_name] = nn.Dropout(lora_dropout) if lora_dropout > 0 else nn.Identity()
        self.lora_A[adapter_name] = nn.Conv2d(base.in_channels, r, base.kernel_size, base.stride, base.padding,
                                              bias=False, device=w.device, dtype=w.dtype)
        self.lora_B[adapter_name] = nn.Conv2d(r, base.out_channels, 1, 1, bias=False, device=w.device, dtype=w.dtype)
        if init_lora_weights:
            nn.init.kaiming_uniform_(self.lora_A[adapter_name].weight, a=math.sqrt(5))
            nn.init.zeros_(self.lora_B[adapter_name].weight)
        self.active_adapter = adapter_name

    def get_delta_weight(self, name):
        a, b = self.lora_A[name].weight, self.lora_B[name].weight
        if a.shape[2:] == (1, 1):
            d = (b.squeeze(3).squeeze(2) @ a.squeeze(3).squeeze(2)).unsqueeze(2).unsqueeze(3)
        else:
            d = F.conv2d(a.permute(1, 0, 2, 3), b).permute(1, 0, 2, 3)
        return d * self.scaling[name]

    def merge(self):
        for name in self.lora_A:
            if name not in self.merged_adapters:
                self.base_layer.weight.data += self.get_delta_weight(name)
                self.merged_adapters.append(name)

    def unmerge(self):
        while self.merged_adapters:
            self.base_layer.weight.data -= self.get_delta_weight(self.merged_adapters.pop())

    def forward(self, x):
        y = self.base_layer(x)
        if self.disable_adapters or self.merged:
            return y
        name = self.active_adapter
        if name in self.lora_A:
            y = y + self.lora_B[name](self.lora_A[name](self.lora_dropout[name](x))) * self.scaling[name]
        return y
