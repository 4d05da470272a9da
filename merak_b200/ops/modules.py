"""``nn.Module`` front-ends of the kernels, parameter-compatible with their ``torch.nn``
counterparts (same parameter names and shapes), plus :func:`inject_kernels` which swaps the
``torch.nn`` layers of an arbitrary model for them in place."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import gemm as G
from .elementwise import embedding_sum
from .linear import linear as k_linear
from .norm import fused_norm


class Linear(nn.Linear):
    """``nn.Linear`` whose CUDA bf16 forward/backward run on the tcgen05 GEMM."""

    def forward(self, x, residual: Optional[torch.Tensor] = None):
        return k_linear(x, self.weight, self.bias, residual)


class LayerNorm(nn.LayerNorm):
    def forward(self, x, residual: Optional[torch.Tensor] = None, p_drop: float = 0.0, return_residual=False):
        y, z = fused_norm(x, self.weight, self.bias, residual, self.eps, False, p_drop, self.training)
        return (y, z) if return_residual else y


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.variance_epsilon = eps
        self.eps = eps

    def forward(self, x, residual: Optional[torch.Tensor] = None, return_residual=False):
        y, z = fused_norm(x, self.weight, None, residual, self.eps, True, 0.0, self.training)
        return (y, z) if return_residual else y

    def extra_repr(self):
        return "%d, eps=%g" % (self.weight.shape[0], self.eps)


class Embedding(nn.Embedding):
    def forward(self, ids):
        if self.padding_idx is not None or self.max_norm is not None:
            return super().forward(ids)
        return embedding_sum([ids], [self.weight])


class Dropout(nn.Dropout):
    """Dropout whose mask comes from the framework's counter-based generator on CUDA."""

    def forward(self, x):
        from .elementwise import dropout
        return dropout(x, self.p, self.training)


def inject_kernels(module: nn.Module) -> nn.Module:
    """Re-classes ``nn.Linear`` / ``nn.LayerNorm`` / ``nn.Embedding`` instances (exact types only)
    to the kernel-backed subclasses above.  Parameters are untouched, so state dicts, optimizers
    and tied weights keep working."""
    for m in module.modules():
        if type(m) is nn.Linear:
            m.__class__ = Linear
        elif type(m) is nn.LayerNorm and len(m.normalized_shape) == 1 and m.elementwise_affine:
            m.__class__ = LayerNorm
        elif type(m) is nn.Embedding:
            m.__class__ = Embedding
        elif type(m) is nn.Dropout:
            m.__class__ = Dropout
    return module


def expose_fused_projection(owner: nn.Module, fused: str, names, sizes=None, has_bias: bool = True):
    """Makes ``owner.<fused>`` (one Linear holding several projections stacked on dim 0) appear in
    state dicts as separate entries ``<name>.weight`` / ``<name>.bias`` - the layout of models that
    keep the projections as individual layers - and accepts either form when loading."""

    def split_sizes(total):
        if sizes is not None:
            full = sum(sizes)
            return [s * total // full for s in sizes]
        return [total // len(names)] * len(names)

    def save_hook(module, state_dict, prefix, local_metadata):
        for kind in ("weight", "bias"):
            key = prefix + fused + "." + kind
            if key not in state_dict:
                continue
            t = state_dict.pop(key)
            off = 0
            for n, sz in zip(names, split_sizes(t.shape[0])):
                state_dict[prefix + n + "." + kind] = t[off:off + sz]
                off += sz
        return state_dict

    def load_hook(module, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        for kind in ("weight", "bias"):
            keys = [prefix + n + "." + kind for n in names]
            if all(k in state_dict for k in keys):
                state_dict[prefix + fused + "." + kind] = torch.cat([state_dict.pop(k) for k in keys], 0)

    owner._register_state_dict_hook(save_hook)
    owner.register_load_state_dict_pre_hook(load_hook)
