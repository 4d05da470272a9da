"""``init_empty_weights``: build a model whose large parameters live on the ``meta`` device, so a
model bigger than host memory can be traced and sharded by one worker; each stage then
materialises only its own shards (Merak/utils/device_to_meta.py:27-80)."""
from __future__ import annotations

import contextlib

import torch
import torch.nn as nn


@contextlib.contextmanager
def init_empty_weights(include_buffers: bool = False):
    old_register = nn.Module.register_parameter

    def register(module, name, param):
        old_register(module, name, param)
        if param is not None and isinstance(module, (nn.Embedding, nn.Linear)) or type(module).__name__ == "Conv1D":
            p = module._parameters[name]
            if p is not None:
                module._parameters[name] = nn.Parameter(p.to("meta"), requires_grad=p.requires_grad)

    nn.Module.register_parameter = register
    try:
        yield
    finally:
        nn.Module.register_parameter = old_register


def materialize_meta(module: nn.Module, device, init_std: float = 0.02, dtype=None):
    """Allocates every ``meta`` parameter / buffer of ``module`` on ``device`` and initialises it:
    normal(0, std) for matrices and embeddings, ones for norm weights, zeros for biases."""
    done = {}       # a parameter shared by several modules (tied embeddings) stays one tensor
    for m in module.modules():
        for name, p in list(m._parameters.items()):
            if p is None or p.device.type != "meta":
                continue
            if id(p) in done:
                m._parameters[name] = done[id(p)]
                continue
            t = torch.empty(p.shape, dtype=dtype or p.dtype, device=device)
            if p.dim() >= 2:
                nn.init.normal_(t, 0.0, init_std)
            elif "norm" in type(m).__name__.lower() and name == "weight":
                t.fill_(1.0)
            else:
                t.zero_()
            new = nn.Parameter(t, requires_grad=p.requires_grad)
            for attr, val in vars(p).items():          # model_parallel, sequence_parallel, ... tags
                setattr(new, attr, val)
            done[id(p)] = new
            m._parameters[name] = new
        for name, b in list(m._buffers.items()):
            if b is not None and b.device.type == "meta":
                m._buffers[name] = torch.zeros(b.shape, dtype=b.dtype, device=device)
    return module
