"""``convert_to_sequential``: model -> traced graph -> list of shard modules
(Merak/core/fx/convert.py:45-123).  Optionally caches the sharded result on disk
(``cache_sharding`` / ``cache_name``)."""
from __future__ import annotations

import os
from typing import Dict, Iterable, List, Optional, Sequence

import torch
import torch.nn as nn

from .shard import shard_model
from .tracer import trace_model


def default_input_names(model: nn.Module) -> List[str]:
    import inspect
    names = []
    for name, p in inspect.signature(model.forward).parameters.items():
        if p.default is inspect.Parameter.empty and p.kind not in (p.VAR_POSITIONAL, p.VAR_KEYWORD):
            names.append(name)
    return names or ["input_ids"]


def convert_to_sequential(model: nn.Module, args, dummy_inputs: Optional[Dict[str, torch.Tensor]] = None,
                          extra_leaf_modules: Iterable[type] = ()):
    """Returns ``(model, shards, input_to_shard)``; ``shards[0].dummy_inputs`` keeps the inputs used."""
    input_names: Sequence[str] = args.input_names or (list(dummy_inputs) if dummy_inputs else default_input_names(model))
    cache = None
    if getattr(args, "cache_sharding", False):
        cache = os.path.join(args.output_dir, (args.cache_name or type(model).__name__) + "_shards.pt")
        if os.path.exists(cache):
            shards, input_to_shard = torch.load(cache, weights_only=False)
            return model, shards, input_to_shard
    gm = trace_model(model, input_names, args.trace_method, extra_leaf_modules, dummy_inputs)
    model_type = getattr(getattr(model, "config", None), "model_type", None)
    shards, input_to_shard = shard_model(gm, args.split_method, args.shard_count, model_type,
                                         args.custom_split_points)
    shards[0].dummy_inputs = dummy_inputs
    # an exported graph that could not keep the batch size symbolic (or was exported for several pipeline
    # stages, between which only tensors travel) accepts only the batch size of its dummy inputs
    static = getattr(gm, "exported_dynamic_batch", True) is False and bool(dummy_inputs)
    shards[0].static_batch_size = int(next(iter(dummy_inputs.values())).shape[0]) if static else None
    if cache is not None:
        os.makedirs(os.path.dirname(cache), exist_ok=True)
        torch.save((shards, input_to_shard), cache)
    return model, shards, input_to_shard
