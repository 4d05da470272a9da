"""Symbolic tracing front-ends.

``trace_model`` turns an ``nn.Module`` into a ``torch.fx.GraphModule`` whose ``call_module``
nodes are the coarse blocks the sharder works with:

* ``method='fx'``: a ``torch.fx.Tracer`` subclass with a leaf-module policy (every ``torch.nn``
  builtin, every class the user lists, and the framework's own block classes are leaves).  This
  replaces the Hugging Face tracer the reference depends on
  (Merak/core/fx/tracer/_symbolic_trace.py:32-127), which no longer exists in transformers 5.x.
* ``method='dynamo'``: ``torch.export`` (Merak/core/fx/tracer/_dynamo_trace.py:22-60) followed by
  folding the flat ATen graph back into calls of the model's leaf modules
  (``fx/export_trace.py``); this is also what ``'fx'`` falls back to for models symbolic tracing
  rejects, which with transformers 5.x is every Hugging Face model.

``make_dummy_inputs`` builds small CPU inputs from a model config for tracing
(Merak/core/fx/tracer/utils.py:62-191).
"""
from __future__ import annotations

import inspect
from typing import Dict, Iterable, Optional, Sequence, Tuple, Type

import torch
import torch.fx as fx
import torch.nn as nn


def framework_leaf_classes() -> Tuple[type, ...]:
    from ..models import bert, gpt2, llama
    from ..ops import modules as km
    from ..parallel import layers as pl
    from ..parallel import tp_transform as tt
    classes = [gpt2.GPT2Block, bert.BertLayer, bert.BertEmbeddings, bert.BertOnlyMLMHead,
               llama.LlamaDecoderLayer, km.Linear, km.LayerNorm, km.RMSNorm, km.Embedding, km.Dropout,
               pl.ColumnParallelLinear, pl.RowParallelLinear, pl.VocabParallelEmbedding, pl.ColParallelConv2d,
               tt.ColPara, tt.RowPara, tt._SeqScatter, tt._GatherThenLinear]
    try:
        from ..parallel import tp_overlap
        classes += [tp_overlap.PipedRowParallelLinear, tp_overlap.PipedColumnParallelLinear,
                    tp_overlap.ChunkPipelinedBlock]
    except Exception:
        pass
    try:
        from ..parallel import ulysses
        classes += [ulysses.SplitSequence, ulysses.GatherSequence]
    except Exception:
        pass
    try:
        from ..models import moe
        classes.append(moe.MoEDecoderLayer)
    except Exception:
        pass
    return tuple(classes)


class MerakTracer(fx.Tracer):
    """fx tracer whose leaves are whole blocks (Merak/core/fx/tracer/tracers.py:20-35)."""

    def __init__(self, leaf_modules: Iterable[type] = (), leaf_names: Iterable[str] = ()):
        super().__init__()
        self.leaf_classes = tuple(leaf_modules) + framework_leaf_classes()
        self.leaf_names = set(leaf_names)

    def is_leaf_module(self, m: nn.Module, qualname: str) -> bool:
        if isinstance(m, self.leaf_classes) or qualname in self.leaf_names:
            return True
        return super().is_leaf_module(m, qualname)


def get_concrete_args(model: nn.Module, input_names: Sequence[str]) -> Dict[str, object]:
    """Defaults for every forward() parameter that is not a traced input."""
    sig = inspect.signature(model.forward)
    out = {}
    for name, p in sig.parameters.items():
        if name in input_names or p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD):
            continue
        out[name] = p.default if p.default is not inspect.Parameter.empty else None
    return out


def fx_trace(model: nn.Module, input_names: Sequence[str], leaf_modules: Iterable[type] = ()) -> fx.GraphModule:
    tracer = MerakTracer(leaf_modules)
    concrete = get_concrete_args(model, input_names)
    if "use_cache" in concrete:
        concrete["use_cache"] = False
    graph = tracer.trace(model, concrete_args=concrete)
    # concrete args leave placeholders (plus an assertion on their value) behind; remove both
    for node in list(graph.nodes):
        if node.op == "placeholder" and node.target not in input_names:
            for user in list(node.users):
                if user.op == "call_function" and "assert" in getattr(user.target, "__name__", ""):
                    graph.erase_node(user)
            if not node.users:
                graph.erase_node(node)
    gm = fx.GraphModule(model, graph, class_name=type(model).__name__)
    return gm


def dynamo_trace(model: nn.Module, dummy_inputs: Dict[str, torch.Tensor],
                 leaf_modules: Iterable[type] = ()) -> fx.GraphModule:
    """``torch.export`` based tracing for models plain fx cannot handle; the flat ATen graph is
    folded back into ``call_module`` nodes on the model's leaf modules (``fx.export_trace``)."""
    from ..parallel import mpu
    from .export_trace import export_trace
    # a symbolic batch size yields integer values in the graph; between pipeline stages only tensors
    # travel, so with more than one stage the batch size of the dummy inputs is baked in
    dynamic = mpu.get_pipe_parallel_world_size() == 1
    return export_trace(model, dummy_inputs, tuple(leaf_modules) + framework_leaf_classes(), dynamic_batch=dynamic)


def trace_model(model: nn.Module, input_names: Sequence[str], method: str = "fx",
                leaf_modules: Iterable[type] = (), dummy_inputs: Optional[Dict[str, torch.Tensor]] = None):
    """``method='fx'`` tries symbolic tracing first and, when the model defeats it (Hugging Face
    models: decorators, mask helpers, data-dependent Python), falls back to the export path if dummy
    inputs are at hand; ``method='dynamo'`` goes to the export path directly."""
    if method == "fx":
        try:
            return fx_trace(model, input_names, leaf_modules)
        except Exception as exc:
            if dummy_inputs is None:
                raise
            from ..printer import log_dist
            log_dist("torch.fx could not trace %s (%s: %s); using torch.export" % (
                type(model).__name__, type(exc).__name__, str(exc).splitlines()[0][:120] if str(exc) else ""), ranks=[0])
            method = "dynamo"
    if method == "dynamo":
        if dummy_inputs is None:
            raise ValueError("trace_method='dynamo' needs dummy inputs")
        dummy = {k: dummy_inputs[k] for k in input_names if k in dummy_inputs} or dict(dummy_inputs)
        return dynamo_trace(model, dummy, leaf_modules)
    raise ValueError("unknown trace method %r" % method)


def make_dummy_inputs(config, input_names: Sequence[str], batch_size: int = 2, seq_length: Optional[int] = None,
                      device="cpu") -> Dict[str, torch.Tensor]:
    """Small random inputs keyed by the names a forward() expects."""
    seq = seq_length or min(int(getattr(config, "max_position_embeddings", 128) or 128), 128)
    vocab = int(getattr(config, "vocab_size", 1000) or 1000)
    out = {}
    for name in input_names:
        if name in ("input_ids", "decoder_input_ids", "labels"):
            out[name] = torch.randint(0, vocab, (batch_size, seq), device=device)
        elif name in ("attention_mask", "decoder_attention_mask"):
            out[name] = torch.ones(batch_size, seq, dtype=torch.long, device=device)
        elif name == "token_type_ids":
            out[name] = torch.zeros(batch_size, seq, dtype=torch.long, device=device)
        elif name == "position_ids":
            out[name] = torch.arange(seq, device=device)[None].expand(batch_size, seq)
        elif name == "pixel_values":
            ch = int(getattr(config, "num_channels", 3))
            size = getattr(config, "image_size", 224)
            size = size if isinstance(size, (tuple, list)) else (size, size)
            out[name] = torch.randn(batch_size, ch, *size, device=device)
        elif name in ("input_features", "input_values"):
            out[name] = torch.randn(batch_size, int(getattr(config, "num_mel_bins", 80)), 3000, device=device)
        else:
            out[name] = torch.randn(batch_size, seq, int(getattr(config, "hidden_size", 64)), device=device)
    return out
