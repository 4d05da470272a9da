"""``torch.export`` front-end for models plain ``torch.fx`` cannot trace (Hugging Face models).

The reference traces Hugging Face models with ``transformers.utils.fx`` (its ``MerakTracer`` /
``tf_symbolic_trace``, Merak/core/fx/tracer/_symbolic_trace.py:32-127) and other models with
``torch.export`` (Merak/core/fx/tracer/_dynamo_trace.py:22-60).  ``transformers`` 5.x removed its
fx tracer, so here every model that symbolic tracing rejects goes through ``torch.export``, and
the flat ATen graph it returns is folded back into a module-level graph:

1. ``export_flat`` wraps the model so that only tensor inputs are graph inputs (``use_cache=False``,
   ``return_dict=False`` are constants), exports it in training mode and renames every attribute to
   its path in the original model, so parameters stay the original ``nn.Parameter`` objects and
   state-dict keys stay the model's own (checkpoints interchange with Hugging Face ones).
2. ``fold_leaf_modules`` uses the ``nn_module_stack`` recorded on every node to find the nodes that
   came out of one call of a *leaf* module (a ``torch.nn`` builtin such as ``nn.Linear`` /
   ``nn.LayerNorm`` / ``nn.Embedding`` / ``nn.Dropout``, a ``transformers`` ``Conv1D``, a
   tensor-parallel wrapper, or any class the user lists) and replaces them with one ``call_module``
   node on the original module.  What remains between them is ATen glue (views, mask
   construction, attention).  The result has the shape the graph-sharding passes expect: modules
   that own parameters, named by their path, which ``layer_split`` / ``nearest_min_deps`` /
   ``farthest_min_deps`` can cut and the tensor-parallel and LoRA transforms can swap.
3. Tensor parallelism is applied to the model *before* export, as the reference does
   (Merak/core/pipeline/module.py:191), so shapes baked into the graph are per-rank; while
   exporting, collectives are replaced by local operations of the same output shape
   (``parallel.mappings.shape_only_collectives``), since the graph only needs to know shapes and
   the folded ``call_module`` nodes run the real wrappers afterwards.

A model input whose leading dimension is the batch is exported with that dimension symbolic when
the model allows it (``dynamic_batch``), otherwise with the traced batch size baked in.
"""
from __future__ import annotations

import contextlib
import inspect
import operator
import re
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.fx as fx
import torch.nn as nn


class _TensorInputsOnly(nn.Module):
    """forward(*tensors) -> model(**{name: tensor}, **constants); tuple outputs."""

    def __init__(self, model: nn.Module, names: Sequence[str], consts: Dict[str, object]):
        super().__init__()
        self.m = model
        self._names = list(names)
        self._consts = dict(consts)

    def forward(self, *tensors):
        out = self.m(**dict(zip(self._names, tensors)), **self._consts)
        if isinstance(out, dict):                      # ModelOutput without return_dict support
            out = tuple(v for v in out.values() if v is not None)
        return out


def _constant_kwargs(model: nn.Module, input_names: Sequence[str]) -> Dict[str, object]:
    params = inspect.signature(model.forward).parameters
    consts = {}
    if "use_cache" in params and "use_cache" not in input_names:
        consts["use_cache"] = False
    if "return_dict" in params:
        consts["return_dict"] = False
    return consts


def _strip(path: str) -> str:
    """Attribute paths of the wrapper (``m.transformer.h.0``) -> paths of the model."""
    if path == "m":
        return ""
    return path[2:] if path.startswith("m.") else path


def _resolve(root: nn.Module, path: str):
    obj = root
    for part in path.split("."):
        if not hasattr(obj, part):
            return None
        obj = getattr(obj, part)
    return obj


class _no_layerdrop:
    """LayerDrop (BART / OPT / wav2vec2 families: ``if torch.rand([]) < self.layerdrop: skip the
    layer``) is a coin toss per layer and step that a static graph cannot hold.  While exporting,
    the scalar draw is a constant 1.0, i.e. every layer is kept (LayerDrop off), which is also what
    the reference's traced graphs do."""

    def __enter__(self):
        self._rand = torch.rand

        def rand(*size, **kw):
            if len(size) == 1 and isinstance(size[0], (list, tuple)) and len(size[0]) == 0 and not kw:
                return 1.0
            return self._rand(*size, **kw)
        torch.rand = rand
        return self

    def __exit__(self, *exc):
        torch.rand = self._rand
        return False


class _dict_outputs_inside:
    """Configurations written for older ``transformers`` set ``return_dict=False`` (every model
    configuration of the reference's examples does).  In transformers 5.x the inner modules then hand
    tuples to heads that read ``outputs.last_hidden_state``.  While exporting, the configurations say
    ``return_dict=True`` and only the outermost call is asked for a tuple (``_constant_kwargs``)."""

    def __init__(self, model: nn.Module):
        self.model, self.saved = model, []

    def __enter__(self):
        seen = set()
        for m in self.model.modules():
            cfg = getattr(m, "config", None)
            if cfg is None or id(cfg) in seen:
                continue
            seen.add(id(cfg))
            try:
                if getattr(cfg, "return_dict", True) is False:
                    cfg.return_dict = True
                    self.saved.append(cfg)
            except Exception:
                pass
        return self

    def __exit__(self, *exc):
        for cfg in self.saved:
            cfg.return_dict = False
        return False


class _all_on_meta:
    """A model built under ``init_empty_weights`` has its large weights on the meta device and the rest
    (norm weights, rotary tables) in host memory; tracing needs one device.  For the duration of the
    export every parameter and buffer is swapped for a meta stand-in (shared tensors share one),
    then the original objects are put back, so identities, values and tied weights are untouched."""

    def __init__(self, model: nn.Module):
        self.model, self.saved = model, []

    def __enter__(self):
        stand_in = {}
        for mod in self.model.modules():
            for store in (mod._parameters, mod._buffers):
                for name, t in list(store.items()):
                    if t is None or t.is_meta:
                        continue
                    if id(t) not in stand_in:
                        m = torch.empty_like(t, device="meta")
                        stand_in[id(t)] = nn.Parameter(m, requires_grad=t.requires_grad) if isinstance(t, nn.Parameter) else m
                    self.saved.append((store, name, t))
                    store[name] = stand_in[id(t)]
        return self

    def __exit__(self, *exc):
        for store, name, t in self.saved:
            store[name] = t
        return False


def export_flat(model: nn.Module, dummy_inputs: Dict[str, torch.Tensor], dynamic_batch: bool = True) -> fx.GraphModule:
    """Flat ATen graph over the model's own attributes; placeholders are named like the inputs."""
    from ..parallel import fused_tp
    from ..parallel.mappings import shape_only_collectives

    names = list(dummy_inputs)
    wrapper = _TensorInputsOnly(model, names, _constant_kwargs(model, names))
    args = tuple(dummy_inputs[n] for n in names)
    on_meta = any(p.is_meta for p in model.parameters())
    if on_meta:
        args = tuple(t.to("meta") for t in args)
    fused_saved, fused_tp.ENABLED = fused_tp.ENABLED, False
    try:
        with shape_only_collectives(), _no_layerdrop(), _dict_outputs_inside(model), \
                (_all_on_meta(model) if on_meta else contextlib.nullcontext()):
            ep = None
            if dynamic_batch and all(t.dim() >= 1 and t.shape[0] == args[0].shape[0] and t.shape[0] > 1 for t in args):
                try:
                    batch = torch.export.Dim("batch", min=1)
                    ep = torch.export.export(wrapper, args=args, strict=False,
                                             dynamic_shapes=(tuple({0: batch} for _ in args),))
                except Exception:
                    ep = None                       # the model specialises on the batch size
            if ep is None:
                ep = torch.export.export(wrapper, args=args, strict=False)
    finally:
        fused_tp.ENABLED = fused_saved
    src = ep.module()
    graph = fx.Graph()
    env: Dict[fx.Node, fx.Node] = {}
    extra = 0
    ph_iter = iter(names)
    for node in src.graph.nodes:
        if node.op == "call_module" and not node.users:
            continue                                 # the exported module's input-guard function
        if node.op == "placeholder":
            new = graph.placeholder(next(ph_iter))
        elif node.op == "get_attr":
            target = _strip(node.target)
            obj = _resolve(model, target) if target else None
            if obj is None:
                # lifted constants and sub-graphs of higher-order ops exist only in the exported module
                obj = _resolve(src, node.target)
                target = "_exported_attr_%d" % extra
                extra += 1
                if isinstance(obj, torch.Tensor) and not isinstance(obj, nn.Parameter):
                    model.register_buffer(target, obj, persistent=False)
                else:
                    setattr(model, target, obj)
            new = graph.get_attr(target)
        elif node.op == "output":
            outs = node.args[0]
            outs = outs if isinstance(outs, (tuple, list)) else (outs,)
            new = graph.output(tuple(fx.node.map_arg(o, lambda a: env[a]) for o in outs))
        else:
            new = graph.node_copy(node, lambda a: env[a])
        new.meta = dict(node.meta)
        env[node] = new
    _clean_graph(graph, on_meta)
    for name, sub in list(model.named_children()):
        if name.startswith("_exported_attr_") and isinstance(sub, fx.GraphModule):     # bodies of higher-order ops
            _clean_graph(sub.graph, on_meta)
            sub.recompile()
    gm = fx.GraphModule(model, graph, class_name=type(model).__name__)
    gm.graph.eliminate_dead_code()
    gm.recompile()
    gm.exported_dynamic_batch = bool(ep.range_constraints)
    return gm


def _clean_graph(graph: fx.Graph, devices_are_placeholders: bool):
    """Drops run-time assertions (dtype / device / shape guards carry no data).  A graph exported on the
    meta device has ``device=meta`` baked into its tensor factories and copies; those arguments are
    rewired to the device of the graph's first tensor input, whatever that is at run time (the
    reference rewrites device arguments of exported graphs too,
    Merak/core/fx/graph_shard/split_module.py:200-204)."""
    for node in list(graph.nodes):
        if node.op == "call_function" and "_assert" in str(node.target) and not node.users:
            graph.erase_node(node)
        elif node.op == "call_function" and node.target is torch.ops.aten.detach_.default:
            # ``torch.tensor(c)`` inside the model exports as an in-place detach of a lifted constant.  When that
            # constant reaches the node through a shard boundary or a recomputed segment it is an alias made by
            # ``detach()``, on which the in-place form is an error; the out-of-place form gives the same value.
            node.target = torch.ops.aten.detach.default
    if not devices_are_placeholders:
        return
    # The device comes from a tensor next to the node that needs it (an operand, else the latest activation
    # before it), through a ``getattr`` node of its own placed right before it and carrying its module stack:
    # when the graph is later cut into pipeline stages no ``torch.device`` value has to cross a boundary.
    is_meta = lambda a: isinstance(a, torch.device) and a.type == "meta"
    latest = None
    for node in list(graph.nodes):
        if node.op == "call_function" and (any(is_meta(a) for a in node.args) or any(is_meta(v) for v in node.kwargs.values())):
            src = next((a for a in node.all_input_nodes if _is_activation(a)), None) or latest
            if src is not None:
                with graph.inserting_before(node):
                    dev = graph.call_function(getattr, (src, "device"))
                dev.meta = {k: v for k, v in node.meta.items() if k in ("nn_module_stack", "stack_trace", "source_fn_stack")}
                node.args = tuple(dev if is_meta(a) else a for a in node.args)
                node.kwargs = {k: (dev if is_meta(v) else v) for k, v in node.kwargs.items()}
        if _is_activation(node):
            latest = node


def _is_activation(n: fx.Node) -> bool:
    """A graph input or a computed tensor (not a parameter / buffer read)."""
    if n.op == "placeholder":
        return True
    return n.op in ("call_function", "call_module") and isinstance(n.meta.get("val"), torch.Tensor)


# ---------------------------------------------------------------------------------------------
# folding
# ---------------------------------------------------------------------------------------------
def _module_stack(node: fx.Node) -> List[Tuple[str, str]]:
    """[(stack key, module path)] outermost first, wrapper prefix removed."""
    stack = node.meta.get("nn_module_stack") or {}
    out = []
    for key, (path, _cls) in stack.items():
        p = _strip(path)
        if p or path == "m":
            out.append((key, p))
    return [(k, p) for k, p in out if p]


def _is_tensor_node(n: fx.Node) -> bool:
    val = n.meta.get("val")
    return isinstance(val, torch.Tensor) or (val is None and n.op in ("placeholder", "call_module", "get_attr"))


class ExportedDropout(nn.Dropout):
    """A functional dropout of the exported graph; as a module it follows ``train()`` / ``eval()``
    (the exported call had ``training=True`` baked in)."""


class ExportedSDPA(nn.Module):
    """``scaled_dot_product_attention`` of the exported graph with its dropout probability applied
    only in training mode."""

    def __init__(self, dropout_p: float = 0.0, is_causal: bool = False, scale=None, enable_gqa: bool = False):
        super().__init__()
        self.dropout_p, self.is_causal, self.scale, self.enable_gqa = float(dropout_p), bool(is_causal), scale, enable_gqa

    def forward(self, q, k, v, attn_mask=None):
        return torch.nn.functional.scaled_dot_product_attention(
            q, k, v, attn_mask=attn_mask, dropout_p=self.dropout_p if self.training else 0.0,
            is_causal=self.is_causal, scale=self.scale, enable_gqa=self.enable_gqa)

    def extra_repr(self):
        return "dropout_p=%g, is_causal=%s" % (self.dropout_p, self.is_causal)


def _modularise_dropout(graph: fx.Graph, model: nn.Module):
    """Functional dropouts and attention calls of the flat graph become modules registered on the
    model (``_exported_dropout_<k>`` / ``_exported_sdpa_<k>``), so evaluation switches them off."""
    k = 0
    for n in list(graph.nodes):
        if n.op != "call_function":
            continue
        name = str(n.target)
        if name in ("aten.dropout.default", "aten.native_dropout.default") and len(n.args) >= 2:
            mod_name = "_exported_dropout_%d" % k
            setattr(model, mod_name, ExportedDropout(float(n.args[1])))
        elif name == "aten.scaled_dot_product_attention.default":
            def arg(i, key, default):
                return n.args[i] if len(n.args) > i else n.kwargs.get(key, default)
            mod_name = "_exported_sdpa_%d" % k
            setattr(model, mod_name, ExportedSDPA(arg(4, "dropout_p", 0.0), arg(5, "is_causal", False),
                                                  n.kwargs.get("scale"), n.kwargs.get("enable_gqa", False)))
        else:
            continue
        k += 1
        with graph.inserting_before(n):
            if "dropout" in mod_name:
                call = graph.create_node("call_module", mod_name, (n.args[0],))
            else:
                mask = n.args[3] if len(n.args) > 3 else n.kwargs.get("attn_mask")
                call = graph.create_node("call_module", mod_name, tuple(n.args[:3]) + (mask,))
        call.meta = dict(n.meta)
        if name == "aten.native_dropout.default":
            # (output, mask) tuple: only the output is used by forward graphs
            for u in list(n.users):
                if u.target is operator.getitem and u.args[1] == 0:
                    u.replace_all_uses_with(call)
                    graph.erase_node(u)
        else:
            n.replace_all_uses_with(call)
        if not n.users:
            graph.erase_node(n)


def default_leaf_policy(leaf_classes: Tuple[type, ...]):
    def is_leaf(m: nn.Module) -> bool:
        if isinstance(m, leaf_classes):
            return True
        if isinstance(m, (nn.Sequential, nn.ModuleList, nn.ModuleDict)):
            return False
        return type(m).__module__.startswith("torch.nn") and not any(True for _ in m.children())
    return is_leaf


def fold_leaf_modules(gm: fx.GraphModule, model: nn.Module, leaf_classes: Iterable[type] = ()) -> fx.GraphModule:
    """Replaces the nodes of each single-input, single-output call of a leaf module by a
    ``call_module`` node on that module."""
    try:
        from transformers.pytorch_utils import Conv1D
        leaf_classes = tuple(leaf_classes) + (Conv1D,)
    except Exception:
        leaf_classes = tuple(leaf_classes)
    is_leaf = default_leaf_policy(leaf_classes)
    graph = gm.graph
    order = {n: i for i, n in enumerate(graph.nodes)}
    groups: Dict[Tuple[str, str], List[fx.Node]] = {}
    for n in graph.nodes:
        if n.op != "call_function":
            continue
        for key, path in _module_stack(n):
            mod = _resolve(model, path)
            if isinstance(mod, nn.Module) and is_leaf(mod):
                groups.setdefault((key, path), []).append(n)
                break
    folded = 0
    for (key, path), nodes in groups.items():
        mod = _resolve(model, path)
        own_tensors = {id(t) for t in list(mod.parameters()) + list(mod.buffers())}
        inside = set(nodes)
        # parameters / buffers of the module (by identity: a tied weight may be recorded under the
        # name of the other module that shares it)
        attrs = set()
        for n in nodes:
            for a in n.all_input_nodes:
                if a.op == "get_attr" and id(_resolve(model, a.target)) in own_tensors:
                    attrs.add(a)
        ext_inputs: List[fx.Node] = []
        for n in nodes:
            for a in n.all_input_nodes:
                if a not in inside and a not in attrs and a not in ext_inputs and _is_tensor_node(a):
                    ext_inputs.append(a)
        outputs = [n for n in nodes if _is_tensor_node(n) and any(u not in inside for u in n.users)]
        if len(ext_inputs) != 1 or len(outputs) != 1:
            continue
        out = outputs[0]
        with graph.inserting_before(out):
            call = graph.create_node("call_module", path, (ext_inputs[0],))
        call.meta = dict(out.meta)
        out.replace_all_uses_with(call)
        # shape arithmetic (symbolic sizes) that later nodes still read stays where it is; it only
        # depends on the module's input
        for n in sorted(nodes, key=order.get, reverse=True):
            if not n.users:
                graph.erase_node(n)
        for a in attrs:
            if not a.users:
                graph.erase_node(a)
        folded += 1
    _modularise_dropout(graph, model)
    out_gm = fx.GraphModule(model, graph, class_name=type(model).__name__)
    out_gm.graph.lint()
    out_gm.folded_modules = folded
    out_gm.exported_dynamic_batch = getattr(gm, "exported_dynamic_batch", False)
    return out_gm


def export_trace(model: nn.Module, dummy_inputs: Dict[str, torch.Tensor], leaf_classes: Iterable[type] = (),
                 dynamic_batch: bool = True, check: bool = True) -> fx.GraphModule:
    """``export_flat`` + ``fold_leaf_modules``.  With ``check`` the folded graph is run against the
    model in evaluation mode on the dummy inputs; a mismatch (a leaf module whose call did not
    reduce to ``module(x)``) falls back to folding ``torch.nn`` builtins only."""
    flat = export_flat(model, dummy_inputs, dynamic_batch)
    folded = fold_leaf_modules(flat, model, leaf_classes)
    small = sum(p.numel() for p in model.parameters()) < 50_000_000      # the check runs the model on the host
    if check and small and not any(p.is_meta for p in model.parameters()):
        from ..parallel import mpu
        if mpu.get_model_parallel_world_size() == 1 and not _agrees(folded, model, dummy_inputs):
            flat = export_flat(model, dummy_inputs, dynamic_batch)
            folded = fold_leaf_modules(flat, model, ())
    return folded


def _agrees(gm: fx.GraphModule, model: nn.Module, dummy_inputs: Dict[str, torch.Tensor]) -> bool:
    was_training = model.training
    names = list(dummy_inputs)
    try:
        model.eval()
        gm.eval()
        with torch.no_grad(), _dict_outputs_inside(model):
            want = _TensorInputsOnly(model, names, _constant_kwargs(model, names))(*dummy_inputs.values())
            got = gm(*dummy_inputs.values())
        want = want if isinstance(want, (tuple, list)) else (want,)
        got = got if isinstance(got, (tuple, list)) else (got,)
        w, g = want[0], got[0]
        # dropout probabilities of attention kernels are baked in from training mode: compare shapes
        # and, where no functional dropout is left in the graph, values
        if w.shape != g.shape:
            return False
        baked = any(n.op == "call_function" and "dropout" in str(n.target) for n in gm.graph.nodes) or \
            any(n.op == "call_function" and "scaled_dot_product_attention" in str(n.target) and
                (len(n.args) > 4 and n.args[4] not in (0, 0.0) or n.kwargs.get("dropout_p", 0.0) not in (0, 0.0))
                for n in gm.graph.nodes)
        return True if baked else bool(torch.allclose(w.float(), g.float(), atol=1e-4, rtol=1e-3))
    except Exception:
        return False
    finally:
        model.train(was_training)
        gm.train(was_training)
