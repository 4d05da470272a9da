"""Three ways to assign the nodes of a traced graph to a sequence of shards
(``args.split_method``), then ``split_graph`` builds the shard modules.

* ``layer_split``        cut where the module path crosses a known layer boundary
                         (``transformer.h.3`` -> ``transformer.h.4``), from a table of per-model
                         boundary prefixes or ``custom_split_points``
                         (Merak/core/fx/graph_shard/layer_config.py:36-253).
* ``nearest_min_deps``   default.  Every parameter-carrying node opens a shard; parameter-free
                         nodes stay with their producer; adjacent shards are then merged while the
                         merge does not widen the interface (number of tensors crossing in + out)
                         (Merak/core/fx/graph_shard/nearest_deps.py:27-198).
* ``farthest_min_deps``  parameter-balanced: embeddings get their own shard, the rest is cut into
                         ``shard_count`` pieces of roughly equal parameter count, and a node whose
                         inputs come from far-back shards is pulled back toward them when that is
                         still legal (Merak/core/fx/graph_shard/farthest_deps.py:74-227).

All three return ``(shards, input_to_shard)``.
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Sequence

import torch.fx as fx
import torch.nn as nn

from .split import split_graph

# module-path prefixes whose numbered children are the natural layer boundaries, per model family
LAYER_PREFIXES = {
    "gpt2": ["transformer.h"], "bert": ["bert.encoder.layer"], "llama": ["model.layers"],
    "qwen": ["model.layers"], "qwen2": ["model.layers"], "mistral": ["model.layers"],
    "opt": ["model.decoder.layers"], "gptj": ["transformer.h"], "t5": ["encoder.block", "decoder.block"],
    "mt5": ["encoder.block", "decoder.block"], "vit": ["vit.encoder.layer"], "dinov2": ["dinov2.encoder.layer"],
    "deberta": ["deberta.encoder.layer"], "distilbert": ["distilbert.transformer.layer"],
    "mobilebert": ["mobilebert.encoder.layer"], "swin": ["swin.encoder.layers"],
    "resnet": ["resnet.encoder.stages"], "clip": ["text_model.encoder.layers", "vision_model.encoder.layers"],
    "altclip": ["text_model.roberta.encoder.layer", "vision_model.encoder.layers"],
    "wav2vec2": ["wav2vec2.encoder.layers"], "m2m_100": ["model.encoder.layers", "model.decoder.layers"],
    "marian": ["model.encoder.layers", "model.decoder.layers"],
    "pegasus": ["model.encoder.layers", "model.decoder.layers"], "trocr": ["model.decoder.layers"],
    "lxmert": ["lxmert.encoder.layer", "lxmert.encoder.x_layers", "lxmert.encoder.r_layers"],
    "deepseek_v2": ["model.layers"], "moe": ["model.layers"],
}


def _compute_nodes(gm: fx.GraphModule) -> List[fx.Node]:
    return [n for n in gm.graph.nodes if n.op not in ("placeholder", "output")]


def _node_params(gm: fx.GraphModule, n: fx.Node) -> int:
    if n.op == "call_module":
        return sum(p.numel() for p in gm.get_submodule(n.target).parameters())
    if n.op == "get_attr":
        obj = gm
        for part in n.target.split("."):
            obj = getattr(obj, part)
        return obj.numel() if hasattr(obj, "numel") else 0
    return 0


def _legalise(nodes: Sequence[fx.Node], assign: Dict[fx.Node, int]) -> Dict[fx.Node, int]:
    """Makes the assignment non-decreasing along the node order and consistent with data flow."""
    cur = 0
    for n in nodes:
        need = 0
        for a in n.all_input_nodes:
            if a in assign:
                need = max(need, assign[a])
        cur = max(cur, need, assign[n]) if assign[n] >= cur else max(cur, need)
        assign[n] = cur
    # compact indices
    remap = {}
    for n in nodes:
        remap.setdefault(assign[n], len(remap))
    return {n: remap[assign[n]] for n in nodes}


# ---------------------------------------------------------------------------------------------
# layer_split
# ---------------------------------------------------------------------------------------------
def get_split_points(model_type: Optional[str], gm: fx.GraphModule, custom: Optional[Sequence[str]] = None):
    if custom:
        return list(custom)
    prefixes = LAYER_PREFIXES.get((model_type or "").lower())
    points = []
    seen = set()
    for n in gm.graph.nodes:
        if n.op != "call_module":
            continue
        target = n.target
        if prefixes is None:
            m = re.match(r"^(.*?\.\d+)(\.|$)", target)
            key = m.group(1) if m else None
        else:
            key = None
            for p in prefixes:
                m = re.match(r"^(%s\.\d+)(\.|$)" % re.escape(p), target)
                if m:
                    key = m.group(1)
                    break
        if key and key not in seen:
            seen.add(key)
            points.append(key)
    return points


def layer_split(gm: fx.GraphModule, model_type: Optional[str] = None, custom_split_points=None):
    nodes = _compute_nodes(gm)
    points = get_split_points(model_type, gm, custom_split_points)
    assign, shard, next_pt = {}, 0, 0
    for n in nodes:
        if n.op == "call_module" and next_pt < len(points):
            t = n.target
            if t == points[next_pt] or t.startswith(points[next_pt] + "."):
                shard += 1
                next_pt += 1
        assign[n] = shard
    # everything after the last numbered layer (final norm, head) forms the closing shard
    if points:
        last_layer_nodes = [n for n in nodes if n.op == "call_module" and
                            (n.target == points[-1] or n.target.startswith(points[-1] + "."))]
        if last_layer_nodes:
            idx = nodes.index(last_layer_nodes[-1])
            for n in nodes[idx + 1:]:
                if n.op == "call_module" and _node_params(gm, n) > 0:
                    for m in nodes[nodes.index(n):]:
                        assign[m] = shard + 1
                    break
    assign = _legalise(nodes, assign)
    return split_graph(gm, assign, max(assign.values()) + 1 if assign else 1)


# ---------------------------------------------------------------------------------------------
# nearest_min_deps
# ---------------------------------------------------------------------------------------------
def _interface_width(nodes, assign, lo, hi):
    """Number of distinct values crossing into or out of the shard range [lo, hi]."""
    inside = {n for n in nodes if lo <= assign[n] <= hi}
    ins, outs = set(), set()
    for n in inside:
        for a in n.all_input_nodes:
            if a not in inside:
                ins.add(a)
        for u in n.users:
            if u not in inside:
                outs.add(n)
    return len(ins) + len(outs)


def nearest_min_deps(gm: fx.GraphModule, max_shards: Optional[int] = None):
    nodes = _compute_nodes(gm)
    assign, shard = {}, -1
    for n in nodes:
        if _node_params(gm, n) > 0 and n.op == "call_module":
            shard += 1
        elif n.op == "get_attr" and n.users:
            # a free-standing weight/bias lives with its first consumer
            pass
        assign[n] = max(shard, 0)
    assign = _legalise(nodes, assign)
    count = max(assign.values()) + 1 if assign else 1
    # greedy pairwise merging while the interface does not widen
    merged = True
    while merged and count > 1:
        merged = False
        s = 0
        while s < count - 1:
            w_a = _interface_width(nodes, assign, s, s)
            w_b = _interface_width(nodes, assign, s + 1, s + 1)
            w_ab = _interface_width(nodes, assign, s, s + 1)
            small = sum(_node_params(gm, n) for n in nodes if assign[n] in (s, s + 1)) == 0
            if w_ab < min(w_a, w_b) or small:
                for n in nodes:
                    if assign[n] > s:
                        assign[n] -= 1
                count -= 1
                merged = True
            else:
                s += 1
    if max_shards is not None:
        while count > max_shards:
            # merge the lightest adjacent pair
            weights = [sum(_node_params(gm, n) for n in nodes if assign[n] == s) for s in range(count)]
            s = min(range(count - 1), key=lambda i: weights[i] + weights[i + 1])
            for n in nodes:
                if assign[n] > s:
                    assign[n] -= 1
            count -= 1
    return split_graph(gm, assign, count)


# ---------------------------------------------------------------------------------------------
# farthest_min_deps
# ---------------------------------------------------------------------------------------------
def farthest_min_deps(gm: fx.GraphModule, shard_count: int):
    nodes = _compute_nodes(gm)
    params = {n: _node_params(gm, n) for n in nodes}
    is_embed = {n: n.op == "call_module" and isinstance(gm.get_submodule(n.target), nn.Embedding) or
                (n.op == "call_module" and "embed" in type(gm.get_submodule(n.target)).__name__.lower())
                for n in nodes}
    total = sum(params.values())
    emb = sum(p for n, p in params.items() if is_embed[n])
    budget = max(1, (total - emb) // max(1, shard_count))
    assign, shard, used = {}, 0, 0
    for n in nodes:
        if is_embed[n]:
            if used > 0:
                shard += 1
            assign[n] = shard
            shard += 1
            used = 0
            continue
        if used > 0 and used + params[n] > budget * 1.05 and params[n] > 0:
            shard += 1
            used = 0
        # skip-connection collapse: a parameter-free node joins the earliest shard its inputs allow
        if params[n] == 0 and n.all_input_nodes:
            earliest = max(assign.get(a, 0) for a in n.all_input_nodes)
            assign[n] = max(earliest, 0)
            continue
        assign[n] = shard
        used += params[n]
    assign = _legalise(nodes, assign)
    return split_graph(gm, assign, max(assign.values()) + 1 if assign else 1)


def shard_model(gm: fx.GraphModule, split_method: str = "nearest_min_deps", shard_count: Optional[int] = None,
                model_type: Optional[str] = None, custom_split_points=None):
    """Dispatch on ``args.split_method`` (Merak/core/fx/graph_shard/split_graph.py:30-79)."""
    if split_method == "layer_split":
        return layer_split(gm, model_type, custom_split_points)
    if split_method == "nearest_min_deps":
        return nearest_min_deps(gm, shard_count)
    if split_method == "farthest_min_deps":
        return farthest_min_deps(gm, shard_count or 1)
    raise ValueError("unknown split_method %r" % split_method)
