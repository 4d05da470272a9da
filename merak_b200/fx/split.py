"""Cut a traced graph into a *sequence* of sub-graphs.

Given a map ``node -> shard index`` (non-decreasing along the topological order), ``split_graph``
builds one ``GraphModule`` per shard such that shard ``i`` receives all of its inputs from shard
``i-1``: a value produced in shard ``a`` and consumed in shard ``b > a+1`` is passed *through*
every shard in between (multi-hop forwarding), because pipeline stages only talk to their
neighbours.  Model inputs are fed to the first shard that uses them (``input_to_shard``), and
forwarded from there if later shards use them too.

This is the behaviour of the reference splitter (Merak/core/fx/graph_shard/split_module.py:
147-196,262-328), re-expressed as a liveness computation over the shard sequence.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch
import torch.fx as fx
import torch.nn as nn


class ShardModule(fx.GraphModule):
    """One shard.  ``input_names`` / ``output_names`` name the values it takes and returns (as a
    tuple, in order); ``external_inputs`` are model inputs this shard reads from the data loader."""

    input_names: List[str]
    output_names: List[str]
    external_inputs: List[str]


def split_graph(gm: fx.GraphModule, node_to_shard: Dict[fx.Node, int], num_shards: int):
    """Returns ``(shards, input_to_shard)``."""
    graph = gm.graph
    nodes = [n for n in graph.nodes if n.op not in ("placeholder", "output")]
    placeholders = [n for n in graph.nodes if n.op == "placeholder"]
    output_node = next(n for n in graph.nodes if n.op == "output")

    def users_shards(n: fx.Node) -> List[int]:
        out = []
        for u in n.users:
            if u.op == "output":
                out.append(num_shards - 1)
            else:
                out.append(node_to_shard[u])
        return out

    # model inputs: first shard that uses each placeholder
    input_to_shard: Dict[str, int] = {}
    def_shard: Dict[fx.Node, int] = {}
    for ph in placeholders:
        us = users_shards(ph)
        first = min(us) if us else 0
        input_to_shard[ph.name] = first
        def_shard[ph] = first
    for n in nodes:
        def_shard[n] = node_to_shard[n]
    last_use: Dict[fx.Node, int] = {}
    for n in placeholders + nodes:
        us = users_shards(n)
        last_use[n] = max(us) if us else def_shard[n]

    order = {n: i for i, n in enumerate(graph.nodes)}
    final_outputs = []          # values the model returns
    def collect(a):
        if isinstance(a, fx.Node):
            final_outputs.append(a)
        return a
    fx.node.map_arg(output_node.args, collect)

    shards: List[ShardModule] = []
    for s in range(num_shards):
        live_in = sorted([n for n in def_shard if def_shard[n] < s and last_use[n] >= s], key=order.get)
        external = [ph for ph in placeholders if def_shard[ph] == s]
        own = [n for n in nodes if node_to_shard[n] == s]
        if s < num_shards - 1:
            live_out = sorted([n for n in def_shard if def_shard[n] <= s and last_use[n] > s], key=order.get)
        else:
            live_out = list(final_outputs)
        g = fx.Graph()
        env: Dict[fx.Node, fx.Node] = {}
        for n in live_in:
            env[n] = g.placeholder(n.name)
        for ph in external:
            env[ph] = g.placeholder(ph.name)
        for n in own:
            env[n] = g.node_copy(n, lambda a: env[a])
        if s < num_shards - 1:
            g.output(tuple(env[n] for n in live_out))
        else:
            g.output(fx.node.map_arg(output_node.args[0], lambda a: env[a]))
        _no_inplace_on_inputs(gm, g)
        sub = ShardModule(gm, g, class_name="Shard%d" % s)
        sub.input_names = [n.name for n in live_in]
        sub.external_inputs = [ph.name for ph in external]
        sub.output_names = [n.name for n in live_out]
        sub.shard_index = s
        shards.append(sub)
    return shards, input_to_shard


def _no_inplace_on_inputs(gm: fx.GraphModule, g: fx.Graph):
    """A shard's inputs arrive as leaf tensors that require grad (stage boundary, recomputed segment); an
    in-place operation on such a tensor is an autograd error.  Where a shard's first use of an input is in
    place (``nn.ReLU(inplace=True)`` right after a cut in torchvision's ResNets, ``x.add_(...)``,
    ``F.relu(x, inplace=True)``), the operation runs out of place and every later reader of that input reads
    its result, which is what the in-place form would have shown them."""
    import copy
    order = {n: i for i, n in enumerate(g.nodes)}
    for node in list(g.nodes):
        first = node.args[0] if node.args and isinstance(node.args[0], fx.Node) else None
        if first is None or first.op != "placeholder":
            continue
        changed = False
        if node.op == "call_module":
            mod = gm.get_submodule(node.target)
            if getattr(mod, "inplace", False) is True:
                name = node.target + "_out_of_place"
                try:
                    gm.get_submodule(name)
                except AttributeError:
                    clone = copy.copy(mod)
                    clone.inplace = False
                    gm.add_submodule(name, clone)
                node.target = name
                changed = True
        elif node.op == "call_function" and node.kwargs.get("inplace") is True:
            node.kwargs = {**node.kwargs, "inplace": False}
            changed = True
        elif node.op == "call_function" and isinstance(node.target, torch._ops.OpOverload) and \
                node.target._schema.name.endswith("_") and node.target._schema.name.startswith("aten::"):
            # an ATen in-place overload of an exported graph (aten.relu_.default, aten.add_.Tensor)
            base = getattr(torch.ops.aten, node.target._schema.name[len("aten::"):-1], None)
            twin = getattr(base, node.target._overloadname, None) if base is not None else None
            if twin is not None:
                node.target = twin
                changed = True
        elif node.op == "call_method" and node.target.endswith("_") and not node.target.endswith("__") and \
                callable(getattr(torch.Tensor, node.target[:-1], None)):       # not ``requires_grad_`` (an attribute)
            node.target = node.target[:-1]
            changed = True
        if changed:
            for user in list(first.users):
                if user is not node and order[user] > order[node]:
                    user.replace_input_with(first, node)


def run_shards(shards: List[ShardModule], inputs: Dict[str, torch.Tensor]):
    """Executes the shard sequence on one device (reference semantics check and single-stage use)."""
    carried: Tuple = ()
    for sh in shards:
        args = list(carried) + [inputs[name] for name in sh.external_inputs]
        out = sh(*args)
        carried = out if isinstance(out, tuple) else (out,)
        last = out
    return last
