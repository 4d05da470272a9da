"""Assigning the shard sequence to pipeline stages (``args.partition_method``).

``uniform`` / ``uniform_floor`` / ``parameters`` / ``custom`` / ``autopipe`` as in the reference
(Merak/core/pipeline/layers_partition.py:62-163, Merak/core/pipeline/module_utils.py:54-157).
``partition_uniform(..., use_ceil=True)`` of the reference overshoots when the item count is not a
multiple of the part count; here the ceil variant hands the remainder to the *first* stages and
always returns a valid boundary list.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence


def partition_uniform(num_items: int, num_parts: int, use_ceil: bool = False) -> List[int]:
    """Boundaries ``[0, ..., num_items]``.  Floor variant (default method ``uniform_floor``): every
    stage gets ``floor(items/parts)`` and the ``r`` left-over items go to stages ``1..r``, so the
    first stage (which also holds the embeddings) stays the lightest - the layer-to-stage map of the
    reference's default method.  Ceil variant: stages ``0..r-1`` receive the left-over items."""
    if num_parts <= 0:
        raise ValueError("num_parts must be positive")
    parts = [0] * (num_parts + 1)
    if num_items <= num_parts:
        for p in range(num_parts + 1):
            parts[p] = min(p, num_items)
        return parts
    base, rem = divmod(num_items, num_parts)
    for p in range(num_parts):
        extra = (1 if p < rem else 0) if use_ceil else (1 if 1 <= p <= rem else 0)
        parts[p + 1] = parts[p] + base + extra
    return parts


def prefix_sum_inc(weights: Sequence[float]) -> List[float]:
    out, acc = [], 0
    for w in weights:
        acc += w
        out.append(acc)
    return out


def _lprobe(prefix: Sequence[float], num_parts: int, bottleneck: float):
    """Greedy check: can the items be cut into ``num_parts`` contiguous parts of weight <= bottleneck?"""
    import bisect
    n = len(prefix)
    parts = [0] * (num_parts + 1)
    for p in range(1, num_parts + 1):
        parts[p] = n
    total = prefix[-1]
    budget = bottleneck
    step = 1
    while step < num_parts and budget < total:
        parts[step] = bisect.bisect_left(prefix, budget)
        if parts[step] < n:
            budget = prefix[parts[step] - 1] + bottleneck if parts[step] > 0 else bottleneck
            if parts[step] == parts[step - 1]:
                return parts, False      # a single item exceeds the bottleneck
        step += 1
    return parts, budget >= total


def partition_balanced(weights: Sequence[float], num_parts: int, eps: float = 1e-3) -> List[int]:
    """Contiguous partition minimising the heaviest part (binary search on the bottleneck)."""
    n = len(weights)
    if n <= num_parts:
        return partition_uniform(n, num_parts)
    prefix = prefix_sum_inc(weights)
    lo, hi = max(max(weights), prefix[-1] / num_parts) - eps, float(prefix[-1])
    lo = max(lo, 0.0)
    while hi - lo > eps:
        mid = lo + (hi - lo) / 2
        _, ok = _lprobe(prefix, num_parts, mid)
        if ok:
            hi = mid
        else:
            lo = mid
    parts, ok = _lprobe(prefix, num_parts, hi)
    assert ok
    return parts


def autopipe_partition(fwd_costs: Sequence[int], bwd_costs: Sequence[int], num_stages: int) -> List[int]:
    """Stage start indices from the native AutoPipe search (``csrc/autopipe.cpp``)."""
    from ..ops import _lib
    lib = _lib.native()
    n = len(fwd_costs)
    if num_stages > n:
        raise ValueError("more stages (%d) than layers (%d)" % (num_stages, n))
    f = (ctypes.c_longlong * n)(*[int(x) for x in fwd_costs])
    b = (ctypes.c_longlong * n)(*[int(x) for x in bwd_costs])
    out = (ctypes.c_int * num_stages)()
    lib.mrk_autopipe_partition.restype = ctypes.c_int
    rc = lib.mrk_autopipe_partition(f, b, n, num_stages, out)
    if rc != 0:
        raise RuntimeError("autopipe partition failed (%d)" % rc)
    return list(out)


def autopipe_simulate(fwd_costs, bwd_costs, starts):
    """(iteration time, critical stage) of a partition under the AutoPipe 1F1B cost model."""
    from ..ops import _lib
    lib = _lib.native()
    n, s = len(fwd_costs), len(starts)
    f = (ctypes.c_longlong * n)(*[int(x) for x in fwd_costs])
    b = (ctypes.c_longlong * n)(*[int(x) for x in bwd_costs])
    st = (ctypes.c_int * s)(*starts)
    crit = ctypes.c_int(-1)
    lib.mrk_autopipe_simulate.restype = ctypes.c_longlong
    t = lib.mrk_autopipe_simulate(f, b, n, st, s, ctypes.byref(crit))
    return int(t), crit.value


def partition_layers(method: str, num_layers: int, num_stages: int, param_counts: Sequence[int] = (),
                     custom: Sequence[int] = (), fwd_costs: Sequence[int] = (), bwd_costs: Sequence[int] = ()):
    """Boundaries ``parts`` with ``parts[s] .. parts[s+1]`` the shards of stage ``s``."""
    method = method.lower()
    if method == "uniform":
        return partition_uniform(num_layers, num_stages, use_ceil=True)
    if method == "uniform_floor":
        return partition_uniform(num_layers, num_stages, use_ceil=False)
    if method == "parameters":
        return partition_balanced(list(param_counts), num_stages)
    if method == "custom":
        parts = [int(x) for x in custom]
        if parts[0] != 0:
            parts = [0] + parts
        if parts[-1] != num_layers:
            parts = parts + [num_layers]
        if len(parts) != num_stages + 1 or any(a > b for a, b in zip(parts, parts[1:])):
            raise ValueError("custom_partition %r does not describe %d stages over %d layers" %
                             (custom, num_stages, num_layers))
        return parts
    if method == "autopipe":
        starts = autopipe_partition(fwd_costs, bwd_costs, num_stages)
        return starts + [num_layers]
    raise ValueError("unknown partition_method %r" % method)


class LayerPartition:
    """The partition methods as an object over one shard list, the form the pipeline module uses
    (Merak/core/pipeline/layers_partition.py:29-163): ``uniform()``, ``uniform_floor()``,
    ``parameters()``, ``custom_layer_idx()`` and ``autopipe()`` each return the stage boundaries;
    ``partition()`` dispatches on ``args.partition_method`` and falls back to ``uniform`` when a
    method would leave a stage without shards."""

    def __init__(self, args, layers: Sequence, num_stages: int, param_counts: Sequence[int] = ()):
        self.args, self.layers, self.num_stages = args, list(layers), int(num_stages)
        self.param_counts = list(param_counts) or self._count_layer_params()

    def _count_layer_params(self) -> List[int]:
        return [sum(p.numel() for p in l.parameters()) if l is not None else 0 for l in self.layers]

    def uniform(self) -> List[int]:
        return partition_layers("uniform", len(self.layers), self.num_stages)

    def uniform_floor(self) -> List[int]:
        return partition_layers("uniform_floor", len(self.layers), self.num_stages)

    def parameters(self) -> List[int]:
        return partition_layers("parameters", len(self.layers), self.num_stages, param_counts=self.param_counts)

    def custom_layer_idx(self) -> List[int]:
        return partition_layers("custom", len(self.layers), self.num_stages, custom=self.args.custom_partition)

    def layer_costs(self) -> List[int]:
        """Per-shard forward cost for ``autopipe``: MFLOPs from the profiler when the shards can be run
        on their dummy inputs; parameter counts stand in when they cannot (meta weights)."""
        dummy = getattr(self.layers[0], "dummy_inputs", None) if self.layers else None
        if dummy is not None:
            try:
                from ..fx.split import run_shards
                from .profiler import profile_layer_costs
                return profile_layer_costs(self.layers, lambda: run_shards(self.layers, dummy))
            except Exception:
                pass
        return [max(1, c // 1000) for c in self.param_counts]

    def autopipe(self) -> List[int]:
        fwd = self.layer_costs()          # the backward pass is taken as three forward passes, as in the reference
        return partition_layers("autopipe", len(self.layers), self.num_stages, fwd_costs=fwd,
                                bwd_costs=[3 * f for f in fwd])

    def partition(self, method: str = None) -> List[int]:
        method = (method or self.args.partition_method).lower()
        table = {"uniform": self.uniform, "uniform_floor": self.uniform_floor, "parameters": self.parameters,
                 "custom": self.custom_layer_idx, "autopipe": self.autopipe}
        if method not in table:
            raise ValueError("unknown partition_method %r" % method)
        parts = table[method]()
        if any(parts[i] == parts[i + 1] for i in range(self.num_stages)) and len(self.layers) >= self.num_stages:
            parts = self.uniform()
        return parts
