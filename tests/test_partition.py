"""Stage-partition math and the native AutoPipe search against recorded outputs of the reference
partitioner (compiled unmodified) on the same cost vectors."""
import pytest

from merak_b200.pipeline import partition as P

AUTOPIPE_GOLDEN = [
    ([1000] * 24, [3000] * 24, 4, [0, 6, 12, 18]),
    ([1000] * 24, [3000] * 24, 2, [0, 12]),
    ([50] + [100, 200] * 12 + [30, 400], None, 4, [0, 8, 15, 21]),
    ([50] + [100, 200] * 12 + [30, 400], None, 2, [0, 15]),
    ([50] + [100, 200] * 12 + [30, 400], None, 8, [0, 4, 8, 12, 16, 19, 22, 25]),
    ([10, 20, 30, 40, 50, 60, 70, 80], "x2", 3, [0, 5, 7]),
    ([5, 5, 5, 5], [5, 5, 5, 5], 4, [0, 1, 2, 3]),
    ([1, 1, 100, 1, 1, 1], "x2", 3, [0, 2, 3]),
]


@pytest.mark.parametrize("fwd,bwd,stages,want", AUTOPIPE_GOLDEN)
def test_autopipe_golden(fwd, bwd, stages, want):
    if bwd is None:
        bwd = [3 * f for f in fwd]
    elif bwd == "x2":
        bwd = [2 * f for f in fwd]
    assert P.autopipe_partition(fwd, bwd, stages) == want


def test_autopipe_never_worse_than_minmax_seed():
    import random
    rnd = random.Random(0)
    for _ in range(20):
        n, s = rnd.randint(6, 30), rnd.randint(2, 5)
        fwd = [rnd.randint(1, 500) for _ in range(n)]
        bwd = [rnd.randint(1, 3) * f for f in fwd]
        starts = P.autopipe_partition(fwd, bwd, s)
        assert starts[0] == 0 and all(a <= b for a, b in zip(starts, starts[1:])) and starts[-1] < n
        t, crit = P.autopipe_simulate(fwd, bwd, starts)
        seed = P.partition_balanced([f + b for f, b in zip(fwd, bwd)], s)[:-1]
        ts, _ = P.autopipe_simulate(fwd, bwd, seed)
        assert t > 0 and (ts < 0 or t <= ts)


UNIFORM_FLOOR = {(28, 2): [0, 14, 28], (28, 4): [0, 7, 14, 21, 28], (52, 4): [0, 13, 26, 39, 52],
                 (52, 8): [0, 6, 13, 20, 27, 34, 40, 46, 52], (100, 8): [0, 12, 25, 38, 51, 64, 76, 88, 100],
                 (27, 4): [0, 6, 13, 20, 27], (12, 5): [0, 2, 5, 8, 10, 12], (7, 4): [0, 1, 3, 5, 7],
                 (3, 4): [0, 1, 2, 3, 3]}


@pytest.mark.parametrize("key", sorted(UNIFORM_FLOOR))
def test_partition_uniform_floor_golden(key):
    """The default method must map layers to stages exactly like the reference does, or
    per-stage checkpoints would not line up."""
    assert P.partition_uniform(*key) == UNIFORM_FLOOR[key]


@pytest.mark.parametrize("items,parts", [(52, 8), (12, 5), (7, 4), (28, 4), (100, 8)])
def test_partition_uniform_ceil_is_valid(items, parts):
    got = P.partition_uniform(items, parts, use_ceil=True)
    assert got[0] == 0 and got[-1] == items and all(a <= b for a, b in zip(got, got[1:]))
    sizes = [b - a for a, b in zip(got, got[1:])]
    assert max(sizes) - min(sizes) <= 1 and sizes[0] == max(sizes)


def test_partition_balanced_golden():
    w = [38597376] + [2362368, 4722432] * 12 + [1536, 0]
    assert P.partition_balanced(w, 4) == [0, 1, 12, 22, 27]
    assert P.partition_balanced(w, 2) == [0, 8, 27]
    assert P.partition_balanced(list(range(1, 11)), 3) == [0, 6, 8, 10]
    assert P.partition_balanced([5] * 10, 4) == [0, 3, 6, 9, 10]


def test_partition_layers_dispatch():
    assert P.partition_layers("custom", 10, 3, custom=[0, 2, 7]) == [0, 2, 7, 10]
    assert P.partition_layers("uniform_floor", 28, 4) == [0, 7, 14, 21, 28]
    assert P.partition_layers("autopipe", 24, 4, fwd_costs=[1000] * 24, bwd_costs=[3000] * 24) == [0, 6, 12, 18, 24]
    with pytest.raises(ValueError):
        P.partition_layers("custom", 10, 3, custom=[0, 8, 4])


def test_layer_partition_object_methods():
    """``LayerPartition`` gives the five methods over one shard list and falls back to ``uniform`` when a
    method would leave a stage empty (Merak/core/pipeline/layers_partition.py:29-163)."""
    from types import SimpleNamespace

    import torch.nn as nn

    from merak_b200.pipeline.partition import LayerPartition
    layers = [nn.Linear(4, 4 * (1 + (i == 0) * 7)) for i in range(6)]          # the first shard is 8 x the others
    args = SimpleNamespace(partition_method="parameters", custom_partition=[0, 1, 6])
    lp = LayerPartition(args, layers, num_stages=2)
    assert lp.param_counts == [sum(p.numel() for p in l.parameters()) for l in layers]
    assert lp.uniform() == [0, 3, 6] and lp.uniform_floor() == [0, 3, 6]
    assert lp.parameters() == [0, 1, 6] == lp.partition()                     # balanced by parameter count
    assert lp.custom_layer_idx() == [0, 1, 6]
    auto = lp.autopipe()                                                      # costs from parameter counts here
    assert auto[0] == 0 and auto[-1] == 6 and len(auto) == 3 and auto[1] in range(1, 6)
    args.custom_partition = [0, 0, 6]                                         # a stage without shards
    assert lp.partition("custom") == lp.uniform()
    import pytest
    with pytest.raises(ValueError):
        lp.partition("nonsense")
