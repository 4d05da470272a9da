"""Rank arithmetic of the parallel grid and the process groups built on it.

``ProcessTopology`` is pure integer math (no ``torch.distributed`` needed) mapping named axes to
global ranks in row-major order.  The axis order used by the framework is
``pipe, data, sequence, model``: tensor-parallel ("model") peers are adjacent global ranks, so on
an NVSwitch node a TP group is any set of neighbouring GPUs, and pipeline neighbours are the
farthest apart.  Same ordering and the same query API as the reference
(Merak/core/mpu/topology.py:14-276).

``ParallelGrid`` creates the process groups once per axis (Merak/core/mpu/topology.py:279-508).
Unlike the reference it accepts any backend (``gloo`` for CPU tests), creates no singleton
groups for size-1 axes (the WORLD-independent ``None``-group fast path is used instead), and adds
expert-parallel groups as sub-groups of the data axis.
"""
from __future__ import annotations

import itertools
from collections import namedtuple
from typing import Dict, List, Optional, Sequence


class ProcessTopology:
    """Cartesian mapping ``coordinate <-> rank`` over named axes, last axis fastest."""

    def __init__(self, axes: Sequence[str], dims: Sequence[int]):
        if len(axes) != len(dims):
            raise ValueError("axes and dims differ in length")
        if any(d < 1 for d in dims):
            raise ValueError("every axis needs at least one rank: %r" % (dims,))
        self.axes = list(axes)
        self.dims = list(dims)
        self.ProcessCoord = namedtuple("ProcessCoord", self.axes)
        self._strides = []
        stride = 1
        for d in reversed(self.dims):
            self._strides.insert(0, stride)
            stride *= d
        self._world = stride

    # -- basic queries ------------------------------------------------------------------------
    def world_size(self) -> int:
        return self._world

    def get_axis_names(self) -> List[str]:
        return list(self.axes)

    def get_dim(self, axis: str) -> int:
        if axis not in self.axes:
            return 0
        return self.dims[self.axes.index(axis)]

    def get_rank(self, **coord) -> int:
        if set(coord) != set(self.axes):
            raise ValueError("get_rank() needs every axis %r, got %r" % (self.axes, sorted(coord)))
        rank = 0
        for axis, stride, dim in zip(self.axes, self._strides, self.dims):
            c = coord[axis]
            if not 0 <= c < dim:
                raise ValueError("coordinate %s=%d outside [0,%d)" % (axis, c, dim))
            rank += c * stride
        return rank

    def get_coord(self, rank: int):
        if not 0 <= rank < self._world:
            raise ValueError("rank %d not in topology of %d ranks" % (rank, self._world))
        vals = []
        for stride, dim in zip(self._strides, self.dims):
            vals.append((rank // stride) % dim)
        return self.ProcessCoord(*vals)

    def get_rank_repr(self, rank: int, omit_axes=("data", "pipe"), inner_sep="_", outer_sep="-") -> str:
        """String such as ``model_01`` used in checkpoint file names."""
        omit = frozenset(omit_axes)
        coord = self.get_coord(rank)
        parts = []
        for axis in self.axes:
            if axis in omit:
                continue
            parts.append("%s%s%02d" % (axis, inner_sep, getattr(coord, axis)))
        return outer_sep.join(parts)

    # -- group enumeration --------------------------------------------------------------------
    def get_axis_comm_lists(self, axis: str) -> List[List[int]]:
        """All rank lists that differ only along ``axis`` (one list per communicator)."""
        if axis not in self.axes:
            return []
        other = [a for a in self.axes if a != axis]
        ranges = [range(self.get_dim(a)) for a in other]
        lists = []
        for combo in itertools.product(*ranges):
            fixed = dict(zip(other, combo))
            lists.append([self.get_rank(**fixed, **{axis: i}) for i in range(self.get_dim(axis))])
        return lists

    def filter_match(self, **filt) -> List[int]:
        """Ranks whose coordinates equal every given ``axis=value``."""
        out = []
        for rank in range(self._world):
            coord = self.get_coord(rank)
            if all(getattr(coord, k) == v for k, v in filt.items()):
                out.append(rank)
        return out

    def get_axis_list(self, axis: str, idx: int) -> List[int]:
        """Ranks whose coordinate on ``axis`` is ``idx``."""
        return self.filter_match(**{axis: idx})

    def __str__(self):
        return "ProcessTopology(%s)" % ", ".join("%s=%d" % ad for ad in zip(self.axes, self.dims))

    __repr__ = __str__


class PipeDataParallelTopology(ProcessTopology):
    def __init__(self, num_pp: int, num_dp: int):
        super().__init__(["pipe", "data"], [num_pp, num_dp])


class PipeModelDataParallelTopology(ProcessTopology):
    def __init__(self, num_pp: int, num_mp: int, num_dp: int):
        super().__init__(["pipe", "data", "model"], [num_pp, num_dp, num_mp])


class PipeDataSequenceParallelTopology(ProcessTopology):
    def __init__(self, num_pp: int, num_dp: int, num_sp: int):
        super().__init__(["pipe", "data", "sequence"], [num_pp, num_dp, num_sp])


class PipeDataSequenceModelParallelTopology(ProcessTopology):
    def __init__(self, num_pp: int, num_dp: int, num_sp: int, num_mp: int):
        super().__init__(["pipe", "data", "sequence", "model"], [num_pp, num_dp, num_sp, num_mp])


def expert_parallel_lists(topo: ProcessTopology, ep: int) -> List[List[int]]:
    """Splits every data-parallel communicator into contiguous expert-parallel groups of ``ep``."""
    if ep <= 1:
        return []
    out = []
    for ranks in topo.get_axis_comm_lists("data"):
        if len(ranks) % ep != 0:
            raise ValueError("expert parallel degree %d does not divide dp=%d" % (ep, len(ranks)))
        for i in range(0, len(ranks), ep):
            out.append(ranks[i:i + ep])
    return out


class ParallelGrid:
    """Process groups for every axis of a topology, for the calling rank.

    ``process_groups=False`` skips ``torch.distributed`` entirely (rank math only), which is how
    unit tests inspect any ``(rank, topology)`` pair inside one process.
    """

    def __init__(self, topology: ProcessTopology, rank: Optional[int] = None, ep: int = 1,
                 process_groups: bool = True):
        self._topo = topology
        self.world_size = topology.world_size()
        self.ep = max(1, ep)
        dist = None
        if process_groups:
            import torch.distributed as dist_mod

            dist = dist_mod
            if not dist.is_initialized():
                raise RuntimeError("torch.distributed is not initialised")
            if dist.get_world_size() != self.world_size:
                raise ValueError("topology has %d ranks but the job has %d" %
                                 (self.world_size, dist.get_world_size()))
            rank = dist.get_rank()
        if rank is None:
            raise ValueError("rank is required when process_groups=False")
        self.global_rank = rank
        coord = topology.get_coord(rank)
        self.pipe_parallel_size = max(1, topology.get_dim("pipe"))
        self.data_parallel_size = max(1, topology.get_dim("data"))
        self.model_parallel_size = max(1, topology.get_dim("model"))       # tensor ("slice") parallel
        self.sequence_parallel_size = max(1, topology.get_dim("sequence"))
        self.stage_id = getattr(coord, "pipe", 0)
        self.data_parallel_id = getattr(coord, "data", 0)
        self.model_parallel_id = getattr(coord, "model", 0)
        self.sequence_parallel_id = getattr(coord, "sequence", 0)

        self._groups: Dict[str, object] = {}
        self._ranks: Dict[str, List[int]] = {}
        for axis in ("data", "pipe", "model", "sequence"):
            lists = topology.get_axis_comm_lists(axis) or [[r] for r in range(self.world_size)]
            self._ranks[axis] = next(l for l in lists if rank in l)
            if dist is not None:
                if len(lists[0]) == 1:
                    self._groups[axis] = None
                elif len(lists) == 1:
                    self._groups[axis] = dist.group.WORLD
                else:
                    for l in lists:                       # collective: every rank creates every group
                        g = dist.new_group(ranks=l)
                        if rank in l:
                            self._groups[axis] = g
        ep_lists = expert_parallel_lists(topology, self.ep)
        if ep_lists:
            self._ranks["expert"] = next(l for l in ep_lists if rank in l)
            if dist is not None:
                for l in ep_lists:
                    g = dist.new_group(ranks=l)
                    if rank in l:
                        self._groups["expert"] = g
        else:
            self._ranks["expert"] = [rank]
            self._groups["expert"] = None

        # pipeline neighbours in global ranks
        pipe_ranks = self._ranks["pipe"]
        self.pp_ranks = pipe_ranks
        self.is_first_stage = self.stage_id == 0
        self.is_last_stage = self.stage_id == self.pipe_parallel_size - 1
        self.prev_rank = pipe_ranks[(self.stage_id - 1) % len(pipe_ranks)]
        self.next_rank = pipe_ranks[(self.stage_id + 1) % len(pipe_ranks)]
        self.p2p_groups = self._build_p2p_pairs()

    def _build_p2p_pairs(self):
        pairs = []
        for ranks in self._topo.get_axis_comm_lists("pipe") or []:
            for i, r in enumerate(ranks):
                pairs.append([r, ranks[(i + 1) % len(ranks)]])
        return pairs

    # -- reference-compatible getters ---------------------------------------------------------
    @property
    def topology(self) -> ProcessTopology:
        return self._topo

    def get_stage_id(self):
        return self.stage_id

    def get_data_parallel_id(self):
        return self.data_parallel_id

    def get_global_rank(self):
        return self.global_rank

    def stage_to_global(self, stage_id: int, **kwargs) -> int:
        coord = self._topo.get_coord(self.global_rank)._asdict()
        coord.update(kwargs)
        coord["pipe"] = stage_id
        return self._topo.get_rank(**coord)

    def group(self, axis: str):
        return self._groups.get(axis)

    def ranks(self, axis: str) -> List[int]:
        return self._ranks[axis]

    def get_pipe_parallel_rank(self):
        return self.stage_id

    def get_pipe_parallel_world_size(self):
        return self.pipe_parallel_size

    def get_pipe_parallel_group(self):
        return self._groups.get("pipe")

    def get_data_parallel_rank(self):
        return self.data_parallel_id

    def get_data_parallel_world_size(self):
        return self.data_parallel_size

    def get_data_parallel_group(self):
        return self._groups.get("data")

    def get_slice_parallel_rank(self):
        return self.model_parallel_id

    def get_slice_parallel_world_size(self):
        return self.model_parallel_size

    def get_slice_parallel_group(self):
        return self._groups.get("model")

    # In the reference the grid's "model parallel" getters describe the whole non-data block, but
    # what Merak.init registers as *the* model-parallel group is the tensor ("slice") group
    # (Merak/initialize.py:78).  The grid follows the registered meaning.
    get_model_parallel_rank = get_slice_parallel_rank
    get_model_parallel_world_size = get_slice_parallel_world_size
    get_model_parallel_group = get_slice_parallel_group

    def get_sequence_parallel_rank(self):
        return self.sequence_parallel_id

    def get_sequence_parallel_world_size(self):
        return self.sequence_parallel_size

    def get_sequence_parallel_group(self):
        return self._groups.get("sequence")

    def get_expert_parallel_rank(self):
        return self._ranks["expert"].index(self.global_rank)

    def get_expert_parallel_world_size(self):
        return len(self._ranks["expert"])

    def get_expert_parallel_group(self):
        return self._groups.get("expert")


# Name kept for users of the reference API.
PipelineParallelGrid = ParallelGrid
