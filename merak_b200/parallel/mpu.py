"""Process-wide registry of the parallel grid and its communicators.

``initialize.init`` builds one :class:`~merak_b200.parallel.topology.ParallelGrid` and registers
it here; every layer, mapping and engine component asks this module for "my tensor-parallel
group / rank / size" and friends.  The getters mirror the names of the reference registry
(Merak/core/mpu/initialize.py:27-181).  Before ``init`` is called (single-process unit tests)
every axis reports size 1 / rank 0 and group ``None``.
"""
from __future__ import annotations

from typing import Optional

_GRID = None
_TOPO = None


def set_grid(grid, topo):
    global _GRID, _TOPO
    _GRID, _TOPO = grid, topo


def get_grid():
    return _GRID


def get_topo():
    return _TOPO


def is_initialized() -> bool:
    return _GRID is not None


def destroy_model_parallel():
    set_grid(None, None)


# ---- tensor ("model" / "slice") parallel ------------------------------------------------------
def get_model_parallel_group():
    return _GRID.get_slice_parallel_group() if _GRID else None


def get_model_parallel_world_size() -> int:
    return _GRID.get_slice_parallel_world_size() if _GRID else 1


def get_model_parallel_rank() -> int:
    return _GRID.get_slice_parallel_rank() if _GRID else 0


def get_model_parallel_ranks():
    return _GRID.ranks("model") if _GRID else [0]


def get_model_parallel_src_rank() -> int:
    """Global rank of the first member of this rank's tensor-parallel group."""
    return _GRID.ranks("model")[0] if _GRID else 0


# ---- data parallel ---------------------------------------------------------------------------
def get_data_parallel_group():
    return _GRID.get_data_parallel_group() if _GRID else None


def get_data_parallel_world_size() -> int:
    return _GRID.get_data_parallel_world_size() if _GRID else 1


def get_data_parallel_rank() -> int:
    return _GRID.get_data_parallel_rank() if _GRID else 0


def get_data_parallel_ranks():
    return _GRID.ranks("data") if _GRID else [0]


# ---- pipeline parallel ---------------------------------------------------------------------
def get_pipe_parallel_group():
    return _GRID.get_pipe_parallel_group() if _GRID else None


def get_pipe_parallel_world_size() -> int:
    return _GRID.get_pipe_parallel_world_size() if _GRID else 1


def get_pipe_parallel_rank() -> int:
    return _GRID.get_pipe_parallel_rank() if _GRID else 0


def get_pipeline_model_parallel_prev_rank() -> Optional[int]:
    return _GRID.prev_rank if _GRID else None


def get_pipeline_model_parallel_next_rank() -> Optional[int]:
    return _GRID.next_rank if _GRID else None


def is_pipeline_first_stage() -> bool:
    return get_pipe_parallel_rank() == 0


def is_pipeline_last_stage() -> bool:
    return get_pipe_parallel_rank() == get_pipe_parallel_world_size() - 1


# ---- sequence (Ulysses) parallel -----------------------------------------------------------
def get_sequence_parallel_group():
    return _GRID.get_sequence_parallel_group() if _GRID else None


def get_sequence_parallel_world_size() -> int:
    return _GRID.get_sequence_parallel_world_size() if _GRID else 1


def get_sequence_parallel_rank() -> int:
    return _GRID.get_sequence_parallel_rank() if _GRID else 0


# ---- expert parallel -----------------------------------------------------------------------
def get_expert_parallel_group():
    return _GRID.get_expert_parallel_group() if _GRID else None


def get_expert_parallel_world_size() -> int:
    return _GRID.get_expert_parallel_world_size() if _GRID else 1


def get_expert_parallel_rank() -> int:
    return _GRID.get_expert_parallel_rank() if _GRID else 0


def get_global_rank() -> int:
    return _GRID.get_global_rank() if _GRID else 0
