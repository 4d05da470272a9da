"""Hook for the fused data-parallel path: gradient reduce-scatter + AdamW + parameter all-gather
in one kernel over peer memory.  ``try_fused_reduce`` returns False when that path is not
available (CPU, single rank, ``comm_mode='nccl'``), and the engine falls back to
``torch.distributed`` collectives."""
from __future__ import annotations


def try_fused_reduce(engine, group) -> bool:
    from . import symm
    if getattr(engine.args, "comm_mode", "fused") != "fused" or engine.flat is None:
        return False
    if not engine.flat.grad.is_cuda or engine.dp_size == 1:
        return False
    return symm.fused_dp_step(engine, group)
