"""Symmetric-memory data plane (peer-mapped buffers + signal pads) for the fused
compute+collective kernels.  Filled in by the multi-GPU kernels; until a buffer set is registered
every entry point reports "not available" so callers use the NCCL path."""
from __future__ import annotations


def fused_dp_step(engine, group) -> bool:
    return False
