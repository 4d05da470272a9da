"""Small helpers of the parallel layers (Merak/core/mpu/utils.py:21-106)."""
from __future__ import annotations

from typing import List

from .layers import VocabUtility, divide, split_tensor_along_last_dim  # noqa: F401  (re-exported)


def ensure_divisibility(numerator: int, denominator: int):
    if numerator % denominator != 0:
        raise ValueError("%d is not divisible by %d" % (numerator, denominator))


def channels_uniform(channels: int, parts: int) -> List[int]:
    """Boundaries ``[c_0 = 0, ..., c_parts = channels]`` of an as-even-as-possible channel split: the
    first ``channels % parts`` parts get one channel more."""
    base, rem = divmod(channels, parts)
    bounds = [0]
    for r in range(parts):
        bounds.append(bounds[-1] + base + (1 if r < rem else 0))
    return bounds
