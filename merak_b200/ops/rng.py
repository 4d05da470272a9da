"""Device-resident state of the counter-based dropout generator.

A dropout call draws its mask from ``philox(seed, offset + call_id, element)``.  ``seed`` and
``offset`` live in a 2-element int64 tensor on the device so that advancing the step (``offset``)
is a device-side add, which keeps a captured CUDA graph valid across steps.  ``call_id`` numbers
the dropout call sites inside one step; activation recomputation restores it so the replayed
forward regenerates identical masks (the role ``RNGStatesTracker`` plays in the reference,
Merak/core/recompute/checkpointing.py:106-184).
"""
from __future__ import annotations

import torch

_STEP_STRIDE = 1 << 20


class DropoutState:
    def __init__(self):
        self._state = {}      # device -> tensor [seed, offset]
        self.call_id = 0
        self.seed = 1234

    def manual_seed(self, seed: int):
        self.seed = int(seed)
        for t in self._state.values():
            t[0] = self.seed
            t[1] = 0
        self.call_id = 0

    def tensor(self, device) -> torch.Tensor:
        key = str(device)
        if key not in self._state:
            self._state[key] = torch.tensor([self.seed, 0], dtype=torch.int64, device=device)
        return self._state[key]

    def next_call_id(self) -> int:
        self.call_id += 1
        return self.call_id

    def advance_step(self):
        """Moves every device state to the next step and restarts call numbering."""
        for t in self._state.values():
            t[1:2].add_(_STEP_STRIDE)
        self.call_id = 0

    def get_call_id(self) -> int:
        return self.call_id

    def set_call_id(self, v: int):
        self.call_id = int(v)


_state = DropoutState()


def dropout_state() -> DropoutState:
    return _state
