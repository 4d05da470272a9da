"""Device-resident state of the counter-based dropout generator.

A dropout call draws its mask from ``philox(seed, offset + call_id, element)``.  ``seed`` and
``offset`` live in a 2-element int64 tensor on the device so that advancing the step or the
micro-batch (``offset``) is a device-side add, which keeps a captured CUDA graph valid across
replays.  ``call_id`` numbers the dropout call sites inside one micro-batch; activation
recomputation restores it so the replayed forward regenerates identical masks (the role
``RNGStatesTracker`` plays in the reference, Merak/core/recompute/checkpointing.py:106-184).

Two generators are kept, as the reference keeps a default CUDA generator and a model-parallel one
(Merak/core/recompute/checkpointing.py:196-251):

* ``replicated``: the same seed on every rank of a tensor-parallel group.  Dropout on activations
  that every tensor-parallel rank holds in full (after a row-parallel all-reduce, on the embedding
  output) must draw the same mask on all of them, or the replicated residual streams and the
  gradients of replicated parameters drift apart.
* ``sharded``: a seed that depends on the tensor-parallel (and sequence-parallel) rank, for
  dropout on tensors each rank holds a different part of: attention probabilities of the rank's
  own heads, sequence-sharded activations under Megatron-style sequence parallelism.

``offset = step * _STEP_STRIDE + micro_batch * _MICRO_STRIDE``.
"""
from __future__ import annotations

import contextlib

import torch

_STEP_STRIDE = 1 << 20
_MICRO_STRIDE = 1 << 12          # graph replays: 256 micro-batches per step, 4095 call sites each
KINDS = ("replicated", "sharded")


class DropoutState:
    def __init__(self):
        self._state = {}      # (device, kind) -> tensor [seed, offset]
        self.call_id = 0
        self.seeds = {"replicated": 1234, "sharded": 1234}
        self.default_kind = "replicated"
        self.step = 0
        self.micro = 0

    # --- seeds ----------------------------------------------------------------------------------
    @property
    def seed(self) -> int:
        return self.seeds["sharded"]

    def manual_seed(self, seed: int, replicated_seed: int | None = None):
        """``seed`` keys the sharded generator; ``replicated_seed`` (default: the same value) the
        replicated one."""
        self.seeds["sharded"] = int(seed)
        self.seeds["replicated"] = int(seed if replicated_seed is None else replicated_seed)
        self.step, self.micro, self.call_id = 0, 0, 0
        self.default_kind = "replicated"
        self._write_all()

    def _offset(self) -> int:
        return self.step * _STEP_STRIDE + self.micro * _MICRO_STRIDE

    def _write_all(self):
        for (_, kind), t in self._state.items():
            t.copy_(torch.tensor([self.seeds[kind], self._offset()], dtype=torch.int64))

    def tensor(self, device, sharded: bool | None = None) -> torch.Tensor:
        kind = self.default_kind if sharded is None else ("sharded" if sharded else "replicated")
        key = (str(device), kind)
        if key not in self._state:
            self._state[key] = torch.tensor([self.seeds[kind], self._offset()], dtype=torch.int64, device=device)
        return self._state[key]

    @contextlib.contextmanager
    def sharded_region(self, on: bool = True):
        """Dropout calls inside draw from the rank-dependent generator."""
        prev = self.default_kind
        self.default_kind = "sharded" if on else "replicated"
        try:
            yield
        finally:
            self.default_kind = prev

    # --- masks for the PyTorch fallback paths ---------------------------------------------------
    def host_keep_mask(self, shape, p: float, device, sharded: bool | None = None) -> torch.Tensor:
        """Boolean keep mask for tensors the kernels do not take (CPU, dtypes other than bf16).  Like the
        kernels' masks it is a pure function of (seed of the chosen generator, offset + call id, element
        index), so it does not depend on how much any torch generator was used before, agrees on every rank
        that shares the seed, and a recomputed forward pass regenerates it from the restored call id."""
        kind = self.default_kind if sharded is None else ("sharded" if sharded else "replicated")
        seed, stream = int(self.seeds[kind]), self._offset() + self.next_call_id()
        m = 0xFFFFFFFF

        def mix(x):
            x = x ^ (x >> 16)
            x = (x * 0x85EBCA6B) & m
            x = x ^ (x >> 13)
            x = (x * 0xC2B2AE35) & m
            return x ^ (x >> 16)

        t = lambda v: torch.tensor(int(v) & m, dtype=torch.int64, device=device)
        base = mix(t(seed) ^ mix((t(seed >> 32) + 0x9E3779B9) & m) ^ mix(((t(stream) * 0x9E3779B1) + t(stream >> 32)) & m))
        n = 1
        for d in shape:
            n *= int(d)
        idx = torch.arange(n, dtype=torch.int64, device=device)
        bits = mix((mix(base ^ (idx & m)) + (idx >> 32) * 0xC2B2AE35) & m)
        thresh = min(int(float(p) * 4294967296.0), m)
        return (bits >= thresh).view(tuple(shape))

    def host_dropout(self, x: torch.Tensor, p: float, sharded: bool | None = None) -> torch.Tensor:
        keep = self.host_keep_mask(x.shape, p, x.device, sharded)
        return x * keep.to(x.dtype) * (1.0 / (1.0 - p))

    # --- call numbering -------------------------------------------------------------------------
    def next_call_id(self) -> int:
        self.call_id += 1
        return self.call_id

    def get_call_id(self) -> int:
        return self.call_id

    def set_call_id(self, v: int):
        self.call_id = int(v)

    # --- advancing ------------------------------------------------------------------------------
    def advance_micro(self):
        """Next micro-batch of the same step: a device-side add, legal between graph replays.  Only
        the graph path uses it (a replay bakes its call ids in); the eager schedules keep one
        offset per step and let ``call_id`` run on across micro-batches, because a recomputation
        must find the offset its forward pass saw."""
        self.micro += 1
        for t in self._state.values():
            t[1:2].add_(_MICRO_STRIDE)

    def advance_step(self):
        """Moves every device state to the next step and restarts micro-batch and call numbering."""
        delta = _STEP_STRIDE - self.micro * _MICRO_STRIDE
        self.step += 1
        self.micro = 0
        for t in self._state.values():
            t[1:2].add_(delta)
        self.call_id = 0

    # --- persistence ----------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"seed": self.seeds["sharded"], "replicated_seed": self.seeds["replicated"], "step": self.step}

    def load_state_dict(self, sd: dict):
        self.seeds["sharded"] = int(sd["seed"])
        self.seeds["replicated"] = int(sd.get("replicated_seed", sd["seed"]))
        self.step, self.micro, self.call_id = int(sd.get("step", 0)), 0, 0
        self._write_all()


_state = DropoutState()


def dropout_state() -> DropoutState:
    return _state
