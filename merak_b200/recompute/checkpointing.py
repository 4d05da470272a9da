"""Activation recomputation with reproducible randomness.

* ``checkpoint(fn, *args)``: run ``fn`` without building a graph, keep only its inputs and the RNG
  state; the backward pass re-runs ``fn`` under that state and differentiates it
  (Merak/core/recompute/checkpointing.py:308-483).
* ``pre_checkpoint(fn, *args)``: same forward, but the re-run can be triggered *early* through
  ``run_pending_recomputes()`` - the pipeline engine does that while a stage waits for the gradient
  of its output, which is what the pre-recompute and shifted-critical-path schedules exploit
  (Merak/core/recompute/checkpointing.py:486-606).
* ``RNGStatesTracker`` / ``model_parallel_manual_seed``: named generator states so that dropout
  differs across tensor-parallel ranks inside TP regions and agrees outside
  (Merak/core/recompute/checkpointing.py:106-251).  Seeds follow the same formula:
  tracker seed = ``seed + 2718 + tp_size * sp_rank + tp_rank``.
* ``RNGManager``: per-pipeline-buffer snapshots of the RNG state taken at forward time and restored
  for an early recompute (Merak/core/recompute/checkpointing.py:609-651).

The framework's own dropout kernels draw from a counter-based generator; its per-step call
counter is part of the captured state, so recomputed forwards regenerate identical masks.
"""
from __future__ import annotations

import contextlib
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..ops.rng import dropout_state
from ..parallel import mpu

_MODEL_PARALLEL_RNG = "model-parallel-rng"


def _get_rng_snapshot(device_type: str):
    snap = {"cpu": torch.get_rng_state(), "call_id": dropout_state().get_call_id(),
            "tracker": get_rng_tracker().get_states()}
    if device_type == "cuda" and torch.cuda.is_available():
        snap["cuda"] = torch.cuda.get_rng_state()
    return snap


def _set_rng_snapshot(snap):
    torch.set_rng_state(snap["cpu"])
    dropout_state().set_call_id(snap["call_id"])
    get_rng_tracker().set_states(snap["tracker"])
    if "cuda" in snap:
        torch.cuda.set_rng_state(snap["cuda"])


class RNGStatesTracker:
    """Named generator states; ``fork(name)`` runs a region under the named state and saves the
    advanced state back."""

    def __init__(self):
        self.states_: Dict[str, Any] = {}
        self.seeds_ = set()

    def reset(self):
        self.states_, self.seeds_ = {}, set()

    def get_states(self):
        return dict(self.states_)

    def set_states(self, states):
        self.states_ = dict(states)

    def add(self, name: str, seed: int):
        if seed in self.seeds_:
            raise RuntimeError("seed %d already present" % seed)
        if name in self.states_:
            raise RuntimeError("rng state %s already present" % name)
        self.seeds_.add(seed)
        if torch.cuda.is_available():
            orig = torch.cuda.get_rng_state()
            torch.cuda.manual_seed(seed)
            self.states_[name] = torch.cuda.get_rng_state()
            torch.cuda.set_rng_state(orig)
        else:
            orig = torch.get_rng_state()
            torch.manual_seed(seed)
            self.states_[name] = torch.get_rng_state()
            torch.set_rng_state(orig)

    @contextlib.contextmanager
    def fork(self, name: str = _MODEL_PARALLEL_RNG):
        if name not in self.states_:
            raise RuntimeError("rng state %s was not added" % name)
        cuda = torch.cuda.is_available()
        orig = torch.cuda.get_rng_state() if cuda else torch.get_rng_state()
        (torch.cuda.set_rng_state if cuda else torch.set_rng_state)(self.states_[name])
        try:
            yield
        finally:
            self.states_[name] = torch.cuda.get_rng_state() if cuda else torch.get_rng_state()
            (torch.cuda.set_rng_state if cuda else torch.set_rng_state)(orig)


_TRACKER = RNGStatesTracker()


def get_rng_tracker() -> RNGStatesTracker:
    return _TRACKER


def model_parallel_manual_seed(seed: int):
    """Default generators get ``seed`` (identical inside a tensor-parallel group); the tracker's
    model-parallel state gets a rank-dependent seed.  The dropout kernels keep the same pair: a
    replicated seed without the tensor-parallel rank (activations every tensor-parallel rank
    holds in full must get one mask) and a sharded seed with it (reference:
    Merak/core/recompute/checkpointing.py:196-251).  Both differ per data-parallel rank, pipeline
    stage and sequence-parallel rank, which hold different samples / layers / tokens."""
    tp_rank, tp_size = mpu.get_model_parallel_rank(), mpu.get_model_parallel_world_size()
    sp_rank = mpu.get_sequence_parallel_rank()
    mp_seed = seed + 2718 + tp_size * sp_rank + tp_rank
    _TRACKER.reset()
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)
    _TRACKER.add(_MODEL_PARALLEL_RNG, mp_seed)
    spread = 7919 * mpu.get_data_parallel_rank() + 104729 * mpu.get_pipe_parallel_rank()
    dropout_state().manual_seed(mp_seed + spread, replicated_seed=seed + 2718 + tp_size * sp_rank + spread + 15485863)
    return mp_seed


def _detach(args):
    out = []
    for a in args:
        if isinstance(a, torch.Tensor):
            d = a.detach()
            d.requires_grad = a.requires_grad
            out.append(d)
        else:
            out.append(a)
    return tuple(out)


def _run_backward(outputs, grads):
    outs, gs = [], []
    if isinstance(outputs, torch.Tensor):
        outputs = (outputs,)
    for o, g in zip(outputs, grads):
        if isinstance(o, torch.Tensor) and o.requires_grad and g is not None:
            outs.append(o)
            gs.append(g)
    if outs:
        torch.autograd.backward(outs, gs)


class CheckpointFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, run_function, holder, *args):
        ctx.run_function = run_function
        ctx.holder = holder
        ctx.rng = _get_rng_snapshot(_device_type(args))
        ctx.tensor_idx = [i for i, a in enumerate(args) if isinstance(a, torch.Tensor)]
        ctx.others = [None if isinstance(a, torch.Tensor) else a for a in args]
        ctx.save_for_backward(*[args[i] for i in ctx.tensor_idx])
        ctx.in_grad = [isinstance(a, torch.Tensor) and a.requires_grad for a in args]
        with torch.no_grad():
            outputs = run_function(*args)
        return outputs

    @staticmethod
    def backward(ctx, *grads):
        args = list(ctx.others)
        for i, t in zip(ctx.tensor_idx, ctx.saved_tensors):
            args[i] = t
        for i, a in enumerate(args):
            if isinstance(a, torch.Tensor):
                d = a.detach()
                d.requires_grad = ctx.in_grad[i]
                args[i] = d
        now = _get_rng_snapshot(_device_type(args))
        _set_rng_snapshot(ctx.rng)
        with torch.enable_grad():
            outputs = ctx.run_function(*args)
        _set_rng_snapshot(now)
        _run_backward(outputs, grads)
        return (None, None) + tuple(a.grad if isinstance(a, torch.Tensor) else None for a in args)


def _device_type(args) -> str:
    for a in args:
        if isinstance(a, torch.Tensor):
            return a.device.type
    return "cpu"


def checkpoint(function: Callable, *args):
    """Checkpoint a segment: activations inside ``function`` are recomputed in the backward pass."""
    return CheckpointFunction.apply(function, None, *args)


# ---------------------------------------------------------------------------------------------
# early ("pre") recompute
# ---------------------------------------------------------------------------------------------
class _PendingRecompute:
    """State shared between a PreCheckpointFunction node and the engine."""

    def __init__(self, run_function, args, rng):
        self.run_function, self.args, self.rng = run_function, args, rng
        self.outputs = None
        self.inputs = None

    def recompute(self):
        if self.outputs is not None:
            return
        args = []
        for a in self.args:
            if isinstance(a, torch.Tensor):
                d = a.detach()
                d.requires_grad = a.requires_grad
                args.append(d)
            else:
                args.append(a)
        now = _get_rng_snapshot(_device_type(args))
        _set_rng_snapshot(self.rng)
        with torch.enable_grad():
            self.outputs = self.run_function(*args)
        _set_rng_snapshot(now)
        self.inputs = args
        self.args = None


_PENDING: List[_PendingRecompute] = []


def pending_recomputes() -> List[_PendingRecompute]:
    return _PENDING


def run_pending_recomputes(records: Optional[List[_PendingRecompute]] = None):
    """Re-runs the forward of every not-yet-recomputed pre-checkpointed segment."""
    for rec in (records if records is not None else list(_PENDING)):
        rec.recompute()


class PreCheckpointFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, run_function, record_list, *args):
        rec = _PendingRecompute(run_function, args, _get_rng_snapshot(_device_type(args)))
        ctx.rec = rec
        ctx.n_args = len(args)
        (record_list if record_list is not None else _PENDING).append(rec)
        with torch.no_grad():
            outputs = run_function(*args)
        return outputs

    @staticmethod
    def backward(ctx, *grads):
        rec = ctx.rec
        rec.recompute()
        _run_backward(rec.outputs, grads)
        in_grads = tuple(a.grad if isinstance(a, torch.Tensor) else None for a in rec.inputs)
        rec.outputs, rec.inputs = None, None
        if rec in _PENDING:
            _PENDING.remove(rec)
        return (None, None) + in_grads


def pre_checkpoint(function: Callable, *args, record_list=None):
    """Like :func:`checkpoint`, but the recomputation can be started before the backward pass via
    :func:`run_pending_recomputes` (``record_list`` collects this call's record)."""
    return PreCheckpointFunction.apply(function, record_list, *args)


class RNGManager:
    """Per-buffer RNG snapshots for schedules that recompute a micro-batch out of order."""

    def __init__(self):
        self.fwd: Dict[int, Any] = {}
        self.saved: Optional[Any] = None

    def store_fwd_rng_state(self, buffer_id: int, device_type: str = "cpu"):
        self.fwd[buffer_id] = _get_rng_snapshot(device_type)

    def set_recompute_rng_state(self, buffer_id: int, device_type: str = "cpu"):
        self.saved = _get_rng_snapshot(device_type)
        if buffer_id in self.fwd:
            _set_rng_snapshot(self.fwd[buffer_id])

    def restore_bwd_rng_state(self, buffer_id: int):
        if self.saved is not None:
            _set_rng_snapshot(self.saved)
            self.saved = None
        self.fwd.pop(buffer_id, None)
