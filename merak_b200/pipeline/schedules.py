"""Pipeline instruction set and the schedule generators that emit it.

A schedule is, per stage, a list of *steps*; a step is a list of instructions the engine runs in
order.  The base timeline is the classic one-forward-one-backward ("1F1B") slot sequence: stage
``s`` of ``S`` alternates forward and backward slots, ``2*(M+S-1)`` slots for ``M`` micro-batches,
most of them empty during warm-up / cool-down.  Each schedule is then a *policy* over that
timeline: which communication instruction precedes a slot, whether neighbouring send/recv pairs
are merged into one batched p2p call, and whether a forward runs as an early-recompute
("pre-checkpoint") forward whose recomputation is overlapped with the wait for the gradient.

Same instruction names, buffer numbering and emitted streams as the reference
(Merak/core/pipeline/exec_schedule.py:48-360, Merak/core/pipeline/schedule.py:22-613), so
engine logs and schedule-level tests are interchangeable.
"""
from __future__ import annotations

from typing import Iterator, List, Optional, Tuple


# ---------------------------------------------------------------------------------------------
# instructions
# ---------------------------------------------------------------------------------------------
class PipeInstruction:
    """Base class: an instruction is a name plus keyword arguments."""

    __slots__ = ("kwargs",)

    def __init__(self, **kwargs):
        self.kwargs = kwargs

    @property
    def name(self) -> str:
        return type(self).__name__

    def __getattr__(self, item):
        try:
            return self.kwargs[item]
        except KeyError:
            raise AttributeError(item)

    def __repr__(self):
        args = ", ".join("%s=%r" % kv for kv in self.kwargs.items())
        return "%s(%s)" % (self.name, args)

    def __eq__(self, other):
        return type(self) is type(other) and self.kwargs == other.kwargs

    def __hash__(self):
        return hash((self.name, tuple(sorted(self.kwargs.items()))))


class OptimizerStep(PipeInstruction):
    """Apply the optimizer (after every gradient reduction has been issued)."""


class ReduceGrads(PipeInstruction):
    """Reduce gradients over the data-parallel group."""


class ReduceTiedGrads(PipeInstruction):
    """Reduce gradients of parameters shared between stages (tied embeddings)."""


class BufferOpInstruction(PipeInstruction):
    """Instruction that works on one pipeline buffer slot."""

    def __init__(self, buffer_id, **kwargs):
        super().__init__(buffer_id=buffer_id, **kwargs)


class LoadMicroBatch(BufferOpInstruction):
    pass


class ForwardPass(BufferOpInstruction):
    pass


class BackwardPass(BufferOpInstruction):
    pass


class SendActivation(BufferOpInstruction):
    pass


class RecvActivation(BufferOpInstruction):
    pass


class SendGrad(BufferOpInstruction):
    pass


class RecvGrad(BufferOpInstruction):
    pass


class SendActivationRecvGrad(BufferOpInstruction):
    """One batched p2p call; ``buffer_id`` is ``(send_buffer, recv_buffer)``."""


class SendGradRecvActivation(BufferOpInstruction):
    """One batched p2p call; ``buffer_id`` is ``(send_buffer, recv_buffer)``."""


class PreCheckpointForwardPass(BufferOpInstruction):
    """Forward without autograd graph whose recomputation may be started early."""


class RecomputeRecvGrad(BufferOpInstruction):
    """Re-run the stage forward with grad for this buffer, then receive its output gradient."""


class RestoreRecomputeStatus(PipeInstruction):
    """Put the module's recompute configuration back after early-recompute instructions."""


_SHORT = {
    "LoadMicroBatch": "L", "ForwardPass": "F", "BackwardPass": "B", "SendActivation": "SA",
    "RecvActivation": "RA", "SendGrad": "SG", "RecvGrad": "RG", "SendActivationRecvGrad": "SARG",
    "SendGradRecvActivation": "SGRA", "PreCheckpointForwardPass": "PF", "RecomputeRecvGrad": "RRG",
    "RestoreRecomputeStatus": "RS", "ReduceTiedGrads": "RT", "ReduceGrads": "RD", "OptimizerStep": "OPT",
}


def format_steps(steps) -> str:
    """Compact text form ``L0+F0 | SA0 | ...`` (empty steps omitted), used by tests and logs."""
    out = []
    for cmds in steps:
        if not cmds:
            continue
        parts = []
        for c in cmds:
            s = _SHORT[c.name]
            b = c.kwargs.get("buffer_id")
            if isinstance(b, tuple):
                s += "%d>%d" % b
            elif b is not None:
                s += str(b)
            parts.append(s)
        out.append("+".join(parts))
    return " | ".join(out)


# ---------------------------------------------------------------------------------------------
# schedules
# ---------------------------------------------------------------------------------------------
class PipeSchedule:
    """Generates the instruction steps of one stage for one batch of ``micro_batches``."""

    def __init__(self, micro_batches: int, stages: int, stage_id: int):
        self.micro_batches = micro_batches
        self.stages = stages
        self.stage_id = stage_id
        self.prev_stage = stage_id - 1
        self.next_stage = stage_id + 1

    def steps(self) -> Iterator[List[PipeInstruction]]:
        raise NotImplementedError

    def num_pipe_buffers(self) -> int:
        return self.micro_batches

    def __iter__(self):
        return iter(self.steps())

    # helpers ---------------------------------------------------------------------------------
    @property
    def is_first_stage(self):
        return self.stage_id == 0

    @property
    def is_last_stage(self):
        return self.stage_id == self.stages - 1

    @property
    def stage(self):
        return self.stage_id

    @property
    def num_stages(self):
        return self.stages

    @property
    def num_micro_batches(self):
        return self.micro_batches

    def _valid_micro_batch(self, mb: int) -> bool:
        return 0 <= mb < self.micro_batches

    def _valid_stage(self, stage: int) -> bool:
        return 0 <= stage < self.stages

    def _buffer_idx(self, mb: int) -> int:
        assert self._valid_micro_batch(mb)
        return mb % self.num_pipe_buffers()


class InferenceSchedule(PipeSchedule):
    """Forward-only pipelining with two alternating buffers; even and odd stages order their
    send/recv oppositely so neighbouring blocking calls pair up."""

    def steps(self):
        total = self.micro_batches + self.stages - 1
        for step in range(total):
            mb = step - self.stage_id
            recv_buf, send_buf = (step % 2, (step + 1) % 2) if self.stage_id % 2 == 0 else ((step + 1) % 2, step % 2)
            cmds = []
            if (self.is_first_stage or self.is_last_stage) and self._valid_micro_batch(mb):
                cmds.append(LoadMicroBatch(recv_buf))
            send = self._valid_stage(self.next_stage) and self._valid_micro_batch(mb - 1)
            recv = self._valid_stage(self.prev_stage) and self._valid_micro_batch(mb)
            if self.stage_id % 2 == 0:
                if send:
                    cmds.append(SendActivation(send_buf))
                if recv:
                    cmds.append(RecvActivation(recv_buf))
            else:
                if recv:
                    cmds.append(RecvActivation(recv_buf))
                if send:
                    cmds.append(SendActivation(send_buf))
            if self._valid_micro_batch(mb):
                cmds.append(ForwardPass(recv_buf))
            yield cmds

    def num_pipe_buffers(self):
        return 2


def _slot(stage_id: int, stages: int, step: int) -> Tuple[int, bool]:
    """Micro-batch index (possibly out of range) and direction of slot ``step`` on ``stage_id``.

    Even stages run forwards on even steps, odd stages on odd steps; a backward of micro-batch
    ``m`` on stage ``s`` comes ``2*(S-1-s)+1`` slots after its forward.
    """
    forward = (step % 2) == (stage_id % 2)
    if forward:
        base = step // 2 if step % 2 == 0 else (step - 1) // 2
        return base - stage_id // 2, True
    if step % 2 == 0:      # odd stage, even step
        return step // 2 - stages + (stage_id + 1) // 2, False
    return (step - 1) // 2 - stages + 1 + stage_id // 2, False


class TrainSchedule(PipeSchedule):
    """Plain 1F1B with one p2p instruction per transfer (``train_schedule='ds_default'``)."""

    merge_p2p = False

    def total_steps(self) -> int:
        return 2 * (self.micro_batches + self.stages - 1)

    def num_pipe_buffers(self):
        return max(2, min(self.stages - self.stage_id + 1, self.micro_batches))

    # -- policy hooks -------------------------------------------------------------------------
    def _comm(self, is_fwd, mb, prev_mb, cur, prev) -> List[PipeInstruction]:
        has_cur, has_prev = self._valid_micro_batch(mb), self._valid_micro_batch(prev_mb)
        cmds = []
        if is_fwd and self._valid_stage(self.prev_stage):
            if self.merge_p2p:
                if has_cur and has_prev:
                    cmds.append(SendGradRecvActivation((prev, cur)))
                elif has_cur:
                    cmds.append(RecvActivation(cur))
                elif has_prev:
                    cmds.append(SendGrad(prev))
            else:
                if has_cur:
                    cmds.append(RecvActivation(cur))
                if has_prev:
                    cmds.append(SendGrad(prev))
        elif not is_fwd and self._valid_stage(self.next_stage):
            if self.merge_p2p:
                if has_cur and has_prev:
                    cmds.append(SendActivationRecvGrad((prev, cur)))
                elif has_prev:
                    cmds.append(SendActivation(prev))
                elif has_cur:
                    cmds.append(self._recv_grad(cur))
            else:
                if has_prev:
                    cmds.append(SendActivation(prev))
                if has_cur:
                    cmds.append(RecvGrad(cur))
        return cmds

    def _recv_grad(self, buf):
        return RecvGrad(buf)

    def _forward(self, mb, buf) -> List[PipeInstruction]:
        return [ForwardPass(buf)]

    def _tail(self) -> List[PipeInstruction]:
        return [ReduceTiedGrads(), ReduceGrads(), OptimizerStep()]

    # -- generator ----------------------------------------------------------------------------
    def steps(self):
        prev_mb = -1
        total = self.total_steps()
        for step in range(total):
            mb, is_fwd = _slot(self.stage_id, self.stages, step)
            cur = self._buffer_idx(mb) if self._valid_micro_batch(mb) else None
            prev = self._buffer_idx(prev_mb) if self._valid_micro_batch(prev_mb) else None
            cmds = self._comm(is_fwd, mb, prev_mb, cur, prev)
            if (self.is_first_stage or self.is_last_stage) and is_fwd and cur is not None:
                cmds.append(LoadMicroBatch(cur))
            if cur is not None:
                cmds.extend(self._forward(mb, cur) if is_fwd else [BackwardPass(cur)])
            if step == total - 1:
                cmds.extend(self._tail())
            prev_mb = mb
            yield cmds


class MergeP2PTrainSchedule(TrainSchedule):
    """1F1B with neighbouring send/recv pairs merged into one batched call (``'1f1b'``, default)."""

    merge_p2p = True


class PreRecomputeTrainSchedule(MergeP2PTrainSchedule):
    """``'pre_recompute_1f1b'``: the cool-down micro-batches of every stage run as pre-checkpoint
    forwards and are recomputed while the stage waits for their gradient."""

    def _is_cooldown_forward(self, mb) -> bool:
        return self.micro_batches - mb + self.stage_id < self.stages

    def _recv_grad(self, buf):
        return RecomputeRecvGrad(buf)

    def _forward(self, mb, buf):
        if self._is_cooldown_forward(mb):
            return [PreCheckpointForwardPass(buf)]
        return [ForwardPass(buf)]

    def _tail(self):
        head = [RestoreRecomputeStatus()] if self.stage_id < self.stages - 1 else []
        return head + super()._tail()


class LastNoRecomputeTrainSchedule(PreRecomputeTrainSchedule):
    """``'last_no_recompute_1f1b'``: the last stage keeps its activations (no recompute at all), the
    stage before it recomputes only its first micro-batch early and un-merges its first p2p pair."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self._first_pair = True
        self._first_fwd = True

    def _recv_grad(self, buf):
        return RecvGrad(buf) if self.stage_id == self.stages - 2 else RecomputeRecvGrad(buf)

    def _comm(self, is_fwd, mb, prev_mb, cur, prev):
        has_cur, has_prev = self._valid_micro_batch(mb), self._valid_micro_batch(prev_mb)
        if has_cur and has_prev and self._first_pair:
            if is_fwd and self.is_last_stage and self._valid_stage(self.prev_stage):
                self._first_pair = False
                return [SendGrad(prev), RecvActivation(cur)]
            if not is_fwd and self.stage_id == self.stages - 2 and self._valid_stage(self.next_stage):
                self._first_pair = False
                return [RecomputeRecvGrad(cur), SendActivation(prev), RestoreRecomputeStatus()]
        return super()._comm(is_fwd, mb, prev_mb, cur, prev)

    def _forward(self, mb, buf):
        if self.stage_id == self.stages - 2:
            if self._first_fwd:
                self._first_fwd = False
                return [PreCheckpointForwardPass(buf), RestoreRecomputeStatus()]
            return [ForwardPass(buf)]
        return super()._forward(mb, buf)

    def steps(self):
        self._first_pair = True
        self._first_fwd = True
        return super().steps()


class FullCriticalPathTrainSchedule(TrainSchedule):
    """``'full_critical_path_1f1b'`` / ``'shifted_critical_path'``.

    The stage before the last runs its third forward *before* its first backward, which moves the
    critical path of the whole pipeline one slot earlier; the two stages around it un-merge the
    affected p2p pairs and recompute early so the shifted transfers still pair up.  Needs
    ``micro_batches >= max(4, stages)``.
    """

    merge_p2p = True

    def steps(self):
        S, s = self.stages, self.stage_id
        pairs_seen = 0            # merged-pair opportunities consumed by special handling
        fwd_seen = 0              # forwards seen on stages S-2 / S-3
        swap_state = 0            # 0: first backward not met, 1: F2 emitted in its place, 2: B0 emitted
        first_pair, second_pair = True, True
        b0 = self._buffer_idx(0)
        f2 = self._buffer_idx(2)
        prev_mb = -1
        total = self.total_steps()
        for step in range(total):
            mb, is_fwd = _slot(s, S, step)
            has_cur, has_prev = self._valid_micro_batch(mb), self._valid_micro_batch(prev_mb)
            cur = self._buffer_idx(mb) if has_cur else None
            prev = self._buffer_idx(prev_mb) if has_prev else None
            cmds: List[PipeInstruction] = []

            # ---- communication ----
            if is_fwd:
                if has_cur and self._valid_stage(self.prev_stage):
                    if has_prev:
                        if s == S - 1 and (first_pair or second_pair):
                            if first_pair:
                                first_pair = False
                            else:
                                second_pair = False
                            cmds += [SendGrad(prev), RecvActivation(cur)]
                        elif s == S - 2 and first_pair:
                            first_pair = False
                            cmds += [RecomputeRecvGrad(b0), SendActivation(f2 - 1), RestoreRecomputeStatus()]
                        else:
                            cmds.append(SendGradRecvActivation((prev, cur)))
                    else:
                        cmds.append(RecvActivation(cur))
                elif has_prev and self._valid_stage(self.prev_stage):
                    cmds.append(SendGrad(prev))
                elif first_pair and S == 2 and has_cur and s == 0 and has_prev:
                    first_pair = False
                    cmds += [RecomputeRecvGrad(b0), SendActivation(f2 - 1), RestoreRecomputeStatus()]
            else:
                if has_prev and self._valid_stage(self.next_stage):
                    if has_cur:
                        if s == S - 2 and first_pair:
                            cmds.append(RecvActivation(f2))
                        elif s == S - 2 and second_pair:
                            second_pair = False
                            cmds += [SendGrad(b0), RecomputeRecvGrad(cur), SendActivation(f2), RestoreRecomputeStatus()]
                        elif s == S - 3 and first_pair:
                            first_pair = False
                            cmds += [SendActivation(prev), RecomputeRecvGrad(cur), RestoreRecomputeStatus()]
                        else:
                            cmds.append(SendActivationRecvGrad((prev, cur)))
                    else:
                        cmds.append(SendActivation(prev))
                elif has_cur and self._valid_stage(self.next_stage):
                    cmds.append(RecvGrad(cur) if s == S - 2 else RecomputeRecvGrad(cur))

            # ---- data ----
            if (self.is_first_stage or self.is_last_stage) and is_fwd and has_cur:
                cmds.append(LoadMicroBatch(cur))

            # ---- compute ----
            if has_cur:
                if is_fwd:
                    cooldown = self.micro_batches - mb + s < S
                    if cooldown and s != S - 2:
                        cmds.append(PreCheckpointForwardPass(cur))
                    elif s == S - 2 and fwd_seen < 2:
                        fwd_seen += 1
                        cmds += [PreCheckpointForwardPass(cur), RestoreRecomputeStatus()]
                    elif s == S - 2 and swap_state == 1:
                        swap_state = 2       # the slot of the third forward now runs the first backward
                        if cmds and isinstance(cmds[-1], LoadMicroBatch):
                            cmds[-1] = BackwardPass(b0)
                        else:
                            cmds.append(BackwardPass(b0))
                    elif s == S - 3 and fwd_seen < 1:
                        fwd_seen += 1
                        cmds += [PreCheckpointForwardPass(cur), RestoreRecomputeStatus()]
                    else:
                        cmds.append(ForwardPass(cur))
                else:
                    if s == S - 2 and swap_state == 0:
                        swap_state = 1       # the slot of the first backward runs the third forward
                        if s == 0:
                            cmds.append(LoadMicroBatch(f2))
                        cmds.append(ForwardPass(f2))
                    else:
                        cmds.append(BackwardPass(cur))

            if step == total - 1:
                if s < S - 1:
                    cmds.append(RestoreRecomputeStatus())
                cmds += [ReduceTiedGrads(), ReduceGrads(), OptimizerStep()]
            prev_mb = mb
            yield cmds


class DataParallelSchedule(PipeSchedule):
    """Gradient accumulation without pipelining (single stage)."""

    def steps(self):
        for mb in range(self.micro_batches):
            cmds = [LoadMicroBatch(0), ForwardPass(0), BackwardPass(0)]
            if mb == self.micro_batches - 1:
                cmds += [ReduceGrads(), OptimizerStep()]
            yield cmds

    def num_pipe_buffers(self):
        return 1


SCHEDULES = {
    "1f1b": MergeP2PTrainSchedule,
    "ds_default": TrainSchedule,
    "pre_recompute_1f1b": PreRecomputeTrainSchedule,
    "last_no_recompute_1f1b": LastNoRecomputeTrainSchedule,
    "full_critical_path_1f1b": FullCriticalPathTrainSchedule,
    "shifted_critical_path": FullCriticalPathTrainSchedule,
}


def make_schedule(name: str, micro_batches: int, stages: int, stage_id: int) -> PipeSchedule:
    if name not in SCHEDULES:
        raise ValueError("unknown train_schedule %r (known: %s)" % (name, ", ".join(sorted(SCHEDULES))))
    if name in ("full_critical_path_1f1b", "shifted_critical_path"):
        if micro_batches < 4 or micro_batches < stages:
            raise ValueError("shifted critical path needs micro_batches >= max(4, stages)")
    return SCHEDULES[name](micro_batches, stages, stage_id)
