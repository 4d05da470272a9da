"""Pipeline point-to-point transport between neighbouring stages.

Transfers stay on ``torch.distributed`` p2p (NCCL on GPUs, gloo on CPU) as batched
``isend``/``irecv`` to the previous / next *global* rank, like the reference
(Merak/core/mpu/p2p_communication.py:27-216).  Differences:

* on CUDA the ops are issued on a dedicated communication stream and ordered against the compute
  stream with events, so a transfer overlaps the next compute instruction instead of ending in a
  device-wide ``torch.cuda.synchronize()``;
* the first exchange of a stage pair carries a small host-side metadata message (count, dtype,
  shape, requires_grad per tensor) so receive buffers can be allocated once.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import mpu

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.int32,
           torch.int16, torch.int8, torch.uint8, torch.bool]
_DTYPE_ID = {d: i for i, d in enumerate(_DTYPES)}

_comm_stream = {}


def _stream_for(device) -> Optional["torch.cuda.Stream"]:
    if device is None or torch.device(device).type != "cuda":
        return None
    key = torch.device(device).index
    if key not in _comm_stream:
        _comm_stream[key] = torch.cuda.Stream(device=device)
    return _comm_stream[key]


class Work:
    """Handle of an in-flight batched transfer."""

    def __init__(self, reqs, stream=None, keep=()):
        self.reqs, self.stream, self.keep = reqs, stream, keep
        self.event = None
        if stream is not None:
            self.event = torch.cuda.Event()

    def wait(self):
        for r in self.reqs:
            r.wait()
        if self.stream is not None:
            # NCCL requests complete on the communication stream; make compute wait on it
            self.event.record(self.stream)
            torch.cuda.current_stream().wait_event(self.event)
        self.reqs = []
        self.keep = ()


def _batch(ops: List[dist.P2POp], device, keep=()) -> Work:
    if not ops:
        return Work([])
    stream = _stream_for(device)
    if stream is None:
        return Work(dist.batch_isend_irecv(ops), None, keep)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream())
    stream.wait_event(ev)
    with torch.cuda.stream(stream):
        reqs = dist.batch_isend_irecv(ops)
    for t in keep:
        if t.is_cuda:
            t.record_stream(stream)
    return Work(reqs, stream, keep)


def communicate(send_next: Sequence[torch.Tensor] = (), send_prev: Sequence[torch.Tensor] = (),
                recv_prev: Sequence[torch.Tensor] = (), recv_next: Sequence[torch.Tensor] = (),
                wait: bool = True) -> Work:
    """Posts all given sends/receives as one batch.  Receive lists hold pre-allocated buffers."""
    prev_rank = mpu.get_pipeline_model_parallel_prev_rank()
    next_rank = mpu.get_pipeline_model_parallel_next_rank()
    ops, keep = [], []
    dev = None
    # a shard may hand over a view (a transposed or sliced activation): the wire wants dense memory
    send_prev = [t if t.is_contiguous() else t.contiguous() for t in send_prev]
    send_next = [t if t.is_contiguous() else t.contiguous() for t in send_next]
    # Order: sends toward prev, receives from prev, sends toward next, receives from next - every
    # rank uses the same order so neighbouring batches match up.
    for t in send_prev:
        ops.append(dist.P2POp(dist.isend, t, prev_rank)); keep.append(t); dev = t.device
    for t in recv_prev:
        ops.append(dist.P2POp(dist.irecv, t, prev_rank)); keep.append(t); dev = t.device
    for t in send_next:
        ops.append(dist.P2POp(dist.isend, t, next_rank)); keep.append(t); dev = t.device
    for t in recv_next:
        ops.append(dist.P2POp(dist.irecv, t, next_rank)); keep.append(t); dev = t.device
    work = _batch(ops, dev, tuple(keep))
    if wait:
        work.wait()
    return work


# ---- reference-named wrappers (Merak/core/mpu/p2p_communication.py:106-216) ---------------------
def send_forward(tensors, wait=True):
    if mpu.is_pipeline_last_stage():
        return Work([])
    return communicate(send_next=_as_list(tensors), wait=wait)


def recv_forward(buffers, wait=True):
    if mpu.is_pipeline_first_stage():
        return Work([])
    return communicate(recv_prev=_as_list(buffers), wait=wait)


def send_backward(tensors, wait=True):
    if mpu.is_pipeline_first_stage():
        return Work([])
    return communicate(send_prev=_as_list(tensors), wait=wait)


def recv_backward(buffers, wait=True):
    if mpu.is_pipeline_last_stage():
        return Work([])
    return communicate(recv_next=_as_list(buffers), wait=wait)


def send_forward_recv_backward(tensors, grad_buffers, wait=True):
    if mpu.is_pipeline_last_stage():
        return Work([])
    return communicate(send_next=_as_list(tensors), recv_next=_as_list(grad_buffers), wait=wait)


def send_backward_recv_forward(grads, buffers, wait=True):
    if mpu.is_pipeline_first_stage():
        return Work([])
    return communicate(send_prev=_as_list(grads), recv_prev=_as_list(buffers), wait=wait)


def _as_list(x):
    if x is None:
        return []
    if isinstance(x, torch.Tensor):
        return [x]
    return [t for t in x if t is not None]


# ---- tensor metadata handshake ----------------------------------------------------------------
# Values that are not tensors travel as 0-dim tensors; the second field of their description says what to
# turn them back into on the receiving stage (Python int / float / bool; a ``torch.device`` becomes the
# receiver's own device).
KIND_INT, KIND_FLOAT, KIND_BOOL, KIND_DEVICE = 10, 11, 12, 13


def to_wire(values, device):
    """``(tensors, kinds)``: every value as a tensor that can be sent, and its kind code (0 for tensors)."""
    tensors, kinds = [], []
    for v in values:
        if isinstance(v, torch.Tensor):
            tensors.append(v)
            kinds.append(0)
        elif isinstance(v, bool):
            tensors.append(torch.tensor(v, dtype=torch.bool, device=device))
            kinds.append(KIND_BOOL)
        elif isinstance(v, int):
            tensors.append(torch.tensor(v, dtype=torch.int64, device=device))
            kinds.append(KIND_INT)
        elif isinstance(v, float):
            tensors.append(torch.tensor(v, dtype=torch.float64, device=device))
            kinds.append(KIND_FLOAT)
        elif isinstance(v, torch.device):
            tensors.append(torch.zeros((), dtype=torch.int64, device=device))
            kinds.append(KIND_DEVICE)
        else:
            raise TypeError("a value of type %s cannot travel between pipeline stages" % type(v).__name__)
    return tensors, kinds


def from_wire(tensors, meta, device):
    """Undoes ``to_wire`` on the receiving stage (``meta`` as returned by ``recv_meta``)."""
    out = []
    for t, (_, kind, _) in zip(tensors, meta):
        if kind == KIND_INT:
            out.append(int(t.item()))
        elif kind == KIND_FLOAT:
            out.append(float(t.item()))
        elif kind == KIND_BOOL:
            out.append(bool(t.item()))
        elif kind == KIND_DEVICE:
            out.append(torch.device(device))
        else:
            out.append(t)
    return out


def encode_meta(tensors: Sequence[torch.Tensor], kinds: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Flat int64 description: [count, (dtype_id, requires_grad or kind code, ndim, *shape) ...]."""
    vals = [len(tensors)]
    for i, t in enumerate(tensors):
        flag = kinds[i] if kinds and kinds[i] else int(t.requires_grad or t.is_floating_point())
        vals += [_DTYPE_ID[t.dtype], flag, t.dim(), *t.shape]
    return torch.tensor(vals, dtype=torch.int64)


def decode_meta(meta: torch.Tensor) -> List[Tuple[torch.dtype, bool, Tuple[int, ...]]]:
    vals = meta.tolist()
    n, pos, out = vals[0], 1, []
    for _ in range(n):
        dt, rg, nd = vals[pos], vals[pos + 1], vals[pos + 2]
        shape = tuple(vals[pos + 3: pos + 3 + nd])
        pos += 3 + nd
        out.append((_DTYPES[dt], int(rg), shape))           # 0 / 1: tensor without / with gradient; >= 10: kind code
    return out


_META_MAX = 4096        # int64 words: room for a few hundred tensors crossing one boundary


def send_meta(tensors: Sequence[torch.Tensor], to_rank: int, device, kinds: Optional[Sequence[int]] = None):
    meta = encode_meta(tensors, kinds)
    buf = torch.zeros(_META_MAX, dtype=torch.int64)
    buf[0] = meta.numel()
    buf[1:1 + meta.numel()] = meta
    dist.send(buf.to(device), to_rank)


def recv_meta(from_rank: int, device):
    buf = torch.zeros(_META_MAX, dtype=torch.int64, device=device)
    dist.recv(buf, from_rank)
    buf = buf.cpu()
    n = int(buf[0])
    return decode_meta(buf[1:1 + n])
