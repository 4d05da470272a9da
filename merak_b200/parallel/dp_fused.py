"""Fused data-parallel optimizer step over symmetric memory.

The flat bf16 model buffer and the flat fp32 gradient buffer of every data-parallel rank live in
peer-mapped memory.  One step is two kernels (``csrc/fused_comm.cu``):

1. reduce-scatter: each rank sums its shard of the gradient out of all ranks' buffers and posts the
   shard's squared norm to everyone.  With the reduction overlapped with the backward pass, the
   pieces of the gradient buffer travel to their owner's staging buffer on the copy engines as soon
   as the backward pass has finished them, and this kernel sums local memory only;
2. clip + AdamW on the shard (optimizer state sharded as in ZeRO-1) + all-gather: the owner stores
   the new bf16 parameters into every rank's model buffer.

That is the work of the reference's bucketed all-reduce, gradient clipping, optimizer step and
ZeRO-1 all-gather (Merak/core/merak_engine.py:552-621, 930-990; Merak/core/zero/stage1.py:476-757)
with the gradients crossing NVLink once and the parameters once.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..ops import _lib
from .symm import SymmGroup

FLAG_DECAY, FLAG_NO_NORM = 1, 2


class FusedDataParallel:
    def __init__(self, symm: SymmGroup):
        self.symm = symm
        self.n, self.rank = symm.n, symm.rank
        self.model_buf = None
        self.grad_buf = None
        self.flags = None
        self._epoch = 0
        self._norm_tmp = None
        self.budget_ms = 20000

    @staticmethod
    def create(group, device: torch.device, args=None) -> Optional["FusedDataParallel"]:
        """Collective over the data-parallel group; None when the fused path cannot be used."""
        if device.type != "cuda" or dist.get_world_size(group) == 1:
            return None
        if args is not None and getattr(args, "comm_mode", "fused") != "fused":
            return None
        sg = SymmGroup.create(group, device)
        return FusedDataParallel(sg) if sg is not None else None

    # FlatBuffers allocator hook: the two flat buffers are symmetric allocations
    def allocator(self, numel: int, dtype: torch.dtype, tag: str) -> torch.Tensor:
        buf = self.symm.alloc(numel * torch.empty(0, dtype=dtype).element_size(), dtype)
        if tag == "model":
            self.model_buf = buf
        elif tag == "grad":
            self.grad_buf = buf
        return buf.tensor[:numel]

    def bind(self, flat, exclude_from_norm=()):
        """Builds the per-granule flag bytes (weight decay / excluded from the norm on this rank)."""
        assert self.model_buf is not None and self.grad_buf is not None, "flat buffers were not allocated here"
        assert flat.numel % (8 * self.n) == 0
        flags = np.zeros(flat.numel // 64 + 1, dtype=np.uint8)
        excluded = {id(p) for p in exclude_from_norm}
        for p, o in zip(flat.params, flat.offsets):
            lo, hi = o // 64, (o + p.numel() + 63) // 64
            bits = 0
            if getattr(p, "_no_weight_decay", False) is False and p.dim() > 1:
                bits |= FLAG_DECAY
            if id(p) in excluded:
                bits |= FLAG_NO_NORM
            flags[lo:hi] = bits
        self.flags = torch.from_numpy(flags).to(flat.model.device)
        self.per = flat.numel // self.n
        self.lo = self.rank * self.per
        self._norm_tmp = torch.zeros(2, dtype=torch.float32, device=flat.model.device)

        self.stage_buf = None
        self._staged_table = None

    @property
    def shard(self):
        return self.lo, self.lo + self.per

    # -- reduction overlapped with the backward pass ------------------------------------------------
    def enable_staging(self):
        """Collective over the group: a staging buffer of ``n`` slots of one shard each.  Slot ``s`` of
        rank ``r`` receives rank ``s``'s contribution to ``r``'s shard of the gradient."""
        if self.stage_buf is None:
            self.stage_buf = self.symm.alloc(self.n * self.per * 4, torch.float32)
            # pointer table for the summing kernel, which reads ``table[k] + lo + i``: its own gradient
            # buffer for k == rank, staging slot k (local memory) for the others
            own = self.grad_buf.ptrs[self.rank]
            base = self.stage_buf.local_ptr
            self._staged_table = (ctypes.c_void_p * self.n)(*[
                own if k == self.rank else base + 4 * (k * self.per - self.lo) for k in range(self.n)])

    def push_region(self, reg_lo: int, reg_hi: int):
        """The piece ``[reg_lo, reg_hi)`` of the flat gradient buffer is final on this rank: copy the
        parts other ranks own into their staging buffers (copy engines over NVLink, current
        stream; no thread block is involved, so the backward pass keeps every SM)."""
        lib = _lib.kernels()
        st = _lib.stream_ptr()
        src = self.grad_buf.ptrs[self.rank]
        for r in range(self.n):
            a, b = max(int(reg_lo), r * self.per), min(int(reg_hi), (r + 1) * self.per)
            if r == self.rank or a >= b:
                continue
            dst = self.stage_buf.ptrs[r] + 4 * (self.rank * self.per + a - r * self.per)
            _lib.check(lib.mrk_memcpy_d2d_async(dst, src + 4 * a, 4 * (b - a), st), "mrk_memcpy_d2d_async")

    def reduce_scatter(self, staged: bool = False):
        """Kernel 1 on the current stream.  ``staged``: every rank has pushed its contributions into
        the staging buffers (``push_region``), so the sum reads local memory only; the kernel's
        barrier then means "every rank's pushes have landed"."""
        self._epoch += 1
        table = self._staged_table if staged else self.grad_buf.table
        _lib.check(_lib.kernels().mrk_dp_reduce_scatter(
            table, self.symm.ctrl.table, self.n, self.rank, self.lo, self.per,
            self.flags.data_ptr(), self._epoch, 1, self.budget_ms, _lib.stream_ptr()), "mrk_dp_reduce_scatter")

    def gathered_sumsq(self) -> torch.Tensor:
        """[sum of squares, non-finite count] of the whole (data-parallel reduced) gradient of this
        model replica, for callers that still have to reduce it over other groups."""
        _lib.check(_lib.kernels().mrk_dp_norm_gather(self.symm.ctrl.table, self.n, self.rank,
                                                     self._norm_tmp.data_ptr(), self._epoch, 1, self.budget_ms,
                                                     _lib.stream_ptr()), "mrk_dp_norm_gather")
        return self._norm_tmp

    def adamw_allgather(self, opt, grad_scale: float, sumsq: Optional[torch.Tensor] = None):
        """Kernel 2 on the current stream.  ``opt`` is the FusedAdamW that owns this rank's shard."""
        opt.step_count += 1
        hp = opt._hp_tensor(opt.weight_decay)
        g = opt.flat.grad
        _lib.check(_lib.kernels().mrk_dp_adamw_allgather(
            self.model_buf.table, self.symm.ctrl.table, self.n, self.rank, self.lo, self.per,
            g.data_ptr() + 4 * self.lo, opt.master.data_ptr(), opt.exp_avg.data_ptr(), opt.exp_avg_sq.data_ptr(),
            self.flags.data_ptr(), hp.data_ptr(), float(grad_scale), float(opt.max_grad_norm),
            sumsq.data_ptr() if sumsq is not None else None, opt._norm.data_ptr(), opt._skip.data_ptr(),
            self._epoch, 1, 0 if sumsq is not None else 1, self.budget_ms, _lib.stream_ptr()),
            "mrk_dp_adamw_allgather")
