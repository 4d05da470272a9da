"""fp32 master weights, loss-scale aware stepping and ZeRO-1 sharding around a user's
``torch.optim`` optimizer.

The reference offers three wrappers for an optimizer the user brings: ``FP16_Optimizer`` (fp32
master copies + loss scaling, Merak/core/amp/fp16_optimizer.py:36-358), the bf16 path that keeps
no master copy at all (Merak/core/amp/amp_engine.py:99-100) and ``ZeroOptimizer_Stage1`` (flatten
every parameter group, pad, split over the data-parallel group, fp32 master of the local
sub-partitions, reduce-scatter / step / all-gather, Merak/core/zero/stage1.py:90-757).  Here one
class does all of it on the engine's flat buffers:

* the parameters of all groups are re-homed, group after group, into one flat model buffer with one
  flat fp32 gradient buffer (``ops.optim.FlatBuffers``);
* this rank owns the slice ``[start, end)`` of them (the whole buffer without ZeRO, ``1/dp`` of it
  with ZeRO-1); one fp32 ``master`` tensor mirrors that slice, and every parameter of the inner
  optimizer is replaced by the view of ``master`` that holds its owned part, so the inner
  optimizer's state (moments, momentum buffers...) exists for the owned slice only;
* ``step`` unscales and clips on the device, hands fp32 gradients to the inner optimizer, and
  writes the updated master values back into the low-precision model buffer.

The class exposes the interface the engine uses for its own fused AdamW (``grad_sumsq``,
``step(grad_scale, sumsq)``, ``skipped``, ``start`` / ``end`` / ``master`` / ``flat``), so the
data-parallel reduce-scatter, the tensor-/pipeline-aware gradient norm, the parameter all-gather
and the ZeRO checkpoint files are shared with that path.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from ..ops.optim import FlatBuffers

# Optimizers whose update is element-wise, so that running them on a slice of a flattened group is
# exact (Merak/core/zero/stage1.py:42-51).
ZERO_SUPPORTED_OPTIMIZERS = ("Adam", "AdamW", "SGD", "ASGD", "Adadelta", "Adamax", "Adagrad", "RMSprop", "NAdam",
                             "RAdam")


def is_zero_supported_optimizer(optimizer) -> bool:
    return type(optimizer).__name__ in ZERO_SUPPORTED_OPTIMIZERS


class ShardedMasterOptimizer:
    """Wraps ``inner`` (a ``torch.optim.Optimizer`` built on the model's parameters)."""

    def __init__(self, inner: torch.optim.Optimizer, dp_rank: int = 0, dp_size: int = 1, shard: bool = False,
                 max_grad_norm: float = 0.0, allow_untested: bool = False, pad_to: Optional[int] = None):
        if shard and dp_size > 1 and not (allow_untested or is_zero_supported_optimizer(inner)):
            raise ValueError("%s is not on the list of optimizers known to be exact on a flattened shard %s; "
                             "pass zero_allow_untested_optimizer to use it anyway"
                             % (type(inner).__name__, list(ZERO_SUPPORTED_OPTIMIZERS)))
        if any(len(st) for st in inner.state.values()):
            raise ValueError("wrap the optimizer before its first step: existing per-parameter state cannot be "
                             "re-sharded")
        self.optimizer = inner
        self.max_grad_norm = float(max_grad_norm or 0.0)
        groups: List[List[torch.nn.Parameter]] = []
        seen = set()
        for g in inner.param_groups:
            ps = [p for p in g["params"] if p.requires_grad and id(p) not in seen]
            seen.update(id(p) for p in ps)
            groups.append(ps)
        params = [p for ps in groups for p in ps]
        if not params:
            raise ValueError("optimizer has no trainable parameters")
        n_shards = dp_size if (shard and dp_size > 1) else 1
        self.flat = FlatBuffers(params, grad_dtype=torch.float32, pad_to=pad_to or 64 * n_shards)
        per = self.flat.numel // n_shards
        self.start, self.end = (dp_rank * per, (dp_rank + 1) * per) if n_shards > 1 else (0, self.flat.numel)
        dev = self.flat.model.device
        self.master = self.flat.model[self.start:self.end].float().clone()
        # every parameter's owned part becomes a view of ``master`` (with the parameter's own shape when
        # the whole of it is owned, so optimizers that look at shapes -- LAMB's per-tensor trust ratio,
        # Adafactor's factored moments -- see what they would see without the wrapper)
        self._views: List[Tuple[torch.Tensor, int, int, Optional[torch.Size]]] = []
        offset_of = {id(p): o for p, o in zip(self.flat.params, self.flat.offsets)}
        for g, ps in zip(inner.param_groups, groups):
            new_params = []
            for p in ps:
                o = offset_of[id(p)]
                s, e = max(o, self.start), min(o + p.numel(), self.end)
                if s >= e:
                    continue
                whole = (s == o and e == o + p.numel())
                view = self.master[s - self.start:e - self.start]
                if whole:
                    view = view.view(p.shape)
                view = view.detach().requires_grad_(True)
                self._views.append((view, s, e, p.shape if whole else None))
                new_params.append(view)
            g["params"] = new_params
        self._sumsq = torch.zeros(2, dtype=torch.float32, device=dev)
        self._skip = torch.zeros(1, dtype=torch.int32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.step_count = 0
        self.overflow = False

    # -- the engine-facing interface -----------------------------------------------------------------
    @property
    def param_groups(self):
        return self.optimizer.param_groups

    @property
    def state(self):
        return self.optimizer.state

    @torch.no_grad()
    def grad_sumsq(self) -> torch.Tensor:
        g = self.flat.grad[self.start:self.end].float()
        self._sumsq[0] = (g * g).sum()
        self._sumsq[1] = (~torch.isfinite(g)).sum()
        return self._sumsq

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, sumsq: Optional[torch.Tensor] = None):
        """``grad_scale`` multiplies the gradients first (1 / loss scale, 1 / dp); ``sumsq`` is the
        squared norm and non-finite count of the whole model when the caller already reduced them
        over the other ranks.  A non-finite norm skips the update (``skipped()`` is then 1)."""
        if sumsq is None:
            sumsq = self.grad_sumsq()
        ss, bad = [float(v) for v in sumsq.tolist()]        # the one host read of this step
        norm = math.sqrt(ss) * grad_scale if ss == ss and ss >= 0 else float("nan")
        self.overflow = (not math.isfinite(norm)) or bad != 0
        self._norm[0] = norm
        self._skip[0] = int(self.overflow)
        if self.overflow:
            return False
        scale = grad_scale
        if self.max_grad_norm > 0 and norm > self.max_grad_norm:
            scale *= self.max_grad_norm / (norm + 1e-6)
        for view, lo, hi, shape in self._views:
            g = self.flat.grad[lo:hi].float() * scale
            view.grad = g.view(shape) if shape is not None else g
        self.optimizer.step()
        self.step_count += 1
        self.flat.model[self.start:self.end].copy_(self.master)
        for view, _, _, _ in self._views:
            view.grad = None
        return True

    def grad_norm(self) -> torch.Tensor:
        return self._norm

    def skipped(self) -> torch.Tensor:
        return self._skip

    def zero_grad(self, set_to_none: bool = True):
        self.flat.zero_grad()

    # -- persistence (keys of Merak/core/zero/stage1.py:819-843 where they apply) -----------------
    def state_dict(self):
        return {"base_optimizer_state": self.optimizer.state_dict(),
                "local_sub_partitions_of_fp32_groups": [self.master],
                "shard": (self.start, self.end), "step": self.step_count, "overflow": self.overflow}

    def load_state_dict(self, sd):
        if tuple(sd["shard"]) != (self.start, self.end):
            raise ValueError("optimizer shard %s of the checkpoint does not match this rank's %s (the data-parallel "
                             "degree must not change between save and load)" % (tuple(sd["shard"]), (self.start, self.end)))
        self.optimizer.load_state_dict(sd["base_optimizer_state"])
        self.master.copy_(sd["local_sub_partitions_of_fp32_groups"][0])
        self.step_count = sd.get("step", 0)
        self.flat.model[self.start:self.end].copy_(self.master)


def configure_zero_optimizer(optimizer: torch.optim.Optimizer, args=None, dp_rank: Optional[int] = None,
                             dp_size: Optional[int] = None) -> ShardedMasterOptimizer:
    """ZeRO-1 wrapper for a user optimizer (Merak/core/zero/stage1.py:53-75)."""
    from ..parallel import mpu
    dp_rank = mpu.get_data_parallel_rank() if dp_rank is None else dp_rank
    dp_size = mpu.get_data_parallel_world_size() if dp_size is None else dp_size
    return ShardedMasterOptimizer(optimizer, dp_rank=dp_rank, dp_size=dp_size, shard=True,
                                  max_grad_norm=getattr(args, "max_grad_norm", 0.0) or 0.0,
                                  allow_untested=bool(getattr(args, "zero_allow_untested_optimizer", False)))
