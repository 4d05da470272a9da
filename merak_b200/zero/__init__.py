"""ZeRO stage 1 (optimizer-state sharding over the data-parallel group).

The reference ports DeepSpeed's stage-1 optimizer (Merak/core/zero/stage1.py:42-843): flatten each
parameter group, pad to ``dp x sub_partition``, keep fp32 master copies of the local
sub-partitions, reduce-scatter gradients, step, all-gather parameters.  Here the engine already
keeps one flat model buffer and one flat fp32 gradient buffer per stage, so stage 1 is "every dp
rank owns one contiguous ``1/dp`` slice of them": ``reduce_scatter_tensor`` on the gradient buffer,
the fused AdamW on the owned slice (fp32 master + moments exist only for that slice), and one
``all_gather_into_tensor`` of the updated bf16 slice.  ``configure_zero_optimizer`` builds that
optimizer for users who construct engines by hand; ``ZeroOptimizer_Stage1`` is its class.
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.distributed as dist

from ..ops.optim import FlatBuffers, FusedAdamW
from ..parallel import mpu
from ..pipeline.engine import DynamicLossScaler  # re-exported: same loss scaler as the fp16 path

ZERO_SUPPORTED_OPTIMIZERS = ("Adam", "AdamW", "FusedAdamW")


class ZeroOptimizer_Stage1(FusedAdamW):
    """Fused AdamW over this rank's slice of the flat buffers plus the two collectives."""

    def __init__(self, flat: FlatBuffers, dp_group=None, **kw):
        self.dp_group = dp_group if dp_group is not None else mpu.get_data_parallel_group()
        self.dp_size = dist.get_world_size(self.dp_group) if (dist.is_initialized() and self.dp_group is not None) else 1
        self.dp_rank = dist.get_rank(self.dp_group) if self.dp_size > 1 else 0
        assert flat.numel % max(1, self.dp_size) == 0, "flat buffer must be padded to a multiple of dp"
        per = flat.numel // max(1, self.dp_size)
        super().__init__(flat, shard=(self.dp_rank * per, (self.dp_rank + 1) * per), **kw)

    def reduce_gradients(self):
        if self.dp_size == 1:
            return
        g = self.flat.grad
        out = torch.empty(self.end - self.start, dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g, group=self.dp_group)
        g[self.start:self.end].copy_(out)

    def step(self, grad_scale: float = 1.0, sumsq=None):
        if sumsq is None and self.dp_size > 1:
            sumsq = self.grad_sumsq().clone()
            dist.all_reduce(sumsq, group=self.dp_group)
        super().step(grad_scale=grad_scale / max(1, self.dp_size) if self.dp_size > 1 else grad_scale, sumsq=sumsq)
        if self.dp_size > 1:
            dist.all_gather_into_tensor(self.flat.model, self.flat.model[self.start:self.end].clone(),
                                        group=self.dp_group)

    def state_dict(self):
        sd = super().state_dict()
        sd["local_sub_partitions_of_fp32_groups"] = [self.master]
        sd["partition_count"] = self.dp_size
        return sd


def configure_zero_optimizer(params: Iterable[torch.nn.Parameter], args, optimizer_name: str = "AdamW"):
    """Flat buffers + stage-1 optimizer for ``params`` (Merak/core/zero/stage1.py:53-75)."""
    if optimizer_name not in ZERO_SUPPORTED_OPTIMIZERS and not getattr(args, "zero_allow_untested_optimizer", False):
        raise ValueError("%s is not a ZeRO-tested optimizer; set zero_allow_untested_optimizer" % optimizer_name)
    dp = mpu.get_data_parallel_world_size()
    flat = FlatBuffers(list(params), grad_dtype=torch.float32, pad_to=64 * dp)
    return ZeroOptimizer_Stage1(flat, lr=args.learning_rate, betas=(args.adam_beta1, args.adam_beta2),
                                eps=args.adam_epsilon, weight_decay=args.weight_decay,
                                max_grad_norm=args.max_grad_norm)
