"""ZeRO stage 1 (optimizer-state sharding over the data-parallel group).

The reference ports DeepSpeed's stage-1 optimizer (Merak/core/zero/stage1.py:42-843): flatten each
parameter group, pad to ``dp x sub_partition``, keep fp32 master copies of the local
sub-partitions, reduce-scatter gradients, step, all-gather parameters.  Here the engine keeps one
flat model buffer and one flat fp32 gradient buffer per stage, so stage 1 is "every dp rank owns
one contiguous ``1/dp`` slice of them": a reduce-scatter on the gradient buffer, the optimizer on
the owned slice (fp32 master + optimizer state exist only for that slice), and one all-gather of
the updated slice.  The engine's own fused AdamW does this natively (``ops.optim.FusedAdamW`` with
a ``shard``); an optimizer the user brings is wrapped by ``ZeroOptimizer_Stage1``
(= ``stage1.ShardedMasterOptimizer``), which the engine applies when ``zero_stage == 1``.
"""
from ..amp.loss_scaler import DynamicLossScaler
from .stage1 import (ZERO_SUPPORTED_OPTIMIZERS, ShardedMasterOptimizer, configure_zero_optimizer,
                     is_zero_supported_optimizer)

ZeroOptimizer_Stage1 = ShardedMasterOptimizer

__all__ = ["ZeroOptimizer_Stage1", "ShardedMasterOptimizer", "configure_zero_optimizer", "DynamicLossScaler",
           "ZERO_SUPPORTED_OPTIMIZERS", "is_zero_supported_optimizer"]
