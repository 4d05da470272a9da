"""Mixed precision (Merak/core/amp/amp_engine.py:33-190, fp16_optimizer.py:36-358, utils.py:32-203).

* bf16 / fp16 parameters always come with fp32 master weights: the engine's fused AdamW keeps them
  for its own optimizer, ``zero.stage1.ShardedMasterOptimizer`` adds them around an optimizer the
  user brings (the reference keeps no master copy for bf16 unless ZeRO is on).
* fp16 uses dynamic loss scaling with hysteresis (``DynamicLossScaler``); the overflow check is the
  non-finite counter of the squared-norm reduction plus the skip flag the optimizer honours, so
  detecting an overflow costs no extra pass over the gradients.
* ``MixedPrecisionConfig`` resolves the ``fp16`` / ``bf16`` / ``half_precision_backend`` / loss-scale
  arguments; the engine builds its loss scaler through it.
* ``FP16_Optimizer`` is the stand-alone form for users who drive a model by hand: master weights +
  loss scaling around any ``torch.optim`` optimizer.
"""
from __future__ import annotations

from typing import Optional

import torch

from .loss_scaler import DynamicLossScaler


class MixedPrecisionConfig:
    def __init__(self, args):
        self.fp16, self.bf16 = bool(args.fp16), bool(args.bf16)
        self.backend = args.half_precision_backend or "cuda_amp"
        if self.backend == "apex":
            raise ValueError("half_precision_backend='apex': apex is not part of this framework; the native "
                             "master-weight path ('cuda_amp') covers its O2 mode")
        self.dtype = torch.float16 if self.fp16 else (torch.bfloat16 if self.bf16 else torch.float32)
        self.loss_scale = args.loss_scale
        self.initial_scale_power = args.initial_scale_power
        self.loss_scale_window = args.loss_scale_window
        self.hysteresis = args.hysteresis
        self.min_loss_scale = args.min_loss_scale

    def dynamic_loss_args(self) -> dict:
        return dict(init_scale=2.0 ** min(self.initial_scale_power, 24), scale_window=self.loss_scale_window,
                    min_scale=self.min_loss_scale, hysteresis=self.hysteresis)

    def make_loss_scaler(self) -> Optional[DynamicLossScaler]:
        """fp16 only: a static scaler when ``loss_scale`` > 0, else the dynamic one."""
        if not self.fp16:
            return None
        if self.loss_scale and self.loss_scale > 0:
            return DynamicLossScaler(init_scale=self.loss_scale, static=True)
        return DynamicLossScaler(**self.dynamic_loss_args())

    def configure(self, model: torch.nn.Module, optimizer=None):
        """Casts the model to the compute dtype and wraps a user optimizer when needed."""
        if self.dtype != torch.float32:
            model.to(self.dtype)
        if optimizer is not None and self.dtype != torch.float32 and not hasattr(optimizer, "master"):
            optimizer = FP16_Optimizer(optimizer, static_loss_scale=self.loss_scale or None,
                                       dynamic_loss_scale=self.fp16 and not self.loss_scale,
                                       dynamic_loss_args=self.dynamic_loss_args())
        return model, optimizer


def check_overflow(params) -> bool:
    """True when any gradient holds inf/nan (one fused reduction, one host read)."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return False
    total = torch.stack([g.float().abs().sum() for g in grads]).sum()
    return not bool(torch.isfinite(total))


class FP16_Optimizer:
    """fp32 master weights + (dynamic) loss scaling around a ``torch.optim`` optimizer, for a
    training loop written by hand::

        opt = FP16_Optimizer(torch.optim.SGD(model.parameters(), lr=...), dynamic_loss_scale=True)
        opt.backward(loss); opt.step()

    A step whose gradients overflowed is skipped and lowers the scale (after ``hysteresis``
    overflows); ``step`` returns False for it.
    """

    def __init__(self, init_optimizer, static_loss_scale: Optional[float] = None, dynamic_loss_scale: bool = False,
                 dynamic_loss_args: Optional[dict] = None, clip_grad: float = 0.0):
        from ..zero.stage1 import ShardedMasterOptimizer
        self.inner = ShardedMasterOptimizer(init_optimizer, shard=False, max_grad_norm=clip_grad)
        if dynamic_loss_scale:
            self.scaler = DynamicLossScaler(**(dynamic_loss_args or {}))
        else:
            self.scaler = DynamicLossScaler(init_scale=static_loss_scale or 1.0, static=True)
        self.overflow = False

    @property
    def optimizer(self):
        return self.inner.optimizer

    @property
    def param_groups(self):
        return self.inner.param_groups

    @property
    def cur_scale(self) -> float:
        return self.scaler.cur_scale

    def backward(self, loss):
        (loss.float() * self.scaler.cur_scale).backward()

    def zero_grad(self, set_to_none: bool = True):
        self.inner.zero_grad()
        for p in self.inner.flat.params:
            p.grad = None

    def step(self) -> bool:
        for p in self.inner.flat.params:            # autograd's .grad joins the flat fp32 buffer
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None
        ok = self.inner.step(grad_scale=1.0 / self.scaler.cur_scale)
        self.overflow = not ok
        self.scaler.update_scale(self.overflow)
        self.inner.zero_grad()
        return ok

    def state_dict(self):
        return {"optimizer_state_dict": self.inner.state_dict(), "loss_scaler": self.scaler.state_dict(),
                "overflow": self.overflow}

    def load_state_dict(self, sd):
        self.inner.load_state_dict(sd["optimizer_state_dict"])
        self.scaler.load_state_dict(sd["loss_scaler"])
