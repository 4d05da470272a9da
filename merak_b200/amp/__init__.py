"""Mixed precision (Merak/core/amp/amp_engine.py:33-190, fp16_optimizer.py:36-358, utils.py:32-203).

* bf16 / fp16 parameters always come with fp32 master weights and moments (``ops.optim``); the
  reference keeps no master copy for bf16 unless ZeRO is on.
* fp16 uses dynamic loss scaling with hysteresis (``DynamicLossScaler``); the overflow check is the
  non-finite counter of the fused squared-norm kernel plus the skip flag the AdamW kernel honours,
  so detecting an overflow costs no extra pass and only one scalar read per step.
* ``MixedPrecisionConfig`` resolves the ``fp16`` / ``bf16`` / ``half_precision_backend`` arguments;
  ``FP16_Optimizer`` wraps any ``torch.optim`` optimizer with master weights + loss scaling for
  users who bring their own optimizer.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..pipeline.engine import DynamicLossScaler


class MixedPrecisionConfig:
    def __init__(self, args):
        self.fp16, self.bf16 = bool(args.fp16), bool(args.bf16)
        self.backend = args.half_precision_backend
        self.dtype = torch.float16 if self.fp16 else (torch.bfloat16 if self.bf16 else torch.float32)
        self.loss_scale = args.loss_scale
        self.use_autocast = self.backend in ("cuda_amp", "cpu_amp") and not (self.fp16 or self.bf16)

    def configure(self, model: torch.nn.Module, optimizer=None):
        """Casts the model to the compute dtype and wraps a user optimizer when needed."""
        if self.dtype != torch.float32:
            model.to(self.dtype)
        if optimizer is not None and self.dtype != torch.float32 and not hasattr(optimizer, "master"):
            optimizer = FP16_Optimizer(optimizer, static_loss_scale=self.loss_scale or None,
                                       dynamic_loss_scale=self.fp16 and not self.loss_scale)
        return model, optimizer


def check_overflow(params) -> bool:
    """True when any gradient holds inf/nan (one fused reduction, one host read)."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return False
    total = torch.stack([g.float().abs().sum() for g in grads]).sum()
    return not bool(torch.isfinite(total))


def get_global_norm(norms: List[float]) -> float:
    return float(sum(n * n for n in norms) ** 0.5)


class FP16_Optimizer:
    """fp32 master weights + (dynamic) loss scaling around a ``torch.optim`` optimizer."""

    def __init__(self, init_optimizer, static_loss_scale: Optional[float] = None, dynamic_loss_scale: bool = False,
                 initial_scale_power: int = 16, loss_scale_window: int = 1000, hysteresis: int = 2,
                 min_loss_scale: float = 1.0, clip_grad: float = 0.0):
        self.optimizer = init_optimizer
        self.clip_grad = clip_grad
        self.fp16_groups, self.fp32_groups = [], []
        for group in self.optimizer.param_groups:
            half = list(group["params"])
            master = [p.detach().clone().float().requires_grad_(True) for p in half]
            self.fp16_groups.append(half)
            self.fp32_groups.append(master)
            group["params"] = master
        if dynamic_loss_scale:
            self.scaler = DynamicLossScaler(init_scale=2.0 ** initial_scale_power, scale_window=loss_scale_window,
                                            min_scale=min_loss_scale, hysteresis=hysteresis)
        else:
            self.scaler = DynamicLossScaler(init_scale=static_loss_scale or 1.0, static=True)
        self.overflow = False

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    @property
    def cur_scale(self):
        return self.scaler.cur_scale

    def backward(self, loss):
        (loss.float() * self.scaler.cur_scale).backward()

    def zero_grad(self, set_to_none: bool = True):
        for g in self.fp16_groups:
            for p in g:
                p.grad = None

    def step(self):
        half = [p for g in self.fp16_groups for p in g]
        self.overflow = check_overflow(half)
        self.scaler.update_scale(self.overflow)
        if self.overflow:
            self.zero_grad()
            return False
        inv = 1.0 / self.scaler.cur_scale
        for hg, mg in zip(self.fp16_groups, self.fp32_groups):
            for h, m in zip(hg, mg):
                m.grad = None if h.grad is None else h.grad.float() * inv
        if self.clip_grad > 0:
            torch.nn.utils.clip_grad_norm_([m for g in self.fp32_groups for m in g], self.clip_grad)
        self.optimizer.step()
        for hg, mg in zip(self.fp16_groups, self.fp32_groups):
            for h, m in zip(hg, mg):
                h.data.copy_(m.data)
        self.zero_grad()
        return True

    def state_dict(self):
        return {"optimizer_state_dict": self.optimizer.state_dict(), "loss_scaler": self.scaler.state_dict(),
                "fp32_groups": [[m.detach().clone() for m in g] for g in self.fp32_groups], "overflow": self.overflow}

    def load_state_dict(self, sd):
        self.optimizer.load_state_dict(sd["optimizer_state_dict"])
        self.scaler.load_state_dict(sd["loss_scaler"])
        for g, saved in zip(self.fp32_groups, sd["fp32_groups"]):
            for m, s in zip(g, saved):
                m.data.copy_(s)
