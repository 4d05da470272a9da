"""Fused AdamW over flat parameter buffers with fp32 master weights.

All parameters of a model (or of one rank's ZeRO shard) are laid out back to back in one bf16
"model" buffer that the ``nn.Parameter`` objects view, one fp32 gradient buffer that the wgrad
GEMM epilogues accumulate into (``param.main_grad``), and fp32 master / moment buffers.  One
optimizer step is then: squared-norm reduction -> clip coefficient (on device) -> one AdamW kernel
that also refreshes the bf16 model buffer.  No per-parameter Python loop and no host sync,
unlike torch.optim.AdamW + the master copy-back loop of the reference
(Merak/core/zero/stage1.py:670-757, Merak/core/amp/fp16_optimizer.py:167-174).
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional

import torch

from . import _lib


def _align(n: int, a: int = 64) -> int:
    return (n + a - 1) // a * a


class FlatBuffers:
    """Re-homes parameters into one contiguous model buffer and one fp32 gradient buffer."""

    def __init__(self, params: Iterable[torch.nn.Parameter], grad_dtype=torch.float32, pad_to: int = 64,
                 allocator=None):
        """``allocator(numel, dtype, tag)`` (tag "model" / "grad") may supply the two buffers, e.g.
        peer-mapped memory for the fused data-parallel kernels; it must return zeroed memory."""
        self.params: List[torch.nn.Parameter] = [p for p in params]
        assert self.params, "no parameters"
        dev, dt = self.params[0].device, self.params[0].dtype
        assert all(p.device == dev and p.dtype == dt for p in self.params), "mixed device/dtype"
        self.offsets = []
        off = 0
        for p in self.params:
            self.offsets.append(off)
            off += _align(p.numel(), 64)
        self.numel = _align(off, pad_to)
        if allocator is not None:
            self.model = allocator(self.numel, dt, "model")
            self.grad = allocator(self.numel, grad_dtype, "grad")
        else:
            self.model = torch.zeros(self.numel, dtype=dt, device=dev)
            self.grad = torch.zeros(self.numel, dtype=grad_dtype, device=dev)
        for p, o in zip(self.params, self.offsets):
            view = self.model[o:o + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.grad[o:o + p.numel()].view(p.shape)
            p.grad = None

    def zero_grad(self):
        self.grad.zero_()


class FusedAdamW:
    """AdamW on a :class:`FlatBuffers` (or on the ``[start, end)`` shard of it that this rank owns)."""

    def __init__(self, flat: FlatBuffers, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 decay_mask: Optional[torch.Tensor] = None, shard=None, max_grad_norm: float = 0.0):
        self.flat = flat
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.start, self.end = shard if shard is not None else (0, flat.numel)
        n = self.end - self.start
        dev = flat.model.device
        self.master = flat.model[self.start:self.end].float()
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        self.step_count = 0
        # segments with / without weight decay (norm weights and biases are excluded by the trainer)
        self.segments = self._segments(decay_mask)
        self._hp = {}
        self._sumsq = torch.zeros(2, dtype=torch.float32, device=dev)
        self._scale = torch.ones(1, dtype=torch.float32, device=dev)
        self._skip = torch.zeros(1, dtype=torch.int32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.param_groups = [{"lr": lr, "betas": betas, "eps": eps, "weight_decay": weight_decay}]
        # single-launch update (bf16 model, fp32 gradients): per-granule weight-decay flags + the
        # shard-update kernel of the fused data-parallel path run as a group of one rank
        self._one_launch = None
        if (dev.type == "cuda" and flat.model.dtype == torch.bfloat16 and flat.grad.dtype == torch.float32
                and n % 8 == 0 and self.start % 64 == 0):
            import ctypes
            import numpy as np
            fl = np.zeros(flat.numel // 64 + 1, dtype=np.uint8)
            for s, e, decay in self.segments:
                if decay:
                    fl[s // 64:(e + 63) // 64] = 1
            ctrl = torch.zeros(int(_lib.kernels().mrk_symm_ctrl_bytes()), dtype=torch.uint8, device=dev)
            self._one_launch = {"flags": torch.from_numpy(fl).to(dev), "ctrl": ctrl,
                                "models": (ctypes.c_void_p * 1)(flat.model.data_ptr()),
                                "ctrls": (ctypes.c_void_p * 1)(ctrl.data_ptr())}

    def _segments(self, decay_mask):
        flat = self.flat
        segs = []
        for p, o in zip(flat.params, flat.offsets):
            s, e = max(o, self.start), min(o + _align(p.numel(), 64), self.end)
            if s >= e:
                continue
            decay = getattr(p, "_no_weight_decay", False) is False and p.dim() > 1
            if segs and segs[-1][2] == decay and segs[-1][1] == s:
                segs[-1] = (segs[-1][0], e, decay)
            else:
                segs.append((s, e, decay))
        return segs

    def _hp_tensor(self, wd: float) -> torch.Tensor:
        lr = self.param_groups[0]["lr"]
        b1, b2 = self.betas
        t = self.step_count
        vals = [lr, b1, b2, self.eps, wd, 1.0 - b1 ** t, 1.0 - b2 ** t]
        key = wd
        if key not in self._hp:
            self._hp[key] = torch.empty(7, dtype=torch.float32, device=self.master.device)
        self._hp[key].copy_(torch.tensor(vals, dtype=torch.float32), non_blocking=True)
        return self._hp[key]

    @torch.no_grad()
    def grad_sumsq(self) -> torch.Tensor:
        """[sum of squares, non-finite count] of this shard's gradients (device tensor)."""
        g = self.flat.grad[self.start:self.end]
        self._sumsq.zero_()
        if g.is_cuda:
            _lib.check(_lib.kernels().mrk_sumsq(g.data_ptr(), g.numel(), self._sumsq.data_ptr(),
                                                int(g.dtype == torch.float32), _lib.stream_ptr()), "mrk_sumsq")
        else:
            gf = g.float()
            self._sumsq[0] = (gf * gf).sum()
            self._sumsq[1] = (~torch.isfinite(gf)).sum()
        return self._sumsq

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, sumsq: Optional[torch.Tensor] = None):
        """One update.  ``grad_scale`` multiplies gradients first (1/loss_scale, 1/accumulation);
        ``sumsq`` lets the caller pass an already all-reduced squared norm."""
        self.step_count += 1
        if sumsq is None:
            sumsq = self.grad_sumsq()
        g = self.flat.grad
        if g.is_cuda and self._one_launch is not None:
            ol = self._one_launch
            hp = self._hp_tensor(self.weight_decay)
            _lib.check(_lib.kernels().mrk_dp_adamw_allgather(
                ol["models"], ol["ctrls"], 1, 0, self.start, self.end - self.start, g.data_ptr() + 4 * self.start,
                self.master.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(), ol["flags"].data_ptr(),
                hp.data_ptr(), float(grad_scale), float(self.max_grad_norm), sumsq.data_ptr(), self._norm.data_ptr(),
                self._skip.data_ptr(), 0, 0, 0, 0, _lib.stream_ptr()), "mrk_dp_adamw_allgather")
        elif g.is_cuda:
            lib = _lib.kernels()
            st = _lib.stream_ptr()
            _lib.check(lib.mrk_clip_coef(sumsq.data_ptr(), float(grad_scale), float(self.max_grad_norm),
                                         self._scale.data_ptr(), self._skip.data_ptr(), self._norm.data_ptr(), st),
                       "mrk_clip_coef")
            for s, e, decay in self.segments:
                hp = self._hp_tensor(self.weight_decay if decay else 0.0)
                lo, n = s - self.start, e - s
                _lib.check(lib.mrk_adamw(self.master.data_ptr() + 4 * lo, self.exp_avg.data_ptr() + 4 * lo,
                                         self.exp_avg_sq.data_ptr() + 4 * lo, g.data_ptr() + g.element_size() * s,
                                         self.flat.model.data_ptr() + self.flat.model.element_size() * s,
                                         hp.data_ptr(), self._scale.data_ptr(), self._skip.data_ptr(), n,
                                         int(g.dtype == torch.float32), int(self.flat.model.dtype == torch.float32),
                                         st), "mrk_adamw")
        else:
            self._step_reference(grad_scale, sumsq)

    def _step_reference(self, grad_scale, sumsq):
        norm = math.sqrt(float(sumsq[0])) * grad_scale
        bad = not math.isfinite(norm) or float(sumsq[1]) != 0
        self._norm[0] = norm
        self._skip[0] = int(bad)
        if bad:
            return
        coef = 1.0
        if self.max_grad_norm > 0 and norm > self.max_grad_norm:
            coef = self.max_grad_norm / (norm + 1e-6)
        scale = grad_scale * coef
        lr = self.param_groups[0]["lr"]
        b1, b2 = self.betas
        t = self.step_count
        for s, e, decay in self.segments:
            wd = self.weight_decay if decay else 0.0
            lo, hi = s - self.start, e - self.start
            g = self.flat.grad[s:e].float() * scale
            m, v, p = self.exp_avg[lo:hi], self.exp_avg_sq[lo:hi], self.master[lo:hi]
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            p.mul_(1 - lr * wd).addcdiv_(m / (1 - b1 ** t), (v / (1 - b2 ** t)).sqrt() + self.eps, value=-lr)
            self.flat.model[s:e].copy_(p)

    def grad_norm(self) -> torch.Tensor:
        return self._norm

    def skipped(self) -> torch.Tensor:
        return self._skip

    def zero_grad(self, set_to_none: bool = False):
        self.flat.zero_grad()

    def state_dict(self):
        return {"step": self.step_count, "master": self.master, "exp_avg": self.exp_avg,
                "exp_avg_sq": self.exp_avg_sq, "shard": (self.start, self.end),
                "param_groups": self.param_groups}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.param_groups[0].update(sd["param_groups"][0])
        self.flat.model[self.start:self.end].copy_(self.master)
