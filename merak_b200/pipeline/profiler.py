"""``FlopsProfiler``: per-module forward FLOPs, MACs, parameters and latency
(Merak/core/pipeline/profiler.py:21-960).

The reference counts FLOPs by monkey-patching ``torch.nn.functional``.  Here the GEMM and attention
wrappers report their own FLOPs to ``ops.flop_counter`` and a fallback formula covers plain
``torch.nn`` layers (Linear, Conv, Embedding, norms); module hooks attribute the counts and the
wall/device time to the innermost active module.  The AutoPipe partitioner uses the per-shard
totals as its cost vector.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..ops import flop_counter
from ..ops import modules as km


def _fallback_flops(m: nn.Module, inputs, output) -> int:
    x = inputs[0] if inputs and isinstance(inputs[0], torch.Tensor) else None
    if x is None:
        return 0
    if type(m) is nn.Linear:                      # kernel-backed Linear reports through the GEMM wrapper
        return 2 * x.numel() // max(1, x.shape[-1]) * m.in_features * m.out_features
    if isinstance(m, nn.Conv2d) and isinstance(output, torch.Tensor):
        k = m.kernel_size[0] * m.kernel_size[1] * m.in_channels // m.groups
        return 2 * output.numel() * k
    if isinstance(m, (nn.LayerNorm, km.RMSNorm)):
        return 5 * x.numel()
    if isinstance(m, (nn.GELU, nn.SiLU, nn.ReLU, nn.Softmax)):
        return x.numel()
    return 0


class FlopsProfiler:

    def __init__(self, model: nn.Module):
        self.model = model
        self.started = False
        self._hooks = []
        self._stack: List[nn.Module] = []
        self.flops: Dict[nn.Module, int] = {}
        self.latency: Dict[nn.Module, float] = {}
        self._t0: Dict[nn.Module, float] = {}

    # -- control ---------------------------------------------------------------------------------
    def start_profile(self, ignore_list=None):
        self.reset_profile()
        ignore = tuple(ignore_list or ())

        def pre(m, inp):
            self._stack.append(m)
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self._t0[m] = time.perf_counter()

        def post(m, inp, out):
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self.latency[m] = self.latency.get(m, 0.0) + time.perf_counter() - self._t0.pop(m, time.perf_counter())
            own = _fallback_flops(m, inp, out)
            if own:
                self._credit(own)
            if self._stack and self._stack[-1] is m:
                self._stack.pop()

        for m in self.model.modules():
            if isinstance(m, ignore):
                continue
            self._hooks.append(m.register_forward_pre_hook(pre))
            self._hooks.append(m.register_forward_hook(post))
        flop_counter.start(self._credit)
        self.started = True

    def _credit(self, flops: int):
        for m in self._stack:            # every enclosing module accumulates
            self.flops[m] = self.flops.get(m, 0) + flops

    def stop_profile(self):
        if self.started:
            flop_counter.stop()
            self.started = False

    def reset_profile(self):
        self.flops, self.latency, self._t0, self._stack = {}, {}, {}, []

    def end_profile(self):
        self.stop_profile()
        for h in self._hooks:
            h.remove()
        self._hooks = []

    # -- results ---------------------------------------------------------------------------------
    def get_total_flops(self, as_string: bool = False):
        total = self.flops.get(self.model, 0)
        return _fmt(total, "FLOPs") if as_string else total

    def get_total_macs(self, as_string: bool = False):
        total = self.get_total_flops() // 2
        return _fmt(total, "MACs") if as_string else total

    def get_total_duration(self, as_string: bool = False):
        t = self.latency.get(self.model, 0.0)
        return "%.2f ms" % (t * 1e3) if as_string else t

    def get_total_params(self, as_string: bool = False):
        n = sum(p.numel() for p in self.model.parameters())
        return _fmt(n, "") if as_string else n

    def module_flops(self, module: nn.Module) -> int:
        return self.flops.get(module, 0)

    def print_model_profile(self, module_depth: int = 2, top_modules: int = 5, printer=print):
        printer("-------------------------- Flops Profiler --------------------------")
        printer("params: %s | fwd FLOPs: %s | fwd latency: %s" % (
            self.get_total_params(True), self.get_total_flops(True), self.get_total_duration(True)))
        rows = []
        for name, m in self.model.named_modules():
            if name and name.count(".") < module_depth:
                rows.append((self.flops.get(m, 0), name, type(m).__name__, self.latency.get(m, 0.0)))
        for f, name, cls, lat in sorted(rows, reverse=True)[:max(top_modules, 1) * 4]:
            printer("  %-48s %-24s %12s  %8.3f ms" % (name, cls, _fmt(f, "FLOPs"), lat * 1e3))
        printer("---------------------------------------------------------------------")


def _fmt(n: float, unit: str) -> str:
    for scale, suffix in ((1e12, "T"), (1e9, "G"), (1e6, "M"), (1e3, "K")):
        if n >= scale:
            return "%.2f %s%s" % (n / scale, suffix, unit)
    return "%d %s" % (n, unit)


def profile_layer_costs(layers, run_all, unit: int = 1_000_000):
    """Forward cost (in MFLOPs, at least 1) of every module in ``layers`` measured while ``run_all()``
    executes them once; used as the AutoPipe cost vector (backward is taken as 3x forward)."""
    holder = nn.ModuleList(list(layers))
    prof = FlopsProfiler(holder)
    prof.start_profile()
    with torch.no_grad():
        run_all()
    prof.end_profile()
    return [max(1, prof.module_flops(l) // unit) for l in layers]
