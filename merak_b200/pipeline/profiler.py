"""``FlopsProfiler``: per-module forward FLOPs, MACs, parameters and latency
(Merak/core/pipeline/profiler.py:21-960).

The reference counts FLOPs by monkey-patching ``torch.nn.functional`` and tensor methods.  Here
the sm_100a kernel wrappers (GEMM, attention) report their own FLOPs to ``ops.flop_counter``, and
everything PyTorch itself executes is counted one level lower, at the ATen dispatcher
(``_AtenFlopMode``), which sees every functional, module and tensor-method call whatever its
spelling: matmul family, convolutions, attention, norms, softmax, activations, pooling,
interpolation, losses and element-wise arithmetic.  Module hooks attribute the counts and the
wall time to every enclosing module.  The AutoPipe partitioner uses the per-shard totals as its
cost vector.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.utils._python_dispatch

from ..ops import flop_counter
from ..ops import modules as km


def _prod(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


def _aten_flops(func, args, kwargs, out) -> int:
    """Forward FLOPs of one ATen call (a multiply-add counts as two).  Covers what the reference
    counts by patching ``torch.nn.functional`` and tensor methods
    (Merak/core/pipeline/profiler.py:487-800): the matmul family, convolutions, attention,
    normalisations, softmax, activations, pooling, interpolation, embeddings and element-wise
    arithmetic; pure data movement (views, copies, indexing) counts as zero."""
    name = func.__name__ if hasattr(func, "__name__") else str(func)
    name = name.split(".")[0]
    t = [a for a in args if isinstance(a, torch.Tensor)]
    o = out[0] if isinstance(out, (tuple, list)) and out and isinstance(out[0], torch.Tensor) else out
    on = o.numel() if isinstance(o, torch.Tensor) else 0
    if name in ("mm", "matmul", "dot", "mv"):
        return 2 * on * int(t[0].shape[-1]) if t else 0
    if name == "addmm":
        return 2 * on * int(t[1].shape[-1]) + on
    if name in ("bmm", "baddbmm"):
        a_ = t[-2]
        return 2 * on * int(a_.shape[-1]) + (on if name == "baddbmm" else 0)
    if name == "linear":
        x, w = t[0], t[1]
        return 2 * (x.numel() // max(1, int(x.shape[-1]))) * int(w.shape[0]) * int(w.shape[1]) + \
            (on if len(t) > 2 else 0)
    if name in ("convolution", "_convolution", "conv1d", "conv2d", "conv3d", "conv_transpose2d", "cudnn_convolution"):
        w = t[1]
        per_out = 2 * _prod(w.shape[1:])                  # in_channels/groups * kernel volume, multiply-add
        transposed = bool(args[6]) if len(args) > 6 and isinstance(args[6], bool) else "transpose" in name
        base = t[0].numel() // max(1, int(t[0].shape[1])) * int(w.shape[1]) if transposed else on
        return base * per_out + (on if len(t) > 2 else 0)
    if name.startswith("scaled_dot_product") or name.startswith("_scaled_dot_product") or \
            name in ("_flash_attention_forward", "_efficient_attention_forward"):
        q, k, v = t[0], t[1], t[2]
        b_h = _prod(q.shape[:-2])
        lq, d, lk, dv = int(q.shape[-2]), int(q.shape[-1]), int(k.shape[-2]), int(v.shape[-1])
        return b_h * (2 * lq * lk * d + 2 * lq * lk * dv + 5 * lq * lk)
    if name in ("native_layer_norm", "layer_norm", "native_group_norm", "group_norm", "native_batch_norm", "batch_norm",
                "_native_batch_norm_legit", "_native_batch_norm_legit_no_training", "cudnn_batch_norm",
                "instance_norm", "rms_norm", "_fused_rms_norm"):
        return 5 * (t[0].numel() if t else 0)
    if name in ("_softmax", "softmax", "_log_softmax", "log_softmax"):
        return 5 * on
    if name in ("gelu", "silu", "tanh", "sigmoid", "erf", "exp", "exp2", "log", "log2", "sqrt", "rsqrt", "pow",
                "reciprocal", "mish", "hardswish", "hardsigmoid", "softplus", "elu", "selu", "celu", "glu"):
        return 4 * on
    if name in ("relu", "relu_", "leaky_relu", "hardtanh", "clamp", "clamp_min", "clamp_max", "threshold", "abs", "neg",
                "add", "add_", "sub", "sub_", "mul", "mul_", "div", "div_", "maximum", "minimum", "where", "masked_fill",
                "addcmul", "addcdiv", "lerp", "rsub", "sign", "floor", "ceil", "round", "native_dropout", "dropout",
                "cumsum"):
        return on
    if name in ("sum", "mean", "var", "std", "var_mean", "amax", "amin", "max", "min", "prod", "norm",
                "linalg_vector_norm", "argmax", "argmin", "logsumexp", "topk", "sort"):
        return t[0].numel() if t else 0
    if name in ("avg_pool2d", "max_pool2d_with_indices", "max_pool2d", "avg_pool1d", "avg_pool3d", "max_pool3d_with_indices"):
        k = args[1] if len(args) > 1 else kwargs.get("kernel_size", 1)
        return on * _prod(k if isinstance(k, (tuple, list)) else (k, k))
    if name in ("_adaptive_avg_pool2d", "adaptive_avg_pool2d", "adaptive_max_pool2d", "_adaptive_avg_pool3d"):
        return t[0].numel() if t else 0
    if name.startswith("upsample_nearest"):
        return 0
    if name.startswith("upsample_bilinear") or name.startswith("upsample_linear"):
        return 4 * on * (2 if "bilinear" in name else 1)
    if name.startswith("upsample_bicubic") or name.startswith("upsample_trilinear"):
        return 16 * on
    if name in ("nll_loss_forward", "nll_loss2d_forward", "mse_loss", "binary_cross_entropy_with_logits", "smooth_l1_loss",
                "huber_loss", "l1_loss", "cross_entropy_loss"):
        return 3 * (t[0].numel() if t else 0)
    return 0            # embedding lookups, views, copies, indexing, comparisons: no arithmetic


class _AtenFlopMode(torch.utils._python_dispatch.TorchDispatchMode):
    """Feeds the FLOPs of every ATen call made while it is active to ``sink(flops)``."""

    def __init__(self, sink):
        super().__init__()
        self.sink = sink

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        out = func(*args, **kwargs)
        try:
            f = _aten_flops(func, args, kwargs, out)
        except Exception:
            f = 0
        if f:
            self.sink(int(f))
        return out


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
            if self._stack and self._stack[-1] is m:
                self._stack.pop()

        for m in self.model.modules():
            if isinstance(m, ignore):
                continue
            self._hooks.append(m.register_forward_pre_hook(pre))
            self._hooks.append(m.register_forward_hook(post))
        # two sources, never both for one op: the kernel wrappers report their own FLOPs (their work
        # is not an ATen call), everything PyTorch executes is counted at the ATen dispatch level
        flop_counter.start(self._credit)
        self._mode = _AtenFlopMode(self._credit)
        self._mode.__enter__()
        self.started = True

    def _credit(self, flops: int):
        for m in self._stack:            # every enclosing module accumulates
            self.flops[m] = self.flops.get(m, 0) + flops

    def stop_profile(self):
        if self.started:
            flop_counter.stop()
            mode, self._mode = getattr(self, "_mode", None), None
            if mode is not None:
                mode.__exit__(None, None, None)
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
