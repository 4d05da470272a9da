"""Pipeline helpers: freeing a stage's output after it has been sent, a backward call that accepts
such freed outputs, and the tensor-parallel-aware gradient norm (Merak/core/pipeline/utils.py:38-196).

* ``deallocate_output_tensor(out)``: once the next stage has the activation, this stage only needs
  the tensor's ``grad_fn``; its storage is replaced by one element.
* ``custom_backward(output, grad_output)``: ``torch.autograd.backward`` insists that output and
  gradient shapes match, which no longer holds for a freed output, so the autograd engine is called
  directly.
* ``clip_grad_norm_``: global L2 norm where parameters replicated over the tensor-parallel group are
  counted by its rank 0 only, summed over the model-parallel group; gradients are scaled in place.
"""
from __future__ import annotations

from typing import Iterable, Union

import torch
import torch.distributed as dist
from torch.autograd import Variable

from ..parallel import mpu


def deallocate_output_tensor(out: torch.Tensor):
    """Pseudo-free ``out`` (keeps ``grad_fn``).  The tensor must not be a view of something else."""
    if out is None:
        return
    assert isinstance(out, torch.Tensor), "expected a tensor, got %s" % type(out).__name__
    assert out._base is None, "cannot free a view: its base would keep the memory alive"
    out.data = torch.empty((1,), device=out.device, dtype=out.dtype)


def custom_backward(output: torch.Tensor, grad_output: torch.Tensor):
    """Backward from an output whose data was freed by :func:`deallocate_output_tensor`."""
    assert output.numel() == 1, "output should have been freed with deallocate_output_tensor"
    assert isinstance(output, torch.Tensor) and (grad_output is None or isinstance(grad_output, torch.Tensor))
    if grad_output is None:
        assert output.numel() == 1, "implicit gradients exist for scalar outputs only"
        grad_output = torch.ones_like(output, memory_format=torch.preserve_format)
    Variable._execution_engine.run_backward(
        tensors=(output,), grad_tensors=(grad_output,), keep_graph=False, create_graph=False, inputs=tuple(),
        allow_unreachable=True, accumulate_grad=True)


def clip_grad_norm_(parameters: Union[torch.Tensor, Iterable[torch.Tensor]], max_norm: float, norm_type: float = 2.0):
    """Returns the global gradient norm and scales the gradients when it exceeds ``max_norm``."""
    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]
    params = [p for p in parameters if p.grad is not None]
    tp_rank = mpu.get_model_parallel_rank()
    tp = mpu.get_model_parallel_world_size()
    device = params[0].grad.device if params else torch.device("cpu")
    if norm_type == float("inf"):
        total = torch.tensor([max((p.grad.abs().max().item() for p in params), default=0.0)], device=device)
        if tp > 1:
            dist.all_reduce(total, op=dist.ReduceOp.MAX, group=mpu.get_model_parallel_group())
        total_norm = float(total.item())
    else:
        acc = torch.zeros(1, dtype=torch.float32, device=device)
        for p in params:
            if tp_rank == 0 or getattr(p, "model_parallel", False):      # replicas are counted once
                acc += p.grad.float().norm(norm_type) ** norm_type
        if tp > 1:
            dist.all_reduce(acc, group=mpu.get_model_parallel_group())
        if mpu.get_pipe_parallel_world_size() > 1:
            dist.all_reduce(acc, group=mpu.get_pipe_parallel_group())
        total_norm = float(acc.item()) ** (1.0 / norm_type)
    coef = max_norm / (total_norm + 1e-6)
    if coef < 1.0:
        for p in params:
            p.grad.mul_(coef)
    return total_norm
