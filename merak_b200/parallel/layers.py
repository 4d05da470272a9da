"""Tensor-parallel layers: column/row-parallel linear, vocab-parallel embedding, channel-parallel
convolution.  Same sharding convention as the reference (Merak/core/mpu/layers.py:92-449):

* ``ColumnParallelLinear``  weight ``[out/tp, in]``; input replicated (or, with Megatron-style
  sequence parallelism, sharded along the sequence and all-gathered first); output sharded.
* ``RowParallelLinear``     weight ``[out, in/tp]``; input sharded on the last dim; partial outputs
  summed by all-reduce (or reduce-scattered along the sequence under sequence parallelism).
* ``VocabParallelEmbedding`` rows ``[vocab/tp, hidden]``; out-of-range ids contribute zero.

The matmuls run on the tcgen05 GEMM (``merak_b200.ops.linear``) for CUDA bf16 tensors and on
``F.linear`` otherwise.  Full-size master weights are drawn from one seeded generator and sliced,
so a sharded model starts from exactly the weights of its unsharded counterpart.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.elementwise import embedding_sum
from ..ops.linear import linear as k_linear
from . import fused_tp
from . import mappings as M
from . import mpu


def _fused_comm(x, weight, sequence_parallel, seq_dim, input_sharded):
    """The fused-collective data plane of the tensor-parallel group, or None when this call has to
    use torch.distributed collectives (CPU, other dtypes or layouts, peer mapping unavailable)."""
    if not fused_tp.ENABLED or not x.is_cuda:
        return None
    n = mpu.get_model_parallel_world_size()
    if n == 1 or not fused_tp.usable(x, weight, n, sequence_parallel, seq_dim, input_sharded):
        return None
    return fused_tp.get_comm(mpu.get_model_parallel_group(), x.device)


def divide(a: int, b: int) -> int:
    if a % b != 0:
        raise ValueError("%d is not divisible by %d" % (a, b))
    return a // b


class VocabUtility:
    """Contiguous vocabulary range ``[first, last)`` owned by a rank."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition: int, rank: int, world_size: int):
        first = rank * per_partition
        return first, first + per_partition

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab: int, rank: int, world_size: int):
        return VocabUtility.vocab_range_from_per_partition_vocab_size(divide(global_vocab, world_size), rank,
                                                                      world_size)


def split_tensor_along_last_dim(t: torch.Tensor, parts: int, contiguous_chunks: bool = False):
    chunks = torch.split(t, divide(t.shape[-1], parts), dim=-1)
    return tuple(c.contiguous() for c in chunks) if contiguous_chunks else chunks


def default_init_method(std: float = 0.02) -> Callable[[torch.Tensor], torch.Tensor]:
    def init_(t):
        return nn.init.normal_(t, mean=0.0, std=std)
    return init_


def _sharded_master_weight(out_f: int, in_f: int, shard_dim: int, init_method, dtype, device, seed: Optional[int]):
    """Draw the full ``[out_f, in_f]`` weight on the CPU and keep this rank's slice."""
    tp, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
    gen_state = None
    if seed is not None:
        gen_state = torch.get_rng_state()
        torch.manual_seed(seed)
    full = torch.empty(out_f, in_f, dtype=torch.float32)
    init_method(full)
    if gen_state is not None:
        torch.set_rng_state(gen_state)
    piece = full.chunk(tp, dim=shard_dim)[rank] if tp > 1 else full
    return piece.to(dtype=dtype, device=device).contiguous()


class ColumnParallelLinear(nn.Module):
    """``Y = X A^T + b`` with ``A`` split along its output dimension.

    Args follow the reference (Merak/core/mpu/layers.py:168-265); ``sequence_parallel`` adds the
    Megatron form: the input is ``[B, L/tp, H]`` and is all-gathered along ``seq_dim`` first.
    """

    def __init__(self, input_size: int, output_size: int, bias: bool = True, gather_output: bool = False,
                 init_method: Optional[Callable] = None, skip_bias_add: bool = False,
                 sequence_parallel: bool = False, seq_dim: int = 1, params_dtype=torch.float32, device=None,
                 seed: Optional[int] = None):
        super().__init__()
        tp = mpu.get_model_parallel_world_size()
        self.input_size, self.output_size = input_size, output_size
        self.output_size_per_partition = divide(output_size, tp)
        self.gather_output, self.skip_bias_add = gather_output, skip_bias_add
        self.sequence_parallel, self.seq_dim = sequence_parallel and tp > 1, seq_dim
        init_method = init_method or default_init_method()
        dev = device if device is not None else "cpu"
        if str(dev) == "meta":
            w = torch.empty(self.output_size_per_partition, input_size, dtype=params_dtype, device="meta")
        else:
            w = _sharded_master_weight(output_size, input_size, 0, init_method, params_dtype, dev, seed)
        self.weight = nn.Parameter(w)
        self.weight.model_parallel = True
        self.weight.partition_dim = 0
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition, dtype=params_dtype, device=dev))
            self.bias.model_parallel = True
            self.bias.partition_dim = 0
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        comm = None if self.gather_output else _fused_comm(x, self.weight, self.sequence_parallel, self.seq_dim, True)
        if comm is not None:
            b = None if self.skip_bias_add else self.bias
            y = fused_tp.column_linear_fused(x, self.weight, b, comm, self.sequence_parallel)
            return (y, self.bias) if self.skip_bias_add else y
        if self.sequence_parallel:
            x = M.gather_from_sequence_parallel_region(x, self.seq_dim, True)
        else:
            x = M.copy_to_model_parallel_region(x)
        b = None if self.skip_bias_add else self.bias
        y = k_linear(x, self.weight, b)
        if self.gather_output:
            y = M.gather_from_model_parallel_region(y)
        if self.skip_bias_add:
            return y, self.bias
        return y

    def extra_repr(self):
        return "in=%d, out=%d (per rank %d), bias=%s, sp=%s" % (
            self.input_size, self.output_size, self.output_size_per_partition, self.bias is not None,
            self.sequence_parallel)


class RowParallelLinear(nn.Module):
    """``Y = X A^T + b`` with ``A`` split along its input dimension (Merak/core/mpu/layers.py:268-369)."""

    def __init__(self, input_size: int, output_size: int, bias: bool = True, input_is_parallel: bool = True,
                 init_method: Optional[Callable] = None, skip_bias_add: bool = False,
                 sequence_parallel: bool = False, seq_dim: int = 1, params_dtype=torch.float32, device=None,
                 seed: Optional[int] = None):
        super().__init__()
        tp = mpu.get_model_parallel_world_size()
        self.input_size, self.output_size = input_size, output_size
        self.input_size_per_partition = divide(input_size, tp)
        self.input_is_parallel, self.skip_bias_add = input_is_parallel, skip_bias_add
        self.sequence_parallel, self.seq_dim = sequence_parallel and tp > 1, seq_dim
        init_method = init_method or default_init_method()
        dev = device if device is not None else "cpu"
        if str(dev) == "meta":
            w = torch.empty(output_size, self.input_size_per_partition, dtype=params_dtype, device="meta")
        else:
            w = _sharded_master_weight(output_size, input_size, 1, init_method, params_dtype, dev, seed)
        self.weight = nn.Parameter(w)
        self.weight.model_parallel = True
        self.weight.partition_dim = 1
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size, dtype=params_dtype, device=dev))
            if self.sequence_parallel:
                self.bias.sequence_parallel = True     # sees this rank's tokens only: summed over the group
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        if not self.input_is_parallel:
            x = M.scatter_to_model_parallel_region(x)
        comm = _fused_comm(x, self.weight, self.sequence_parallel, self.seq_dim, False)
        if comm is not None:
            b = None if self.skip_bias_add else self.bias
            y = fused_tp.row_linear_fused(x, self.weight, b, comm, self.sequence_parallel)
            return (y, self.bias) if self.skip_bias_add else y
        y = k_linear(x, self.weight, None)
        if self.sequence_parallel:
            y = M.reduce_scatter_to_sequence_parallel_region(y, self.seq_dim)
        else:
            y = M.reduce_from_model_parallel_region(y)
        if self.skip_bias_add:
            return y, self.bias
        if self.bias is not None:
            y = y + self.bias
        return y

    def extra_repr(self):
        return "in=%d (per rank %d), out=%d, bias=%s, sp=%s" % (
            self.input_size, self.input_size_per_partition, self.output_size, self.bias is not None,
            self.sequence_parallel)


class VocabParallelEmbedding(nn.Module):
    """Embedding table split along the vocabulary (Merak/core/mpu/layers.py:92-165)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, init_method: Optional[Callable] = None,
                 params_dtype=torch.float32, device=None, seed: Optional[int] = None,
                 padding_idx: Optional[int] = None):
        super().__init__()
        tp, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padding_idx = padding_idx
        self.vocab_start_index, self.vocab_end_index = VocabUtility.vocab_range_from_global_vocab_size(
            num_embeddings, rank, tp)
        self.num_embeddings_per_partition = self.vocab_end_index - self.vocab_start_index
        init_method = init_method or default_init_method()
        dev = device if device is not None else "cpu"
        if str(dev) == "meta":
            w = torch.empty(self.num_embeddings_per_partition, embedding_dim, dtype=params_dtype, device="meta")
        else:
            w = _sharded_master_weight(num_embeddings, embedding_dim, 0, init_method, params_dtype, dev, seed)
        self.weight = nn.Parameter(w)
        self.weight.model_parallel = True
        self.weight.partition_dim = 0

    def forward(self, ids):
        out = embedding_sum([ids], [self.weight], [self.vocab_start_index])
        return M.reduce_from_model_parallel_region(out)


class ColParallelConv2d(nn.Module):
    """2-D convolution whose *input channels* are split across tensor-parallel ranks; the partial
    outputs are summed (Merak/core/mpu/layers.py:371-449).  The reference's scatter returned the
    unsplit input; here the input really is split, so results equal the unsharded convolution."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, init_method=None, params_dtype=torch.float32, device=None, seed=None):
        super().__init__()
        tp, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.in_per_partition = divide(in_channels, tp)
        self.stride, self.padding, self.dilation, self.groups = stride, padding, dilation, groups
        ks = kernel_size if isinstance(kernel_size, tuple) else (kernel_size, kernel_size)
        gen_state = None
        if seed is not None:
            gen_state = torch.get_rng_state()
            torch.manual_seed(seed)
        full = torch.empty(out_channels, in_channels // groups, *ks)
        (init_method or (lambda t: nn.init.kaiming_uniform_(t, a=math.sqrt(5))))(full)
        if gen_state is not None:
            torch.set_rng_state(gen_state)
        piece = full.chunk(tp, dim=1)[rank] if tp > 1 else full
        self.weight = nn.Parameter(piece.to(dtype=params_dtype, device=device or "cpu").contiguous())
        self.weight.model_parallel = True
        self.weight.partition_dim = 1
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_channels, dtype=params_dtype, device=device or "cpu"))
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        tp, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
        if tp > 1:
            x = _ScatterChannels.apply(x)
        y = F.conv2d(x, self.weight, None, self.stride, self.padding, self.dilation, self.groups)
        y = M.reduce_from_model_parallel_region(y)
        if self.bias is not None:
            y = y + self.bias.view(1, -1, 1, 1)
        return y


class _ScatterChannels(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        tp, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
        return x.chunk(tp, dim=1)[rank].contiguous()

    @staticmethod
    def backward(ctx, g):
        group, tp = mpu.get_model_parallel_group(), mpu.get_model_parallel_world_size()
        return M._gather_dim(g, 1, group, tp)
