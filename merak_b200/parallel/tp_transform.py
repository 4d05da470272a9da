"""Turning a model's ``nn.Linear`` layers into tensor-parallel layers from a per-model "feature
dict" (which layers are column-parallel, which are row-parallel), the reference's mechanism
(Merak/core/tensor_parallel/mp_attrs.py:24-202, mp_mapping.py:21-51, mp_layers.py:74-184,
model_parallel.py:38-193).

* ``set_tp_layer_lists(col_para_list=..., row_para_list=..., ...)`` registers name fragments for
  models without a built-in entry (same public function as the reference).
* ``apply_tensor_parallel(model, ...)`` swaps matching ``nn.Linear`` modules for ``ColPara`` /
  ``RowPara`` wrappers.  The wrappers keep the reference's parameter naming
  (``<layer>.col_linear.weight`` / ``<layer>.row_linear.weight``), which is part of the checkpoint
  format ``tools/convert_safetensor.py`` understands.
* Fused projections (``fused_parts`` / ``fused_sizes`` on a Linear: QKV, gate|up) are split part by
  part so every rank holds matching slices of each part.
* ``vocab_parallel`` replaces the input embedding and the output projection by their
  vocabulary-sharded forms.
* With ``megatron_sp=True`` column layers all-gather their input along the sequence and row
  layers reduce-scatter their output (sequence parallelism inside the tensor-parallel group); the
  embedding output is scattered along the sequence and norm parameters are flagged so their
  gradients get summed over the group.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence

import torch
import torch.nn as nn

from . import mappings as M
from . import mpu
from .layers import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding, divide

# process-global registries, like the reference's module-level lists
COL_PARA_LIST: List[str] = []
ROW_PARA_LIST: List[str] = []
CONV_PARA_LIST: List[str] = []
WEIGHT_CHANGE_LIST: List = []       # (name fragment, dimension): weights that are not linear layers but hold one slice per head
TP_ATTR_LIST: List[str] = ["num_heads", "split_size", "n_heads", "inner_dim", "num_attention_heads",
                           "all_head_size", "num_key_value_heads", "embed_dim"]
MANUAL = {"set": False}

DEFAULT_FEATURES: Dict[str, Dict[str, List[str]]] = {
    "gpt2": {"col": ["c_attn", "c_fc"], "row": ["c_proj"]},
    "bert": {"col": ["self.qkv", "self.query", "self.key", "self.value", "intermediate.dense"],
             "row": ["attention.output.dense", "output.dense"]},
    "llama": {"col": ["qkv_proj", "q_proj", "k_proj", "v_proj", "gate_up_proj", "gate_proj", "up_proj"],
              "row": ["o_proj", "down_proj"]},
    "t5": {"col": ["SelfAttention.q", "SelfAttention.k", "SelfAttention.v", "EncDecAttention.q", "EncDecAttention.k",
                   "EncDecAttention.v", "DenseReluDense.wi"], "row": ["SelfAttention.o", "EncDecAttention.o",
                                                                       "DenseReluDense.wo"],
           # the relative position bias is an embedding [buckets, heads]: each rank keeps its heads' columns
           # (Merak/core/tensor_parallel/mp_mapping.py:34-40)
           "weight": [("relative_attention_bias", 1)]},
    "vit": {"col": ["attention.query", "attention.key", "attention.value", "intermediate.dense"],
            "row": ["attention.output.dense", "output.dense"]},
}
for alias, base in (("qwen", "llama"), ("qwen2", "llama"), ("mistral", "llama"), ("deepseek_v2", "llama"),
                    ("moe", "llama"), ("mt5", "t5"), ("roberta", "bert")):
    DEFAULT_FEATURES[alias] = DEFAULT_FEATURES[base]


def set_tp_layer_lists(col_para_list: Optional[Sequence[str]] = None, row_para_list: Optional[Sequence[str]] = None,
                       conv_para_list: Optional[Sequence[str]] = None, input_output_mapping=None,
                       weight_change_list=None, tp_attr_list: Optional[Sequence[str]] = None):
    """Registers which layers (by name fragment) become column-/row-parallel.  ``weight_change_list``:
    ``(name fragment, dim)`` pairs of other weights that are cut along ``dim`` (T5's relative position bias;
    a linear layer named there becomes column-parallel for ``dim`` 0 and row-parallel for ``dim`` 1, as in
    Merak/core/tensor_parallel/mp_attrs.py:57-81).  ``input_output_mapping`` is accepted for signature
    compatibility: shapes are derived from the layers themselves here."""
    if weight_change_list is not None:
        WEIGHT_CHANGE_LIST[:] = [(str(n), int(d)) for n, d in weight_change_list]
    if col_para_list is not None:
        COL_PARA_LIST[:] = list(col_para_list)
    if row_para_list is not None:
        ROW_PARA_LIST[:] = list(row_para_list)
    if conv_para_list is not None:
        CONV_PARA_LIST[:] = list(conv_para_list)
    if tp_attr_list is not None:
        TP_ATTR_LIST[:] = list(tp_attr_list)
    MANUAL["set"] = True


def _unit_range(total: int, tp: int, rank: int, unit: int = 1):
    """``[start, start + size)`` of rank ``rank`` when ``total`` elements made of indivisible groups of
    ``unit`` (attention heads) are split over ``tp`` ranks; the first ``groups % tp`` ranks get one
    group more (GPT-2 1.5B: 25 heads over 2 ranks -> 13 + 12)."""
    groups = total // max(1, unit)
    base, rem = divmod(groups, tp)
    n = base + (1 if rank < rem else 0)
    start = base * rank + min(rank, rem)
    return start * unit, n * unit


def _slice_fused(weight: torch.Tensor, dim: int, rank: int, tp: int, parts=None, sizes=None, unit: int = 1) -> torch.Tensor:
    """This rank's slice of a (possibly fused) weight along ``dim``."""
    if sizes is None and parts:
        sizes = [weight.shape[dim] // parts] * parts
    if not sizes:
        sizes = [weight.shape[dim]]
    pieces, off = [], 0
    for sz in sizes:
        start, n = _unit_range(sz, tp, rank, unit if sz % max(1, unit) == 0 else 1)
        pieces.append(weight.narrow(dim, off + start, n))
        off += sz
    return torch.cat(pieces, dim=dim).contiguous()


class ColPara(nn.Module):
    """Column-parallel replacement of a Linear; parameters live under ``col_linear``."""

    def __init__(self, linear: nn.Linear, gather_output: bool = False, sequence_parallel: bool = False,
                 seq_dim: int = 1):
        super().__init__()
        tp, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
        w = linear.weight
        self.in_features, self.out_features = linear.in_features, linear.out_features
        parts, sizes = getattr(linear, "fused_parts", None), getattr(linear, "fused_sizes", None)
        unit = int(getattr(linear, "tp_unit", 1) or 1)
        self.col_linear = ColumnParallelLinear(linear.in_features, linear.out_features,
                                               bias=linear.bias is not None, gather_output=gather_output,
                                               sequence_parallel=sequence_parallel, seq_dim=seq_dim,
                                               params_dtype=w.dtype, device="meta")
        # slicing works on meta tensors too (shapes only), so models built under init_empty_weights pass
        self.col_linear.weight = nn.Parameter(_slice_fused(w.data, 0, rank, tp, parts, sizes, unit))
        if linear.bias is not None:
            self.col_linear.bias = nn.Parameter(_slice_fused(linear.bias.data, 0, rank, tp, parts, sizes, unit))
        self.col_linear.output_size_per_partition = self.col_linear.weight.shape[0]
        for p in self.col_linear.parameters():
            p.model_parallel, p.partition_dim = True, 0
        self.fused_parts, self.fused_sizes = parts, sizes

    # model code that inspects ``layer.weight`` / ``layer.bias`` (dtype checks in Hugging Face's T5) sees the shard
    @property
    def weight(self):
        return self.col_linear.weight

    @property
    def bias(self):
        return self.col_linear.bias

    def forward(self, x, residual=None):
        y = self.col_linear(x)
        return y if residual is None else y + residual


class RowPara(nn.Module):
    """Row-parallel replacement of a Linear; parameters live under ``row_linear``."""

    def __init__(self, linear: nn.Linear, input_is_parallel: bool = True, sequence_parallel: bool = False,
                 seq_dim: int = 1):
        super().__init__()
        tp, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
        w = linear.weight
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.row_linear = RowParallelLinear(linear.in_features, linear.out_features, bias=linear.bias is not None,
                                            input_is_parallel=input_is_parallel,
                                            sequence_parallel=sequence_parallel, seq_dim=seq_dim,
                                            params_dtype=w.dtype, device="meta")
        unit = int(getattr(linear, "tp_unit", 1) or 1)
        self.row_linear.weight = nn.Parameter(_slice_fused(w.data, 1, rank, tp, None, None, unit))
        self.row_linear.input_size_per_partition = self.row_linear.weight.shape[1]
        if linear.bias is not None:
            self.row_linear.bias = nn.Parameter(linear.bias.data.clone())
        self.row_linear.weight.model_parallel, self.row_linear.weight.partition_dim = True, 1
        if self.row_linear.bias is not None and self.row_linear.sequence_parallel:
            # added to this rank's sequence shard only: its gradient is summed over the group
            self.row_linear.bias.sequence_parallel = True

    @property
    def weight(self):
        return self.row_linear.weight

    @property
    def bias(self):
        return self.row_linear.bias

    def forward(self, x, residual=None):
        y = self.row_linear(x)
        return y if residual is None else y + residual


class ConvPara(nn.Module):
    """Channel-parallel replacement of a ``nn.Conv2d`` named in ``CONV_PARA_LIST``: the input channels
    are split over the tensor-parallel ranks and the partial outputs summed; parameters live under
    ``conv`` (Merak/core/tensor_parallel/mp_layers.py:186-226)."""

    def __init__(self, conv: nn.Conv2d):
        super().__init__()
        from .layers import ColParallelConv2d
        tp, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
        self.conv = ColParallelConv2d(conv.in_channels, conv.out_channels, conv.kernel_size, conv.stride, conv.padding,
                                      conv.dilation, conv.groups, bias=conv.bias is not None,
                                      params_dtype=conv.weight.dtype, device=conv.weight.device)
        self.conv.weight = nn.Parameter(conv.weight.data.chunk(tp, dim=1)[rank].contiguous())
        self.conv.weight.model_parallel, self.conv.weight.partition_dim = True, 1
        if conv.bias is not None:
            self.conv.bias = nn.Parameter(conv.bias.data.clone())

    def forward(self, x):
        return self.conv(x)


class _SeqScatter(nn.Module):
    """Wraps a module whose output starts the sequence-parallel region: scatters along ``dim``."""

    def __init__(self, inner: nn.Module, dim: int = 1):
        super().__init__()
        self.inner, self.dim = inner, dim

    def forward(self, *a, **k):
        return M.scatter_to_sequence_parallel_region(self.inner(*a, **k), self.dim)


def _matches(name: str, fragments: Iterable[str]) -> bool:
    return any(name.endswith(f) or ("." + f + ".") in ("." + name + ".") for f in fragments)


def feature_lists(model_type: Optional[str]):
    if MANUAL["set"]:
        return list(COL_PARA_LIST), list(ROW_PARA_LIST)
    feats = DEFAULT_FEATURES.get((model_type or "").lower())
    if feats is None:
        raise ValueError("no tensor-parallel feature dict for model type %r; call set_tp_layer_lists(...)" % model_type)
    return feats["col"], feats["row"]


def weight_change_list(model_type: Optional[str]):
    if MANUAL["set"]:
        return list(WEIGHT_CHANGE_LIST)
    return list((DEFAULT_FEATURES.get((model_type or "").lower()) or {}).get("weight", []))


def _shard_listed_weights(model: nn.Module, pairs, tp: int, rank: int) -> List[str]:
    """Cuts the ``weight`` of every non-linear module named in ``pairs`` along the given dimension and keeps
    this rank's slice (rank order, like the heads of the column-parallel projections beside it)."""
    done = []
    for name, m in model.named_modules():
        for frag, d in pairs:
            w = getattr(m, "weight", None)
            if not _matches(name, [frag]) or isinstance(m, (nn.Linear, ColPara, RowPara)) or \
                    not isinstance(w, nn.Parameter) or getattr(w, "model_parallel", False):
                continue
            if w.shape[d] % tp:
                raise ValueError("%s.weight has %d entries along dim %d, not divisible by tp=%d" % (name, w.shape[d], d, tp))
            piece = nn.Parameter(w.data.chunk(tp, dim=d)[rank].contiguous(), requires_grad=w.requires_grad)
            piece.model_parallel, piece.partition_dim = True, d
            m.weight = piece
            if isinstance(m, nn.Embedding):
                m.num_embeddings, m.embedding_dim = piece.shape
            done.append(name)
    return done


def convert_conv1d(model: nn.Module, fragments: Sequence[str]) -> int:
    """Hugging Face GPT-2 style ``Conv1D`` layers (``y = x @ W + b`` with ``W`` of shape [in, out])
    named in the feature lists become ``nn.Linear`` layers holding ``W^T``, the form the column /
    row wrappers slice (the reference lists ``Conv1D`` next to ``nn.Linear``,
    Merak/core/tensor_parallel/mp_attrs.py:22,43-147).  A fused query/key/value projection
    (``out = 3 * in``) is marked so that each of its three parts is split separately."""
    try:
        from transformers.pytorch_utils import Conv1D
    except Exception:
        return 0
    n = 0
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            full = (parent_name + "." if parent_name else "") + child_name
            if not isinstance(child, Conv1D) or not _matches(full, fragments):
                continue
            in_f, out_f = child.weight.shape
            lin = nn.Linear(in_f, out_f, bias=child.bias is not None, device="meta")
            lin.weight = nn.Parameter(child.weight.data.t().contiguous())
            if child.bias is not None:
                lin.bias = nn.Parameter(child.bias.data)
            lin.from_conv1d = True
            if out_f == 3 * in_f:
                lin.fused_parts = 3
            setattr(parent, child_name, lin)
            n += 1
    return n


def apply_tensor_parallel(model: nn.Module, model_type: Optional[str] = None, megatron_sp: bool = False,
                          seq_dim: int = 1, vocab_parallel: bool = False, skip: Sequence[str] = ("lm_head",)):
    """In-place transform; returns the list of replaced module names."""
    tp = mpu.get_model_parallel_world_size()
    if tp == 1:
        return []
    model_type = model_type or getattr(getattr(model, "config", None), "model_type", None)
    col, row = feature_lists(model_type)
    extra = weight_change_list(model_type)
    col = list(col) + [f for f, d in extra if d == 0]          # linear layers named there: dim 0 = column, 1 = row
    row = list(row) + [f for f, d in extra if d == 1]
    replaced = []
    convert_conv1d(model, col + row)
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            full = (parent_name + "." if parent_name else "") + child_name
            if isinstance(child, nn.Conv2d) and CONV_PARA_LIST and _matches(full, CONV_PARA_LIST) and \
                    child.groups == 1 and child.in_channels % tp == 0:
                setattr(parent, child_name, ConvPara(child))
                replaced.append(full)
                continue
            if not isinstance(child, nn.Linear) or any(s in full for s in skip):
                continue
            if _matches(full, row):          # row first: "output.dense" also ends with "dense"
                setattr(parent, child_name, RowPara(child, sequence_parallel=megatron_sp, seq_dim=seq_dim))
                replaced.append(full)
            elif _matches(full, col):
                setattr(parent, child_name, ColPara(child, sequence_parallel=megatron_sp, seq_dim=seq_dim))
                replaced.append(full)
    replaced += _shard_listed_weights(model, extra, tp, mpu.get_model_parallel_rank())
    # head-count style attributes are per-rank after sharding
    for m in model.modules():
        if any(isinstance(c, (ColPara, RowPara)) for c in m.children()):
            for attr in TP_ATTR_LIST:
                v = getattr(m, attr, None)
                if isinstance(v, int) and not isinstance(v, bool) and v % tp == 0 and v >= tp:
                    setattr(m, attr, v // tp)
    if megatron_sp:
        _enter_sequence_parallel(model, seq_dim)
        # activations between the blocks are sequence shards: their dropout is rank-dependent
        from ..ops.rng import dropout_state
        dropout_state().default_kind = "sharded"
    if vocab_parallel:
        apply_vocab_parallel(model, megatron_sp, seq_dim)
    return replaced


def _scatter_output_hook(seq_dim: int):
    def hook(module, inputs, output):
        return M.scatter_to_sequence_parallel_region(output, seq_dim)
    return hook


def _enter_sequence_parallel(model: nn.Module, seq_dim: int):
    """Starts the sequence-parallel region after the input embeddings.  A single token embedding
    (Llama) is wrapped; where several embeddings are summed first (GPT-2: ``wte + wpe`` then ``drop``;
    BERT: the ``embeddings`` block with its own LayerNorm) the output of that last module is
    scattered by a forward hook, which keeps every parameter name.  Norms computed before the
    scatter see the whole sequence on every rank and are therefore not marked sequence-parallel."""
    emb_owner, emb_name = _find_input_embedding(model)
    full_sequence_params = set()
    if emb_owner is not None:
        if hasattr(emb_owner, "wpe") and isinstance(getattr(emb_owner, "drop", None), nn.Module):
            emb_owner.drop.register_forward_hook(_scatter_output_hook(seq_dim))
        elif type(emb_owner).__name__.endswith("Embeddings"):
            emb_owner.register_forward_hook(_scatter_output_hook(seq_dim))
            full_sequence_params = {id(p) for p in emb_owner.parameters()}
        else:
            setattr(emb_owner, emb_name, _SeqScatter(getattr(emb_owner, emb_name), seq_dim))
    for m in model.modules():
        if isinstance(m, nn.LayerNorm) or type(m).__name__.endswith("RMSNorm"):
            for p in m.parameters():
                if id(p) not in full_sequence_params:
                    p.sequence_parallel = True
    head = _find_output_projection(model)
    if head is not None:
        owner, name = head
        lin = getattr(owner, name)
        if isinstance(lin, nn.Linear):
            setattr(owner, name, _GatherThenLinear(lin, seq_dim))
            # other replicated layers of the same head (BERT's transform) still run on this rank's
            # tokens only: their gradients are summed over the group like the norms'
            proj = {id(p) for p in lin.parameters()}
            if owner is not model:      # a dedicated head module; the root model owns everything else too
                for p in owner.parameters():
                    if id(p) not in proj and not getattr(p, "model_parallel", False):
                        p.sequence_parallel = True


class _GatherThenLinear(nn.Module):
    """Output projection at the end of a sequence-parallel region: gather the sequence, then project."""

    def __init__(self, linear: nn.Linear, dim: int):
        super().__init__()
        self.linear, self.dim = linear, dim

    @property
    def weight(self):
        return self.linear.weight

    def forward(self, x):
        return self.linear(M.gather_from_sequence_parallel_region(x, self.dim, False))


def _find_input_embedding(model: nn.Module):
    getter = getattr(model, "get_input_embeddings", None)
    target = getter() if callable(getter) else None
    for owner in model.modules():
        for name, child in owner.named_children():
            if child is target and target is not None:
                # scatter after the whole embedding block when there is one (BERT), else after wte
                return owner, name
    return None, None


def _find_output_projection(model: nn.Module):
    getter = getattr(model, "get_output_embeddings", None)
    target = getter() if callable(getter) else None
    if target is None:
        return None
    for owner in model.modules():
        for name, child in owner.named_children():
            if child is target:
                return owner, name
    return None


def apply_vocab_parallel(model: nn.Module, megatron_sp: bool = False, seq_dim: int = 1):
    """Embedding -> VocabParallelEmbedding, output projection -> column-parallel without gather
    (the loss must then be the vocab-parallel cross entropy)."""
    tp, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
    if tp == 1:
        return
    owner, name = _find_input_embedding(model)
    head = _find_output_projection(model)
    tied = False
    if owner is not None:
        emb = getattr(owner, name)
        inner = emb.inner if isinstance(emb, _SeqScatter) else emb
        if isinstance(inner, nn.Embedding) and inner.num_embeddings % tp == 0:
            if head is not None:
                h = getattr(head[0], head[1])
                tied = getattr(h, "weight", None) is inner.weight
            vpe = VocabParallelEmbedding(inner.num_embeddings, inner.embedding_dim, params_dtype=inner.weight.dtype,
                                         device="meta")
            if inner.weight.device.type != "meta":
                vpe.weight = nn.Parameter(inner.weight.data.chunk(tp, 0)[rank].contiguous())
                vpe.weight.model_parallel, vpe.weight.partition_dim = True, 0
            if isinstance(emb, _SeqScatter):
                emb.inner = vpe
            else:
                setattr(owner, name, vpe)
            new_emb = vpe
        else:
            new_emb = None
    else:
        new_emb = None
    if head is not None:
        h_owner, h_name = head
        h = getattr(h_owner, h_name)
        lin = h.linear if isinstance(h, _GatherThenLinear) else h
        if isinstance(lin, nn.Linear) and lin.out_features % tp == 0:
            cp = ColPara(lin, gather_output=False, sequence_parallel=False)
            if tied and new_emb is not None:
                cp.col_linear.weight = new_emb.weight
            if isinstance(h, _GatherThenLinear):
                h.linear = cp
            else:
                setattr(h_owner, h_name, cp)
    model.vocab_parallel = True
