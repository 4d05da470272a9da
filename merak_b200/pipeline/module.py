"""``PipelineModule``: the part of a model one pipeline stage owns.

Construction (Merak/core/pipeline/module.py:69-256): cast to the compute dtype -> apply the
tensor-parallel transform on the module tree -> trace and shard the model into a sequence of
sub-graphs -> assign shards to stages -> keep this stage's shards, registered under their global
index (``self._modules[str(idx)]``, which is what gives checkpoint keys their
``"{layer_idx}.{module.path}.{param}"`` form) -> discover weights shared between stages (tied
embeddings) -> configure activation recomputation.

``forward`` runs the local shards in order, wrapping ranges of them in ``checkpoint`` /
``pre_checkpoint`` according to the recompute configuration: off, every ``n`` shards, explicit
boundaries, or the stage-aware ratio (``activation_checkpoint_ratio``) under which later stages,
which hold fewer in-flight micro-batches in 1F1B, recompute a smaller share of their layers
(Merak/core/pipeline/module.py:217-238,420-567).
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..fx.convert import convert_to_sequential
from ..parallel import mpu
from ..parallel.tp_transform import apply_tensor_parallel
from ..recompute import checkpoint, get_rng_tracker, pre_checkpoint
from .partition import LayerPartition, partition_balanced


def stage_aware_ratios(r0: float, stages: int) -> List[float]:
    """``ratio[i] = 1 - (1-r0)(S-1)/(S-1-i)`` for ``i < S-1`` and 0 for the last stage; negative
    values mean "no recomputation on that stage" (Merak/core/pipeline/module.py:220-232)."""
    if stages == 1:
        return [max(0.0, r0)]
    out = []
    for i in range(stages - 1):
        out.append(max(0.0, 1.0 - (1.0 - r0) * (stages - 1) / (stages - 1 - i)))
    out.append(0.0)
    return out


class PipelineModule(nn.Module):

    def __init__(self, model: nn.Module, args, loss_fn: Optional[Callable] = None, topology=None,
                 communicaiton_grid=None, activation_checkpoint_func: Callable = checkpoint,
                 leaf_modules: Iterable[type] = (), dummy_inputs: Optional[Dict[str, torch.Tensor]] = None,
                 layers: Optional[Sequence[nn.Module]] = None):
        super().__init__()
        self.args = args
        self.loss_fn = loss_fn
        self.act_ckpt_func = activation_checkpoint_func
        self._default_ckpt_func = activation_checkpoint_func
        self.num_stages = mpu.get_pipe_parallel_world_size()
        self.stage_id = mpu.get_pipe_parallel_rank()
        self.config = getattr(model, "config", None)
        self.tied_specs: Dict[str, dict] = {}
        self.tie_groups: Dict[str, object] = {}
        self.pending_records: Dict[int, list] = {}
        self.current_buffer: Optional[int] = None

        if args.params_dtype is not None and args.params_dtype != torch.float32 and model is not None:
            model.to(args.params_dtype)
        tp = mpu.get_model_parallel_world_size()
        from ..parallel import fused_tp
        fused_tp.ENABLED = getattr(args, "comm_mode", "fused") == "fused"
        from ..parallel import expert as _expert
        _expert.FUSED_ENABLED = fused_tp.ENABLED
        if tp > 1 and model is not None:
            apply_tensor_parallel(model, megatron_sp=getattr(args, "megatron_sequence_parallel", False),
                                  seq_dim=args.sequence_dim, vocab_parallel=args.parallel_vocab)
        if tp > 1 and model is not None and getattr(args, "tp_overlapping_level", 0) > 0:
            from ..fx.tracer import framework_leaf_classes
            from ..parallel.tp_overlap import apply_tp_overlap
            blocks = tuple(c for c in framework_leaf_classes() if c.__name__.endswith(("Block", "DecoderLayer", "BertLayer")))
            apply_tp_overlap(model, args.tp_overlapping_level, getattr(args, "comm_mode", "nccl"), blocks)
        if getattr(args, "sequence_parallel", False) and mpu.get_sequence_parallel_world_size() > 1:
            from ..parallel.ulysses import replace_to_sp_module
            replace_to_sp_module(model, args)

        if layers is not None:
            self.all_layers = list(layers)
            self.input_to_shard = {n: 0 for n in (args.input_names or ["input_ids"])}
        else:
            _, self.all_layers, self.input_to_shard = convert_to_sequential(model, args, dummy_inputs, leaf_modules)
        self.num_layers_total = len(self.all_layers)
        self.static_batch_size = getattr(self.all_layers[0], "static_batch_size", None) if self.all_layers else None
        self.param_counts = [sum(p.numel() for p in l.parameters()) for l in self.all_layers]
        self.parts = self._partition()
        self.local_start, self.local_stop = self.parts[self.stage_id], self.parts[self.stage_id + 1]
        self._find_tied(model)
        self._build()
        self._configure_recompute()
        # shards of other stages are dropped so their parameters can be freed
        kept = set(range(self.local_start, self.local_stop))
        self.all_layers = [l if i in kept else None for i, l in enumerate(self.all_layers)]

    # ------------------------------------------------------------------------------------------
    def _partition(self) -> List[int]:
        return LayerPartition(self.args, self.all_layers, self.num_stages, self.param_counts).partition()

    def stage_owner(self, layer_idx: int) -> int:
        for s in range(self.num_stages):
            if self.parts[s] <= layer_idx < self.parts[s + 1]:
                return s
        raise IndexError(layer_idx)

    def _find_tied(self, model):
        """Parameters that appear in shards of more than one stage (tied embeddings).  Keyed by
        object identity; the checkpoint name keeps the reference's ``tied_modules.<shape>`` form."""
        if getattr(self.args, "no_tie_modules", False):
            return
        owners: Dict[int, dict] = {}
        for idx, layer in enumerate(self.all_layers):
            for name, p in layer.named_parameters():
                rec = owners.setdefault(id(p), {"param": p, "uses": []})
                rec["uses"].append((idx, name))
        for rec in owners.values():
            stages = sorted({self.stage_owner(i) for i, _ in rec["uses"]})
            if len(stages) > 1:
                key = "x".join(str(d) for d in rec["param"].shape)
                self.tied_specs[key] = {"stages": stages, "uses": rec["uses"], "param": rec["param"]}

    def _build(self):
        self.local_layers: List[nn.Module] = []
        for idx in range(self.local_start, self.local_stop):
            layer = self.all_layers[idx]
            self.add_module(str(idx), layer)
            self.local_layers.append(layer)
        self.input_to_stage_dic: Dict[int, List[str]] = {}
        for name, shard in self.input_to_shard.items():
            self.input_to_stage_dic.setdefault(self.stage_owner(shard) if self.num_layers_total else 0, []).append(name)
        for p in self.parameters():
            if not hasattr(p, "model_parallel"):
                p.model_parallel = False
        # local copies of tied weights on non-owning stages are kept in sync by the engine
        self.tied_local = {k: v for k, v in self.tied_specs.items() if self.stage_id in v["stages"]}

    def is_checkpointable(self, layer: nn.Module) -> bool:
        """Embedding-only and parameter-free shards are not worth recomputing."""
        params = list(layer.parameters())
        if not params:
            return False
        mods = [m for m in layer.modules() if len(list(m.children())) == 0 and list(m.parameters(recurse=False))]
        return not all(isinstance(m, nn.Embedding) or "Embedding" in type(m).__name__ for m in mods)

    def _configure_recompute(self):
        a = self.args
        n_local = len(self.local_layers)
        self.ckpt_ratio: Optional[float] = None
        self.ckpt_boundaries: Optional[List[int]] = None
        self.act_ckpt_interval = a.checkpoint_num_layers if a.activation_checkpointing else 0
        if not a.activation_checkpointing:
            return
        if a.activation_checkpoint_ratio:
            vals = [float(v) for v in a.activation_checkpoint_ratio]
            if len(vals) == 1:
                ratios = stage_aware_ratios(vals[0], self.num_stages)
            else:
                ratios = vals + [vals[-1]] * max(0, self.num_stages - len(vals))
            self.stage_ratios = ratios
            self.ckpt_ratio = ratios[self.stage_id]
            if self.ckpt_ratio <= 0:
                self.act_ckpt_interval = 0
                self.ckpt_ratio = None
            return
        if a.split_method == "nearest_min_deps" and n_local > 1 and a.num_layers:
            # recompute granularity of about one transformer layer: parameter-balanced boundaries
            groups = max(1, min(n_local, a.num_layers // max(1, self.num_stages)))
            counts = self.param_counts[self.local_start:self.local_stop]
            if sum(counts) > 0 and groups > 1:
                self.ckpt_boundaries = partition_balanced(counts, groups)

    # ------------------------------------------------------------------------------------------
    def _run_range(self, lo: int, hi: int):
        layers = self.local_layers[lo:hi]
        externals = self._externals

        hook = getattr(self, "layer_input_hook", None)

        def run(*carried):
            for k, layer in enumerate(layers):
                if hook is not None and torch.is_grad_enabled():
                    hook(lo + k, carried)             # the engine watches for this layer's input gradient
                ext = [externals[n] for n in getattr(layer, "external_inputs", [])]
                out = layer(*carried, *ext)
                carried = out if isinstance(out, tuple) else (out,)
            return carried if len(carried) > 1 else carried[0]
        return run

    def _ckpt(self, fn, *x):
        if self.act_ckpt_func is pre_checkpoint:
            recs = self.pending_records.setdefault(self.current_buffer if self.current_buffer is not None else -1, [])
            return pre_checkpoint(fn, *x, record_list=recs)
        return self.act_ckpt_func(fn, *x)

    def forward(self, carried: Tuple[torch.Tensor, ...], externals: Optional[Dict[str, torch.Tensor]] = None):
        """``carried``: tensors arriving from the previous stage (empty on the first stage);
        ``externals``: model inputs this stage reads itself.  Returns the tuple for the next stage, or
        the model output on the last stage."""
        self._externals = externals or {}
        n = len(self.local_layers)
        x = tuple(carried)
        fork = mpu.get_model_parallel_world_size() > 1 or mpu.get_sequence_parallel_world_size() > 1
        ctx = get_rng_tracker().fork() if fork and get_rng_tracker().get_states() else _null()
        with ctx:
            ranges = self._recompute_ranges(n)
            for lo, hi, ckpt in ranges:
                fn = self._run_range(lo, hi)
                needs_grad = torch.is_grad_enabled()
                # a checkpointed segment needs an input that carries gradient, or autograd would
                # never reach the parameters inside it
                if ckpt and needs_grad and x and all(isinstance(t, torch.Tensor) for t in x) and \
                        any(t.requires_grad for t in x):
                    out = self._ckpt(fn, *x)
                else:
                    out = fn(*x)
                x = out if isinstance(out, tuple) else (out,)
        self._externals = {}
        if self.stage_id == self.num_stages - 1:
            return x[0] if len(x) == 1 else x
        return x

    def _recompute_ranges(self, n: int) -> List[Tuple[int, int, bool]]:
        """List of (lo, hi, checkpointed) covering the local shards."""
        last_stage = self.stage_id == self.num_stages - 1
        if self.act_ckpt_interval == 0 or not self.training:
            return [(0, n, False)]
        ok = [self.is_checkpointable(l) for l in self.local_layers]
        out: List[Tuple[int, int, bool]] = []
        if self.ckpt_ratio is not None:
            free = n - int(n * self.ckpt_ratio)          # leading shards that keep their activations
            bounds = list(range(0, n + 1))
            for lo, hi in zip(bounds, bounds[1:]):
                out.append((lo, hi, lo >= free and ok[lo]))
        elif self.ckpt_boundaries is not None:
            b = self.ckpt_boundaries
            for lo, hi in zip(b, b[1:]):
                if hi > lo:
                    out.append((lo, hi, any(ok[lo:hi])))
        else:
            step = max(1, self.act_ckpt_interval)
            for lo in range(0, n, step):
                hi = min(n, lo + step)
                out.append((lo, hi, any(ok[lo:hi])))
        if last_stage and out:
            lo, hi, _ = out[-1]
            out[-1] = (lo, hi, False)       # the tail of the last stage feeds the loss directly
        # leading shards that are not worth recomputing (embeddings) run outside the segment
        peeled: List[Tuple[int, int, bool]] = []
        for lo, hi, ck in out:
            while ck and lo < hi and not ok[lo]:
                peeled.append((lo, lo + 1, False))
                lo += 1
            if lo < hi:
                peeled.append((lo, hi, ck))
        out = peeled
        # merge neighbouring non-checkpointed ranges
        merged: List[Tuple[int, int, bool]] = []
        for r in out:
            if merged and not merged[-1][2] and not r[2]:
                merged[-1] = (merged[-1][0], r[1], False)
            else:
                merged.append(r)
        return merged

    # ------------------------------------------------------------------------------------------
    def set_recompute(self, func: Optional[Callable] = None, interval: Optional[int] = None):
        if func is not None:
            self.act_ckpt_func = func
        if interval is not None:
            self.act_ckpt_interval = interval

    def restore_recompute(self):
        self.act_ckpt_func = self._default_ckpt_func
        self.act_ckpt_interval = (self.args.checkpoint_num_layers if self.args.activation_checkpointing else 0)
        if getattr(self, "_force_no_recompute", False):
            self.act_ckpt_interval = 0

    def configure_distributed_model(self, device):
        if any(p.device.type == "meta" for p in self.parameters()):
            # the model was built under ``init_empty_weights``: only this stage's (tensor-parallel
            # slices of the) parameters are ever allocated, directly on the training device
            from ..utils.device_to_meta import materialize_meta
            std = float(getattr(self.config, "initializer_range", 0.02) or 0.02)
            materialize_meta(self, device, init_std=std)
            for spec in self.tied_local.values():          # the tied tensors are new objects now
                for idx, name in spec["uses"]:
                    if self.local_start <= idx < self.local_stop:
                        spec["param"] = dict(self.all_layers[idx].named_parameters())[name]
                        break
        self.to(device)
        self._broadcast_model()

    def _broadcast_model(self):
        """Rank 0 of every data-parallel group sends its parameters to the others
        (Merak/core/pipeline/module.py:377-391)."""
        group, n = mpu.get_data_parallel_group(), mpu.get_data_parallel_world_size()
        if n == 1:
            return
        src = mpu.get_data_parallel_ranks()[0]
        ep = mpu.get_expert_parallel_world_size()
        for p in self.parameters():
            if ep > 1 and getattr(p, "expert_parallel", False):
                continue        # every rank of the expert-parallel group holds different experts
            dist.broadcast(p.data, src, group=group)

    # -- tied weights ------------------------------------------------------------------------------
    def tie_modules(self):
        """One process group per tied weight spanning the stages that hold a copy (same dp/tp
        coordinates), then a broadcast from the first owner (Merak/core/pipeline/module.py:601-696)."""
        grid = mpu.get_grid()
        if grid is None or not self.tied_specs or self.num_stages == 1:
            return
        for key in sorted(self.tied_specs):
            spec = self.tied_specs[key]
            my_group = None
            topo = grid.topology
            for dp in range(grid.data_parallel_size):
                for sp in range(grid.sequence_parallel_size):
                    for tp in range(grid.model_parallel_size):
                        ranks = sorted(topo.get_rank(pipe=s, data=dp, sequence=sp, model=tp) for s in spec["stages"])
                        g = dist.new_group(ranks=ranks)
                        if grid.global_rank in ranks:
                            my_group, spec["ranks"] = g, ranks
            self.tie_groups[key] = my_group
        self._synchronize_tied_weights()

    def _synchronize_tied_weights(self):
        for key, spec in self.tied_local.items():
            g = self.tie_groups.get(key)
            if g is not None:
                dist.broadcast(spec["param"].data, spec["ranks"][0], group=g)

    def allreduce_tied_weight_gradients(self):
        for key, spec in self.tied_local.items():
            g = self.tie_groups.get(key)
            if g is None:
                continue
            p = spec["param"]
            grad = getattr(p, "main_grad", None)
            if grad is None:
                grad = p.grad
            if grad is not None:
                dist.all_reduce(grad, group=g)

    def state_dict_for_checkpoint(self):
        sd = self.state_dict()
        for key, spec in self.tied_local.items():
            sd["tied_modules." + key + ".weight"] = spec["param"].detach()
        return sd


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
