"""Saving, loading and rotating checkpoints (Merak/core/checkpoint/checkpoint.py:71-853).

One model file per (tensor-parallel rank, pipeline stage), written by data-parallel rank 0; with
ZeRO-1 every data-parallel rank adds its optimizer shard.  File content (same keys as the
reference): ``args, checkpoint_version (3.0), iteration, model, optimizer, lr_scheduler,
random_rng_state, np_rng_state, torch_rng_state, cuda_rng_state, rng_tracker_states``.  Model keys
are ``"{global_shard_idx}.{module.path}.{param}"`` with ``col_linear.`` / ``row_linear.`` inserted
by tensor-parallel layers and ``tied_modules.{shape}.weight`` entries for weights shared between
stages.
"""
from __future__ import annotations

import datetime
import json
import os
import re
import random
import shutil
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..ops.rng import dropout_state
from ..parallel import mpu
from ..printer import log_dist, logger
from ..recompute import get_rng_tracker
from . import utils as U

CHECKPOINT_VERSION = 3.0


def _barrier():
    if dist.is_initialized():
        dist.barrier()


def _is_rank0():
    return not dist.is_initialized() or dist.get_rank() == 0


class CheckpointSaver:

    def __init__(self, args):
        self.args = args
        self.date = datetime.date.today().strftime("%Y-%m-%d")
        self.root_dir = os.path.join(args.output_dir, "%s_ckpt" % self.date)
        self.best_root = os.path.join(args.output_dir, "best_ckpt")
        self.best_loss = float("inf")

    def _model_state(self, module):
        if hasattr(module, "state_dict_for_checkpoint"):
            return module.state_dict_for_checkpoint()
        return module.state_dict()

    def save_checkpoint(self, iteration: int, model, optimizer=None, lr_scheduler=None, engine=None,
                        best_model: bool = False, loss: Optional[float] = None, release: bool = False, **kwargs):
        a = self.args
        root = self.best_root if best_model else self.root_dir
        if best_model and loss is not None:
            if loss >= self.best_loss:
                return None
            self.best_loss = loss
        lora = bool(getattr(model, "lora_active", False))
        name = U.get_checkpoint_name(root, iteration, release=release, best=best_model, lora=lora)
        zero = bool(engine is not None and getattr(engine, "zero", False))
        if mpu.get_data_parallel_rank() == 0:
            U.ensure_directory_exists(name)
            sd = {"args": a, "checkpoint_version": CHECKPOINT_VERSION, "iteration": iteration}
            model_sd = self._model_state(model)
            if lora:
                from ..lora import lora_state_dict
                model_sd = lora_state_dict(model_sd)
                cfg = getattr(model, "lora_config", None)
                if cfg is not None:
                    with open(os.path.join(os.path.dirname(name), "lora_config.json"), "w") as f:
                        json.dump(cfg.to_dict(), f, indent=2)
            sd["model"] = {k: v.detach().cpu() for k, v in model_sd.items()}
            if not a.no_save_optim and not zero and optimizer is not None:
                sd["optimizer"] = _cpu(optimizer.state_dict())
            if lr_scheduler is not None and not a.no_save_optim:
                sd["lr_scheduler"] = lr_scheduler.state_dict()
            if not a.no_save_rng:
                sd["random_rng_state"] = random.getstate()
                sd["np_rng_state"] = np.random.get_state()
                sd["torch_rng_state"] = torch.get_rng_state()
                sd["cuda_rng_state"] = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
                sd["rng_tracker_states"] = get_rng_tracker().get_states()
                sd["dropout_state"] = dropout_state().state_dict()
            if engine is not None and engine.loss_scaler is not None:
                sd["loss_scaler"] = engine.loss_scaler.state_dict()
            torch.save(sd, name, _use_new_zipfile_serialization=False)
        if zero and not a.no_save_optim:
            zname = U.get_zero_checkpoint_name(root, iteration, release=release, best=best_model)
            U.ensure_directory_exists(zname)
            torch.save({"optimizer_state_dict": _cpu(optimizer.state_dict()),
                        "param_shapes": U.get_zero_param_shapes(model, engine.flat)}, zname,
                       _use_new_zipfile_serialization=False)
        if engine is not None and getattr(engine, "flat_expert", None) is not None:
            # expert-parallel parameters differ per rank of the expert-parallel group: one file each
            ename = _expert_file(name)
            U.ensure_directory_exists(ename)      # dp ranks > 0 may get here before dp rank 0 made it
            esd = {"model": {k: v.detach().cpu() for k, v in model.state_dict().items() if _is_expert_key(model, k)}}
            if not a.no_save_optim:
                esd["optimizer"] = _cpu(engine.optimizer_expert.state_dict())
            torch.save(esd, ename, _use_new_zipfile_serialization=False)
        _barrier()
        if _is_rank0():
            if best_model:
                with open(U.best_loss_filename(self.best_root), "w") as f:
                    f.write(str(loss))
            else:
                with open(U.tracker_filename(root), "w") as f:
                    f.write("release" if release else str(iteration))
            log_dist("saved checkpoint at iteration %s to %s" % (iteration, os.path.dirname(name)), ranks=[0])
        _barrier()
        return name


def _expert_file(name: str) -> str:
    """File of this rank's experts next to the model file ``name``."""
    return os.path.join(os.path.dirname(name), "expert_parallel_rank_{:02d}_states.pt".format(
        mpu.get_expert_parallel_rank()))


def _is_expert_key(model, key: str) -> bool:
    p = dict(model.named_parameters()).get(key)
    return p is not None and getattr(p, "expert_parallel", False)


def _cpu(obj):
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_cpu(v) for v in obj)
    return obj


class CheckpointLoader:

    def __init__(self, args):
        self.args = args

    def load_checkpoint(self, model, optimizer=None, lr_scheduler=None, path: Optional[str] = None, engine=None,
                        peft_config=None, verbose: bool = True, strict: bool = True) -> int:
        """Returns the iteration to resume from (0 for release / Hugging Face checkpoints)."""
        a = self.args
        path = path or a.resume_from_checkpoint
        fmt = U.detect_checkpoint_format(path)
        if fmt == "unknown":
            # a dated root may have been given one level up
            subs = sorted(d for d in os.listdir(path) if d.endswith("_ckpt")) if os.path.isdir(path) else []
            if subs:
                path = os.path.join(path, subs[-1])
                fmt = U.detect_checkpoint_format(path)
        if fmt in ("hf_bin", "hf_safetensors", "hf_safetensors_sharded"):
            self._load_hf(model, path, fmt)
            return 0
        if fmt != "merak":
            raise FileNotFoundError("no checkpoint found under %r" % path)
        iteration, release = U.read_metadata(U.tracker_filename(path))
        lora = bool(getattr(model, "lora_active", False))
        name = U.get_checkpoint_name(path, iteration, release=release, lora=lora)
        if not os.path.isfile(name) and lora:
            name = U.get_checkpoint_name(path, iteration, release=release, lora=False)
        sd = torch.load(name, map_location="cpu", weights_only=False)
        model_sd = sd["model"]
        keys = list(model.state_dict().keys())
        tied = {k: v for k, v in model_sd.items() if k.startswith("tied_modules.")}
        model_sd = {k: v for k, v in model_sd.items() if not k.startswith("tied_modules.")}
        mapped, is_strict = U.check_state_dict(keys, model_sd)
        missing, unexpected = model.load_state_dict(mapped, strict=False)
        if (missing or unexpected) and verbose and not lora:
            log_dist("checkpoint load: %d missing, %d unexpected keys" % (len(missing), len(unexpected)), ranks=[-1])
        if strict and is_strict and (missing or unexpected):
            raise RuntimeError("state dict mismatch: missing %s unexpected %s" % (missing[:5], unexpected[:5]))
        for key, spec in getattr(model, "tied_local", {}).items():
            t = tied.get("tied_modules." + key + ".weight")
            if t is not None:
                spec["param"].data.copy_(t)
        finetune = a.finetune or release
        esd = None
        if engine is not None and getattr(engine, "flat_expert", None) is not None and os.path.isfile(_expert_file(name)):
            esd = torch.load(_expert_file(name), map_location="cpu", weights_only=False)
            own = dict(model.state_dict())
            for k, v in esd["model"].items():
                if k in own:
                    own[k].copy_(v)
            if not finetune and not a.no_load_optim and "optimizer" in esd:
                engine.optimizer_expert.load_state_dict(_to_device(esd["optimizer"], _device_of(model)))
            else:
                eo = engine.optimizer_expert
                eo.master.copy_(eo.flat.model[eo.start:eo.end].float())
        if not finetune and not a.no_load_optim:
            zero = bool(engine is not None and getattr(engine, "zero", False))
            if zero:
                zname = U.get_zero_checkpoint_name(path, iteration, release=release)
                zsd = torch.load(zname, map_location="cpu", weights_only=False)
                optimizer.load_state_dict(_to_device(zsd["optimizer_state_dict"], _device_of(model)))
            elif optimizer is not None and "optimizer" in sd:
                optimizer.load_state_dict(_to_device(sd["optimizer"], _device_of(model)))
            elif optimizer is not None and hasattr(optimizer, "master"):
                optimizer.master.copy_(optimizer.flat.model[optimizer.start:optimizer.end].float())
            if lr_scheduler is not None and "lr_scheduler" in sd:
                lr_scheduler.load_state_dict(sd["lr_scheduler"])
            if engine is not None and engine.loss_scaler is not None and "loss_scaler" in sd:
                engine.loss_scaler.load_state_dict(sd["loss_scaler"])
        elif optimizer is not None and hasattr(optimizer, "master"):
            optimizer.master.copy_(optimizer.flat.model[optimizer.start:optimizer.end].float())
        if not finetune and not a.no_load_rng and "torch_rng_state" in sd:
            random.setstate(sd["random_rng_state"])
            np.random.set_state(sd["np_rng_state"])
            torch.set_rng_state(sd["torch_rng_state"])
            if sd.get("cuda_rng_state") is not None and torch.cuda.is_available():
                torch.cuda.set_rng_state(sd["cuda_rng_state"])
            if sd.get("rng_tracker_states"):
                get_rng_tracker().set_states(sd["rng_tracker_states"])
            if sd.get("dropout_state"):
                dropout_state().load_state_dict(sd["dropout_state"])
        _barrier()
        if verbose:
            log_dist("loaded checkpoint %s (iteration %s)" % (name, iteration), ranks=[0])
        return 0 if finetune else iteration

    def _load_hf(self, model, path: str, fmt: str):
        """Hugging Face weights as a release checkpoint: keys are matched by their path below the
        shard index; tensor-parallel layers take their slice of the full tensor."""
        if fmt == "hf_bin":
            full = torch.load(os.path.join(path, "pytorch_model.bin"), map_location="cpu", weights_only=False)
            getter = lambda k: full[k]
            names = list(full)
        else:
            loader = U.ShardedSafetensorLoader(path)
            getter = loader.get
            names = loader.keys()
        tp, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
        target = model.state_dict()
        loaded = 0
        # Hugging Face GPT-2 stores its projections as Conv1D ([in, out]); this framework's are [out, in]
        conv1d = False
        cfg_file = os.path.join(path, "config.json")
        if os.path.isfile(cfg_file):
            with open(cfg_file) as f:
                conv1d = json.load(f).get("model_type") == "gpt2"
        fused_parts = {"c_attn": 3, "qkv": 3, "qkv_proj": 3, "gate_up_proj": 2}
        for key, dst in target.items():
            parts = key.split(".")
            body = ".".join(parts[1:]) if parts[0].isdigit() else key
            plain = body.replace("col_linear.", "").replace("row_linear.", "")
            src_name = plain if plain in names else next((n for n in names if n.endswith("." + plain)), None)
            if src_name is None:
                continue
            t = getter(src_name)
            if conv1d and t.dim() == 2 and re.search(r"\.(c_attn|c_proj|c_fc)\.weight$", plain):
                t = t.t().contiguous()
            if t.shape != dst.shape and tp > 1:
                nfused = next((v for k, v in fused_parts.items() if ("." + k + ".") in ("." + plain)), 1)
                if "col_linear" in key and nfused > 1 and t.shape[0] % (nfused * tp) == 0:
                    # fused [q; k; v] / [gate; up] rows: every part is split on its own
                    t = torch.cat([part.chunk(tp, 0)[rank] for part in t.chunk(nfused, 0)], 0)
                elif "col_linear" in key or (t.dim() >= 1 and t.shape[0] == dst.shape[0] * tp):
                    t = t.chunk(tp, 0)[rank]
                elif "row_linear" in key and t.dim() == 2:
                    t = t.chunk(tp, 1)[rank]
            if t.shape == dst.shape:
                dst.copy_(t)
                loaded += 1
        log_dist("loaded %d/%d tensors from Hugging Face checkpoint %s" % (loaded, len(target), path), ranks=[0])
        _barrier()


def _device_of(model):
    try:
        return next(model.parameters()).device
    except StopIteration:
        return torch.device("cpu")


def _to_device(obj, device):
    if isinstance(obj, torch.Tensor):
        return obj.to(device)
    if isinstance(obj, dict):
        return {k: _to_device(v, device) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_device(v, device) for v in obj)
    return obj


def _sorted_checkpoints(root: str):
    if not os.path.isdir(root):
        return []
    dirs = [d for d in os.listdir(root) if d.startswith("iter_") and os.path.isdir(os.path.join(root, d))]
    return sorted(dirs, key=lambda d: int(d.split("_")[1]))


def rotate_checkpoints(args, root: str):
    """Keeps the newest ``save_total_limit`` iteration directories (Merak/core/checkpoint/checkpoint.py:804-853)."""
    limit = getattr(args, "save_total_limit", -1)
    if limit is None or limit <= 0:
        return
    if _is_rank0():
        ckpts = _sorted_checkpoints(root)
        for d in ckpts[:-limit] if len(ckpts) > limit else []:
            shutil.rmtree(os.path.join(root, d), ignore_errors=True)
    _barrier()
