"""Checkpoint naming, tracker files, format detection and state-dict key reconciliation
(Merak/core/checkpoint/utils.py:39-426).

On-disk layout (kept identical to the reference so checkpoints interchange and
``tools/convert_safetensor.py`` works on them):

    {output_dir}/{YYYY-MM-DD}_ckpt/
        latest_checkpointed_iteration.txt          # integer, or the word "release"
        iter_0000100/  (or release/)
            model_optim.pt                                     tp=1, pp=1
            mp_rank_{tp:02d}/partial_model_optim.pt            pp=1, tp>1
            mp_rank_{tp:02d}_pp_rank_{pp:03d}/partial_model_optim.pt
            zero_dp_rank_{dp:05d}[_mp_rank_{tp:02d}[_pp_rank_{pp:03d}]]_opt_states.pt   (ZeRO-1)
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..parallel import mpu

TRACKER = "latest_checkpointed_iteration.txt"


def iteration_dir(root: str, iteration, release: bool = False, best: bool = False) -> str:
    if best:
        return os.path.join(root, "best_model")
    if release or iteration == "release":
        return os.path.join(root, "release")
    return os.path.join(root, "iter_{:07d}".format(int(iteration)))


def get_checkpoint_name(root: str, iteration, release: bool = False, best: bool = False, lora: bool = False,
                        tp_rank: Optional[int] = None, pp_rank: Optional[int] = None,
                        tp_size: Optional[int] = None, pp_size: Optional[int] = None) -> str:
    tp_rank = mpu.get_model_parallel_rank() if tp_rank is None else tp_rank
    pp_rank = mpu.get_pipe_parallel_rank() if pp_rank is None else pp_rank
    tp_size = mpu.get_model_parallel_world_size() if tp_size is None else tp_size
    pp_size = mpu.get_pipe_parallel_world_size() if pp_size is None else pp_size
    d = iteration_dir(root, iteration, release, best)
    prefix = "lora_" if lora else ""
    if tp_size == 1 and pp_size == 1:
        return os.path.join(d, prefix + "model_optim.pt")
    if pp_size == 1:
        return os.path.join(d, "mp_rank_{:02d}".format(tp_rank), prefix + "partial_model_optim.pt")
    return os.path.join(d, "mp_rank_{:02d}_pp_rank_{:03d}".format(tp_rank, pp_rank), prefix + "partial_model_optim.pt")


def get_zero_checkpoint_name(root: str, iteration, release: bool = False, best: bool = False) -> str:
    d = iteration_dir(root, iteration, release, best)
    name = "zero_dp_rank_{:05d}".format(mpu.get_data_parallel_rank())
    tp, pp = mpu.get_model_parallel_world_size(), mpu.get_pipe_parallel_world_size()
    if tp > 1 or pp > 1:
        name += "_mp_rank_{:02d}".format(mpu.get_model_parallel_rank())
    if pp > 1:
        name += "_pp_rank_{:03d}".format(mpu.get_pipe_parallel_rank())
    return os.path.join(d, name + "_opt_states.pt")


def tracker_filename(root: str) -> str:
    return os.path.join(root, TRACKER)


def best_loss_filename(root: str) -> str:
    return os.path.join(root, "best_model_loss.txt")


def ensure_directory_exists(filename: str):
    os.makedirs(os.path.dirname(filename), exist_ok=True)


def read_metadata(tracker: str) -> Tuple[int, bool]:
    """Iteration stored in the tracker file; all ranks agree on the maximum they see."""
    with open(tracker) as f:
        text = f.read().strip()
    release = text == "release"
    iteration = 0 if release else int(text)
    if dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([iteration], dtype=torch.long)
        if dist.get_backend() == "nccl":
            t = t.cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        iteration = int(t.item())
    return iteration, release


def detect_checkpoint_format(path: str) -> str:
    """'merak' (tracker + iteration dirs), 'hf_bin', 'hf_safetensors', 'hf_safetensors_sharded',
    'adapter' or 'unknown'."""
    if os.path.isfile(os.path.join(path, TRACKER)):
        return "merak"
    if os.path.isfile(os.path.join(path, "model.safetensors.index.json")):
        return "hf_safetensors_sharded"
    if os.path.isfile(os.path.join(path, "model.safetensors")):
        return "hf_safetensors"
    if os.path.isfile(os.path.join(path, "pytorch_model.bin")):
        return "hf_bin"
    if os.path.isfile(os.path.join(path, "adapter_model.bin")):
        return "adapter"
    return "unknown"


def _split(key: str) -> List[str]:
    return key.split(".")


def check_state_dict(model_keys: List[str], ckpt: Dict[str, torch.Tensor]) -> Tuple[Dict[str, torch.Tensor], bool]:
    """Maps checkpoint keys onto the module's keys.  Exact match first; otherwise a module key
    ``"{idx}.{path}"`` matches a checkpoint key whose path equals ``path`` after dropping up to two
    leading components (``module.``, a different layer index ...), or one with the same layer-index
    digits and the same trailing components.  Returns (remapped dict, strict?)."""
    if set(model_keys) == set(ckpt.keys()):
        return ckpt, True
    out: Dict[str, torch.Tensor] = {}
    used = set()
    by_tail: Dict[str, List[str]] = {}
    for k in ckpt:
        parts = _split(k)
        for drop in range(0, 3):
            if len(parts) > drop:
                by_tail.setdefault(".".join(parts[drop:]), []).append(k)
    for mk in model_keys:
        if mk in ckpt:
            out[mk] = ckpt[mk]
            used.add(mk)
            continue
        parts = _split(mk)
        cands: List[str] = []
        for drop in (1, 0, 2):
            if len(parts) > drop:
                cands += by_tail.get(".".join(parts[drop:]), [])
        if not cands:
            digits = [p for p in parts if p.isdigit()]
            tail_n = 2 if len(parts) <= 3 else 4
            tail = parts[-tail_n:]
            for k in ckpt:
                kp = _split(k)
                if kp[-len(tail):] == tail and [p for p in kp if p.isdigit()][-len(digits[1:]):] == digits[1:]:
                    cands.append(k)
        cands = [c for c in cands if c not in used and ckpt[c].shape == ckpt[c].shape]
        if cands:
            out[mk] = ckpt[cands[0]]
            used.add(cands[0])
    strict = len(out) == len(model_keys) and len(used) == len(ckpt)
    return out, strict


def get_zero_param_shapes(module, flat) -> List[Dict[str, torch.Size]]:
    """name -> shape of every parameter in the flat buffer, in buffer order (one group)."""
    names = {id(p): n for n, p in module.named_parameters()}
    from collections import OrderedDict
    return [OrderedDict((names.get(id(p), "param%d" % i), p.shape) for i, p in enumerate(flat.params))]


class ShardedSafetensorLoader:
    """Lazy reader of a Hugging Face safetensors checkpoint (single file or index + shards).
    ``get(name)`` returns the full tensor; ``get_slice(name, dim, rank, world)`` the tensor-parallel
    slice (the reference loads full tensors only, so HF -> tp>1 was a gap there)."""

    def __init__(self, path: str):
        from safetensors import safe_open
        self._open = safe_open
        self.path = path
        index = os.path.join(path, "model.safetensors.index.json")
        if os.path.isfile(index):
            with open(index) as f:
                meta = json.load(f)
            self.weight_map = meta["weight_map"]
            self.tp_meta = meta.get("metadata", {}).get("tp_meta_data")
        else:
            fn = "model.safetensors"
            with safe_open(os.path.join(path, fn), framework="pt") as f:
                self.weight_map = {k: fn for k in f.keys()}
            self.tp_meta = None
        self._handles = {}

    def keys(self):
        return list(self.weight_map)

    def _file(self, name):
        fn = self.weight_map[name]
        if fn not in self._handles:
            self._handles[fn] = self._open(os.path.join(self.path, fn), framework="pt")
        return self._handles[fn]

    def get(self, name: str) -> torch.Tensor:
        return self._file(name).get_tensor(name)

    def get_slice(self, name: str, dim: int, rank: int, world: int) -> torch.Tensor:
        sl = self._file(name).get_slice(name)
        shape = sl.get_shape()
        per = shape[dim] // world
        idx = [slice(None)] * len(shape)
        idx[dim] = slice(rank * per, (rank + 1) * per)
        return sl[tuple(idx)]

    def state_dict(self, strip_prefix_components: int = 0) -> Dict[str, torch.Tensor]:
        out = {}
        for k in self.weight_map:
            parts = k.split(".")
            out[".".join(parts[strip_prefix_components:])] = self.get(k)
        return out
