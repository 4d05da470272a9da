"""Finding target modules, swapping in adapter layers, freezing everything else, and extracting the
adapter-only state dict (Merak/core/finetuning/lora/utils.py:69-150)."""
from __future__ import annotations

import re
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..parallel import mpu
from .config import LoraConfig
from .layer import Conv2d, Embedding, Linear, LoraLayer


def _is_target(name: str, targets: List[str], cfg: LoraConfig) -> bool:
    hit = any(name == t or name.endswith("." + t) for t in targets)
    if hit and cfg.layers_to_transform is not None:
        m = re.search(r"\.(\d+)\.", "." + name + ".")
        if m is None or int(m.group(1)) not in cfg.layers_to_transform:
            return False
    return hit


def find_and_replace(model: nn.Module, cfg: LoraConfig, adapter_name: str = "default",
                     model_type: Optional[str] = None) -> List[str]:
    targets = cfg.resolve_targets(model_type)
    replaced = []
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            full = (parent_name + "." if parent_name else "") + child_name
            # shard modules prefix names with the shard index and fx-flattened paths
            plain = re.sub(r"^\d+\.", "", full)
            if isinstance(child, LoraLayer) or not _is_target(plain.replace("_", "."), targets, cfg) and \
                    not _is_target(plain, targets, cfg):
                continue
            r = cfg.rank_pattern.get(child_name, cfg.r)
            alpha = cfg.alpha_pattern.get(child_name, cfg.lora_alpha)
            if isinstance(child, nn.Linear):
                new = Linear(child, adapter_name, r, alpha, cfg.lora_dropout, cfg.fan_in_fan_out, cfg.init_lora_weights)
            elif isinstance(child, nn.Embedding):
                new = Embedding(child, adapter_name, r, alpha, cfg.lora_dropout, cfg.init_lora_weights)
            elif isinstance(child, nn.Conv2d):
                new = Conv2d(child, adapter_name, r, alpha, cfg.lora_dropout, cfg.init_lora_weights)
            else:
                continue
            setattr(parent, child_name, new)
            replaced.append(full)
    if not replaced:
        raise ValueError("no module matched LoRA targets %s" % targets)
    return replaced


def mark_only_lora_as_trainable(model: nn.Module, bias: str = "none", modules_to_save=None):
    for n, p in model.named_parameters():
        p.requires_grad = "lora_" in n
    if bias == "all":
        for n, p in model.named_parameters():
            if n.endswith("bias"):
                p.requires_grad = True
    elif bias == "lora_only":
        for m in model.modules():
            if isinstance(m, LoraLayer) and getattr(m, "bias", None) is not None:
                m.bias.requires_grad = True
    for frag in modules_to_save or []:
        for n, p in model.named_parameters():
            if frag in n:
                p.requires_grad = True


def lora_state_dict(state_dict: Dict[str, torch.Tensor], bias: str = "none", modules_to_save=None):
    keep = {}
    for k, v in state_dict.items():
        if "lora_" in k or (bias == "all" and k.endswith("bias")) or any(f in k for f in (modules_to_save or [])):
            keep[k] = v
    return keep


def inject_lora(engine, cfg: LoraConfig, adapter_name: str = "default"):
    """Adds adapters to the engine's stage module and rebuilds the optimizer over the adapter
    parameters only (Merak/merak_trainer.py:387-390).  Tensor parallelism must be 1."""
    if mpu.get_model_parallel_world_size() != 1:
        raise ValueError("LoRA requires tensor parallel degree 1")
    module = engine.module
    model_type = getattr(module.config, "model_type", None)
    replaced = find_and_replace(module, cfg, adapter_name, model_type)
    mark_only_lora_as_trainable(module, cfg.bias, cfg.modules_to_save)
    module.lora_active, module.lora_config = True, cfg
    module.to(engine.device)
    params = [p for p in module.parameters() if p.requires_grad]
    for p in module.parameters():
        if hasattr(p, "main_grad") and not p.requires_grad:
            del p.main_grad
    engine._configure_optimizer(None, None, None, getattr(engine, "_lr_scheduler_factory", None), params)
    return replaced
