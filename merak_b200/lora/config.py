"""LoRA configuration (Merak/core/finetuning/lora/config.py:67-184) and default target modules per
model type (Merak/core/finetuning/lora/mappings.py:22-55)."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Union

DEFAULT_TARGET_MODULES: Dict[str, List[str]] = {
    "t5": ["q", "v"], "mt5": ["q", "v"], "bart": ["q_proj", "v_proj"], "gpt2": ["c_attn"],
    "bloom": ["query_key_value"], "blip-2": ["q", "v", "q_proj", "v_proj"], "opt": ["q_proj", "v_proj"],
    "gptj": ["q_proj", "v_proj"], "gpt_neox": ["query_key_value"], "gpt_neo": ["q_proj", "v_proj"],
    "bert": ["query", "value", "qkv"], "roberta": ["query", "value"], "xlm-roberta": ["query", "value"],
    "electra": ["query", "value"], "deberta-v2": ["query_proj", "value_proj"], "deberta": ["in_proj"],
    "layoutlm": ["query", "value"], "llama": ["q_proj", "v_proj", "qkv_proj"], "chatglm": ["query_key_value"],
    "gpt_bigcode": ["c_attn"], "mpt": ["Wqkv"], "RefinedWebModel": ["query_key_value"],
    "RefinedWeb": ["query_key_value"], "falcon": ["query_key_value"], "btlm": ["c_proj", "c_attn"],
    "codegen": ["qkv_proj"], "mistral": ["q_proj", "v_proj"], "mixtral": ["q_proj", "v_proj"],
    "stablelm": ["q_proj", "v_proj"], "phi": ["q_proj", "v_proj", "fc1", "fc2"], "gemma": ["q_proj", "v_proj"],
    "qwen2": ["q_proj", "v_proj", "qkv_proj"], "vit": ["query", "value"],
}


@dataclass
class LoraConfig:
    r: int = 8
    target_modules: Optional[Union[List[str], str]] = None
    lora_alpha: int = 8
    lora_dropout: float = 0.0
    fan_in_fan_out: bool = False
    bias: str = "none"                       # none | all | lora_only
    modules_to_save: Optional[List[str]] = None
    init_lora_weights: bool = True
    layers_to_transform: Optional[Union[List[int], int]] = None
    layers_pattern: Optional[Union[List[str], str]] = None
    rank_pattern: Dict[str, int] = field(default_factory=dict)
    alpha_pattern: Dict[str, int] = field(default_factory=dict)
    peft_type: str = "LORA"
    task_type: Optional[str] = None
    inference_mode: bool = False

    def __post_init__(self):
        if self.bias not in ("none", "all", "lora_only"):
            raise ValueError("bias must be none, all or lora_only")
        if isinstance(self.layers_to_transform, int):
            self.layers_to_transform = [self.layers_to_transform]

    def to_dict(self):
        return asdict(self)

    @classmethod
    def from_json_file(cls, path: str) -> "LoraConfig":
        with open(path) as f:
            data = json.load(f)
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in data.items() if k in known})

    def resolve_targets(self, model_type: Optional[str]) -> List[str]:
        if self.target_modules:
            return [self.target_modules] if isinstance(self.target_modules, str) else list(self.target_modules)
        if model_type in DEFAULT_TARGET_MODULES:
            return DEFAULT_TARGET_MODULES[model_type]
        raise ValueError("please set target_modules: no default for model type %r" % model_type)
