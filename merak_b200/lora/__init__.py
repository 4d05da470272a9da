from .config import DEFAULT_TARGET_MODULES, LoraConfig
from .layer import Conv2d, Embedding, Linear, LoraLayer
from .utils import find_and_replace, inject_lora, lora_state_dict, mark_only_lora_as_trainable
