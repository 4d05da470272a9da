"""Swin Transformer image classification (examples/models/swin): the Hugging Face ``SwinForImageClassification`` with random weights on generated data.

    torchrun --nproc_per_node=4 --master-addr 127.0.0.1 examples/models/swin/run_swin.py \\
        --output_dir ./out --per_device_train_batch_size 4 --gradient_accumulation_steps 4 --max_steps 50
    PP=2 TP=2 ...   (degrees come from the environment; ``--tiny 1`` shrinks the model for a CPU run)
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import transformers as T  # noqa: E402
from _hf import run  # noqa: E402

# the tiny shape: per-stage lists; the generic scalar aliases of those fields are dropped (None)
TINY_SWIN = dict(num_heads=[2, 4], depths=[1, 1], embed_dim=16, window_size=2, patch_size=4,
                 num_attention_heads=None, num_hidden_layers=None, num_layers=None, hidden_size=None)

if __name__ == "__main__":
    run(T.SwinConfig, T.SwinForImageClassification, mode="vision_only", tiny_overrides=TINY_SWIN)
