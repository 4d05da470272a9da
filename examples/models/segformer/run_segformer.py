"""SegFormer image classification (examples/models/segformer): the Hugging Face ``SegformerForImageClassification`` with random weights on generated data.

    torchrun --nproc_per_node=4 --master-addr 127.0.0.1 examples/models/segformer/run_segformer.py \\
        --output_dir ./out --per_device_train_batch_size 4 --gradient_accumulation_steps 4 --max_steps 50
    PP=2 TP=2 ...   (degrees come from the environment; ``--tiny 1`` shrinks the model for a CPU run)
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import transformers as T  # noqa: E402
from _hf import run  # noqa: E402

# the tiny shape: per-stage lists; the generic scalar aliases of those fields are dropped (None)
TINY_SEGFORMER = dict(num_encoder_blocks=2, num_attention_heads=[1, 2], hidden_sizes=[16, 32], depths=[1, 1],
                      sr_ratios=[2, 1], patch_sizes=[3, 3], strides=[2, 2], decoder_hidden_size=32,
                      num_hidden_layers=None, hidden_size=None, num_layers=None)

if __name__ == "__main__":
    run(T.SegformerConfig, T.SegformerForImageClassification, mode="vision_only", tiny_overrides=TINY_SEGFORMER)
