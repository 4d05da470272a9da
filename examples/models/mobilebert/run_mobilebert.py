"""MobileBERT masked language modelling (examples/models/mobilebert): the Hugging Face ``MobileBertForMaskedLM`` with random weights on generated data.

    torchrun --nproc_per_node=4 --master-addr 127.0.0.1 examples/models/mobilebert/run_mobilebert.py \\
        --output_dir ./out --per_device_train_batch_size 4 --gradient_accumulation_steps 4 --max_steps 50
    PP=2 TP=2 ...   (degrees come from the environment; ``--tiny 1`` shrinks the model for a CPU run)
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import transformers as T  # noqa: E402
from _hf import run  # noqa: E402

if __name__ == "__main__":
    run(T.MobileBertConfig, T.MobileBertForMaskedLM, mode="text_only",
        tiny_overrides=dict(embedding_size=64, use_bottleneck=False))
