"""MarianMT translation (examples/models/marianmt): the Hugging Face ``MarianMTModel`` with random weights on generated data.

    torchrun --nproc_per_node=4 --master-addr 127.0.0.1 examples/models/marianmt/run_marianmt.py \\
        --output_dir ./out --per_device_train_batch_size 4 --gradient_accumulation_steps 4 --max_steps 50
    PP=2 TP=2 ...   (degrees come from the environment; ``--tiny 1`` shrinks the model for a CPU run)
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import transformers as T  # noqa: E402
from _hf import run  # noqa: E402

if __name__ == "__main__":
    run(T.MarianConfig, T.MarianMTModel, mode="condition",
        tiny_overrides=dict(pad_token_id=0, decoder_start_token_id=0, eos_token_id=1))
