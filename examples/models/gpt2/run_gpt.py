"""GPT-2 language modelling on generated token data (the reference's examples/models/gpt2/run_gpt.py:
meta-style construction, default tracing and splitting).

    torchrun --nproc_per_node=4 --master-addr 127.0.0.1 examples/models/gpt2/run_gpt.py \
        --output_dir ./out --per_device_train_batch_size 4 --gradient_accumulation_steps 4 --max_steps 50
    PP=4 TP=1 DP=1 ... (degrees come from the environment; default is data parallel over all ranks)
"""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from _common import degrees, parse

import merak_b200 as Merak
from merak_b200.models.gpt2 import GPT2LMHeadModel, gpt2_config
from merak_b200.utils.datasets import DynamicGenDataset


def main():
    args, own = parse({"model_size": "gpt2", "seq_length": 1024, "dataset_size": 4096})
    Merak.init(**degrees())
    config = gpt2_config(own.model_size)
    model = GPT2LMHeadModel(config)
    seq = min(own.seq_length, config.n_positions)
    train = DynamicGenDataset(config, mode="text_only", dataset_size=own.dataset_size, seq_length=seq)
    trainer = Merak.MerakTrainer(model, args, train_dataset=train)
    trainer.train()


if __name__ == "__main__":
    main()
