"""Text generation through the pipeline engine: the prompt runs through all stages for every new
token, the last stage samples (temperature / top-k / top-p) and broadcasts the token (the
reference's examples/text_generation/run_gpt_text_generation.py:50-96).  Without a tokenizer the
script works on token ids; pass ``--tokenizer_dir`` (a local Hugging Face tokenizer) for text and
``--interactive true`` for the prompt loop."""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from _common import degrees, parse

import torch

import merak_b200 as Merak
from merak_b200.inference.text_generation import text_generation_pipeline
from merak_b200.models.gpt2 import GPT2LMHeadModel, gpt2_config
from merak_b200.utils.datasets import DynamicGenDataset


def main():
    args, own = parse({"model_size": "gpt2", "tokenizer_dir": None, "interactive": "false", "prompt_length": 8,
                       "new_tokens": 16})
    Merak.init(**degrees())
    config = gpt2_config(own.model_size)
    model = GPT2LMHeadModel(config)
    tokenizer = None
    if own.tokenizer_dir:
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(own.tokenizer_dir, local_files_only=True)
    args.text_generation = True
    # the dataset only tells the tracer what an input looks like
    shape_data = DynamicGenDataset(config, mode="text_only", dataset_size=4, seq_length=own.prompt_length)
    trainer = Merak.MerakTrainer(model, args, train_dataset=shape_data, tokenizer=tokenizer)
    pipe = text_generation_pipeline(trainer, args, tokenizer)
    if own.interactive.lower() == "true" and tokenizer is not None:
        pipe.generate_samples_interactive()
        return
    g = torch.Generator().manual_seed(args.seed)
    prompts = torch.randint(0, min(config.vocab_size, 1000), (2, own.prompt_length), generator=g).tolist()
    out = pipe.generate(prompts, max_new_tokens=own.new_tokens, seed=args.seed)
    if Merak.mpu.get_global_rank() == 0:
        ids = out[0] if tokenizer is not None else out
        for row in ids:
            print("generated ids:", row)


if __name__ == "__main__":
    main()
