"""Greedy / sampled generation with the text-generation pipeline under a parallel layout; rank 0
writes the generated token ids.  Launched through torch.distributed.run on CPU/gloo."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ.setdefault("MERAK_QUIET", "1")

import torch
import faulthandler
if os.environ.get("DUMP_AFTER"):
    faulthandler.dump_traceback_later(int(os.environ["DUMP_AFTER"]), exit=True)

import merak_b200 as Merak
from merak_b200.inference import text_generation_pipeline
from merak_b200.models.gpt2 import GPT2LMHeadModel, gpt2_config
from merak_b200.utils.datasets import SyntheticTokenDataset


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--new_tokens", type=int, default=6)
    ap.add_argument("--out", required=True)
    o = ap.parse_args()
    Merak.init(o.pp, o.tp, 1, backend="gloo")
    torch.manual_seed(1234)
    V = 512
    model = GPT2LMHeadModel(gpt2_config("gpt2-tiny", vocab_size=V, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0))
    args = Merak.MerakArguments(output_dir="/tmp/merak_b200_gen", per_device_train_batch_size=2, max_steps=1,
                                logging_steps=0, wall_clock_breakdown=False, report_to="none", no_cuda=True,
                                activation_checkpointing=False, seed=1234, comm_mode="nccl", out_seq_length=64,
                                temperature=0.8, top_k=20, top_p=0.9, parallel_vocab=o.tp > 1)
    trainer = Merak.MerakTrainer(model, args, train_dataset=SyntheticTokenDataset(V, 16, 8, seed=3))
    pipe = text_generation_pipeline(trainer, args, eos_token_id=None)
    prompts = [[5, 17, 99, 256, 3, 44, 7, 120], [400, 2, 2, 81, 310, 9, 64, 1]]
    greedy = pipe.generate(prompts, max_new_tokens=o.new_tokens, greedy=True)
    sampled = pipe.generate(prompts, max_new_tokens=o.new_tokens, greedy=False, seed=11)
    if torch.distributed.get_rank() == 0:
        with open(o.out, "w") as f:
            json.dump({"greedy": greedy, "sampled": sampled}, f)
    torch.distributed.barrier()
    Merak.initialize.destroy()


if __name__ == "__main__":
    main()
