"""LoRA supervised fine-tuning of a Llama / Qwen2 checkpoint stored in Hugging Face format
(``config.json`` + ``model.safetensors`` or sharded ``model-0000x-of-0000y.safetensors``), the
counterpart of the reference's examples/deepseek-r1/finetune.py:125-227 (DeepSeek-R1-Distill-Llama-8B
/ Qwen-7B/14B/32B):

* the model is built from ``config.json`` with ``transformers`` under ``init_empty_weights`` (no memory for
  the full model on any rank), traced, sharded over ``PP`` stages and ``TP`` ranks;
* the base weights come from the safetensors files (``resume_from_checkpoint`` = the directory; every
  rank reads only its own stage's tensors and takes its tensor-parallel slice);
* LoRA adapters from ``--lora_config`` are injected after the engine is built, only they train, and the
  checkpoints hold only them (``lora_model_optim.pt`` per stage + ``lora_config.json``);
* samples are (prompt, answer) token sequences of different lengths; the collator pads them to the longest
  of the batch (to a multiple of 8) and masks prompt and padding positions out of the loss with -100, like
  ``DataCollatorForSeq2Seq(padding=True, label_pad_token_id=-100)`` in the reference script.

    PP=2 TP=2 torchrun --nproc_per_node=4 --master-addr 127.0.0.1 examples/deepseek-r1/finetune.py \\
        --model_path /models/DeepSeek-R1-Distill-Llama-8B --data_path sft.jsonl \\
        --lora_config examples/deepseek-r1/lora_config.json --output_dir ./out --bf16 true \\
        --per_device_train_batch_size 1 --gradient_accumulation_steps 16 --max_steps 1000

``--data_path`` is a JSON-lines file of ``{"input_ids": [...], "labels": [...]}`` records (already
tokenised; no tokenizer download is needed at run time); without it, random prompt / answer pairs are
generated so the script can be tried anywhere.
"""
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from _common import degrees, parse  # noqa: E402

import torch  # noqa: E402

import merak_b200 as Merak  # noqa: E402


class SFTDataset(torch.utils.data.Dataset):
    """Tokenised (prompt, answer) pairs; the loss covers the answer tokens only."""

    def __init__(self, path, vocab_size, size, max_len, seed=0):
        self.records = None
        if path:
            with open(path) as f:
                self.records = [json.loads(line) for line in f if line.strip()]
        self.vocab, self.size, self.max_len, self.seed = vocab_size, size, max_len, seed

    def __len__(self):
        return len(self.records) if self.records is not None else self.size

    def __getitem__(self, i):
        if self.records is not None:
            r = self.records[i]
            return {"input_ids": torch.tensor(r["input_ids"][:self.max_len]),
                    "labels": torch.tensor(r["labels"][:self.max_len])}
        g = torch.Generator().manual_seed(self.seed * 7919 + i)
        n_prompt = int(torch.randint(4, self.max_len // 2, (), generator=g))
        n_answer = int(torch.randint(4, self.max_len - n_prompt, (), generator=g))
        ids = torch.randint(3, self.vocab, (n_prompt + n_answer,), generator=g)
        labels = ids.clone()
        labels[:n_prompt] = -100
        return {"input_ids": ids, "labels": labels}


class PadToLongest:
    """Pads ``input_ids`` (pad id) and ``labels`` (-100) to the longest sample of the batch, rounded up
    to ``multiple``; also returns the attention mask."""

    def __init__(self, pad_token_id=0, multiple=8, fixed_length=None):
        self.pad, self.multiple, self.fixed = pad_token_id, multiple, fixed_length

    def __call__(self, samples):
        longest = max(len(s["input_ids"]) for s in samples)
        n = self.fixed or (longest + self.multiple - 1) // self.multiple * self.multiple
        ids = torch.full((len(samples), n), self.pad, dtype=torch.long)
        labels = torch.full((len(samples), n), -100, dtype=torch.long)
        mask = torch.zeros(len(samples), n, dtype=torch.long)
        for r, s in enumerate(samples):
            k = min(len(s["input_ids"]), n)
            ids[r, :k], labels[r, :k], mask[r, :k] = s["input_ids"][:k], s["labels"][:k], 1
        return {"input_ids": ids, "attention_mask": mask, "labels": labels}


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    args, own = parse({"model_path": "", "data_path": "", "max_length": 1024, "dataset_size": 2048,
                       "lora_config": os.path.join(here, "lora_config.json")})
    if not own.model_path:
        raise SystemExit("--model_path: a directory with config.json and safetensors weights")
    Merak.init(**degrees())
    import transformers as T
    config = T.AutoConfig.from_pretrained(own.model_path)
    config.use_cache = False
    with Merak.init_empty_weights():
        model = T.AutoModelForCausalLM.from_config(config)
    args.resume_from_checkpoint = own.model_path          # base weights: the Hugging Face directory
    args.input_names = ["input_ids", "attention_mask"]
    pad_id = config.pad_token_id if config.pad_token_id is not None else 0
    # pipeline stages exchange fixed-shape activations: every batch is padded to max_length
    collate = PadToLongest(pad_id, fixed_length=own.max_length)
    train = SFTDataset(own.data_path or None, config.vocab_size, own.dataset_size, own.max_length, seed=args.seed)
    trainer = Merak.MerakTrainer(model, args, train_dataset=train, data_collator=collate)
    trainer.train()
    if Merak.mpu.get_global_rank() == 0:
        mod = trainer.engine.module
        trainable = sum(p.numel() for p in mod.parameters() if p.requires_grad)
        print("trainable (LoRA) parameters on stage 0: %d of %d" % (trainable, sum(p.numel() for p in mod.parameters())))


if __name__ == "__main__":
    main()
