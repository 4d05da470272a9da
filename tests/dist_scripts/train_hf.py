"""Trains a tiny Hugging Face model (``transformers`` classes, random weights) under a parallel
layout through the trainer and writes the loss curve.  Launched by the tests through
torch.distributed.run on CPU/gloo."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
os.environ.setdefault("MERAK_QUIET", "1")

import torch

import merak_b200 as Merak
from train_small import FixedOrderTrainer


class TinyData(torch.utils.data.Dataset):
    def __init__(self, kind, n=16, seq=16, vocab=256):
        g = torch.Generator().manual_seed(7)
        self.kind = kind
        self.ids = torch.randint(0, vocab, (n, seq), generator=g)
        self.dec = torch.randint(0, vocab, (n, 8), generator=g)
        self.pix = torch.randn(n, 3, 32, 32, generator=g)
        self.cls = torch.randint(0, 10, (n,), generator=g)

    def __len__(self):
        return self.ids.shape[0]

    def __getitem__(self, i):
        if self.kind == "vit":
            return {"pixel_values": self.pix[i], "labels": self.cls[i]}
        if self.kind == "t5":
            return {"input_ids": self.ids[i], "decoder_input_ids": self.dec[i], "labels": self.dec[i].clone()}
        if self.kind == "bert":
            lab = self.ids[i].clone()
            lab[::2] = -100
            return {"input_ids": self.ids[i], "attention_mask": torch.ones_like(self.ids[i]), "labels": lab}
        return {"input_ids": self.ids[i], "labels": self.ids[i].clone()}


def build(kind):
    import transformers as T
    common = dict(vocab_size=256)
    if kind == "gpt2":
        return T.GPT2LMHeadModel(T.GPT2Config(n_layer=2, n_embd=64, n_head=4, n_positions=32, resid_pdrop=0.0,
                                              embd_pdrop=0.0, attn_pdrop=0.0, **common))
    if kind == "bert":
        return T.BertForMaskedLM(T.BertConfig(num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                                              intermediate_size=128, max_position_embeddings=32,
                                              hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, **common))
    if kind == "llama":
        return T.LlamaForCausalLM(T.LlamaConfig(num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                                                num_key_value_heads=2, intermediate_size=128,
                                                max_position_embeddings=32, **common))
    if kind == "vit":
        return T.ViTForImageClassification(T.ViTConfig(num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                                                       intermediate_size=128, image_size=32, patch_size=8,
                                                       num_labels=10, hidden_dropout_prob=0.0,
                                                       attention_probs_dropout_prob=0.0))
    if kind == "t5":
        return T.T5ForConditionalGeneration(T.T5Config(num_layers=2, num_decoder_layers=2, d_model=64, num_heads=4,
                                                       d_kv=16, d_ff=128, dropout_rate=0.0, **common))
    raise ValueError(kind)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2")
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--gas", type=int, default=4)
    ap.add_argument("--split", default="nearest_min_deps")
    ap.add_argument("--out", required=True)
    o = ap.parse_args()
    Merak.init(o.pp, o.tp, o.dp, backend="gloo")
    torch.manual_seed(1234)
    model = build(o.model)
    args = Merak.MerakArguments(
        output_dir="/tmp/merak_b200_test_hf", per_device_train_batch_size=2, gradient_accumulation_steps=o.gas,
        max_steps=o.steps, logging_steps=0, learning_rate=3e-3, lr_scheduler_type="constant", weight_decay=0.0,
        wall_clock_breakdown=False, report_to="none", no_cuda=True, activation_checkpointing=False,
        split_method=o.split, seed=1234, comm_mode="nccl", max_grad_norm=1.0)
    FixedOrderTrainer.user_opt = ""
    trainer = FixedOrderTrainer(model, args, train_dataset=TinyData(o.model))
    engine = trainer.init_engine()
    data_iter = trainer._batch_iter(trainer.train_dataloader)
    losses = [float(engine.train_batch(data_iter)) for _ in range(o.steps)]
    if torch.distributed.get_rank() == 0:
        with open(o.out, "w") as f:
            json.dump({"losses": losses, "shards": engine.module.num_layers_total}, f)
    torch.distributed.barrier()
    Merak.initialize.destroy()


if __name__ == "__main__":
    main()
