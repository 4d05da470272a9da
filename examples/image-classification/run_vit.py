"""Vision-transformer image classification with a custom collate function and an accuracy metric
on the evaluation split (the reference's examples/image-classification/run_vit.py:40-86 on ImageNet;
here the images are generated, pass your own ``Dataset`` of ``{"pixel_values", "labels"}`` dicts).
The encoder uses the framework's linear / norm / attention ops, so on a GPU it runs on the sm_100a
kernels."""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from _common import degrees, parse

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

import merak_b200 as Merak
from merak_b200.ops.attention import flash_attention_packed
from merak_b200.ops.modules import LayerNorm, Linear
from merak_b200.utils.datasets import DynamicGenDataset


@dataclass
class ViTConfig:
    image_size: int = 224
    patch_size: int = 16
    num_channels: int = 3
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    num_labels: int = 1000
    model_type: str = "vit"


class ViTLayer(nn.Module):
    def __init__(self, c: ViTConfig):
        super().__init__()
        self.heads, self.dim = c.num_attention_heads, c.hidden_size // c.num_attention_heads
        self.layernorm_before = LayerNorm(c.hidden_size)
        self.qkv = Linear(c.hidden_size, 3 * c.hidden_size)
        self.out = Linear(c.hidden_size, c.hidden_size)
        self.layernorm_after = LayerNorm(c.hidden_size)
        self.fc1 = Linear(c.hidden_size, c.intermediate_size)
        self.fc2 = Linear(c.intermediate_size, c.hidden_size)

    def forward(self, x):
        B, L, H = x.shape
        qkv = self.qkv(self.layernorm_before(x)).view(B, L, 3 * self.heads, self.dim)
        x = x + self.out(flash_attention_packed(qkv, self.heads, self.heads).reshape(B, L, H))
        return x + self.fc2(F.gelu(self.fc1(self.layernorm_after(x))))


class ViTForImageClassification(nn.Module):
    def __init__(self, c: ViTConfig):
        super().__init__()
        self.config = c
        n = (c.image_size // c.patch_size) ** 2
        self.patch = nn.Conv2d(c.num_channels, c.hidden_size, c.patch_size, c.patch_size)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, c.hidden_size))
        self.position = nn.Parameter(torch.zeros(1, n + 1, c.hidden_size))
        self.layers = nn.ModuleList([ViTLayer(c) for _ in range(c.num_hidden_layers)])
        self.norm = LayerNorm(c.hidden_size)
        self.classifier = Linear(c.hidden_size, c.num_labels)

    def forward(self, pixel_values):
        x = self.patch(pixel_values).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1) + self.position.to(x.dtype)
        for l in self.layers:
            x = l(x)
        return self.classifier(self.norm(x)[:, 0])


def collate(features):
    return {"pixel_values": torch.stack([f["pixel_values"] for f in features]),
            "labels": torch.stack([torch.as_tensor(f["labels"]) for f in features])}


def accuracy(p):
    """Top-1 accuracy of one evaluation step (``p.predictions``: logits, ``p.label_ids``: classes)."""
    return {"accuracy": (p.predictions.argmax(dim=-1) == p.label_ids).float().mean().item()}


def main():
    args, own = parse({"image_size": 224, "hidden_size": 768, "layers": 12, "heads": 12, "num_labels": 1000,
                       "dataset_size": 2048})
    Merak.init(**degrees())
    cfg = ViTConfig(image_size=own.image_size, hidden_size=own.hidden_size, num_hidden_layers=own.layers,
                    num_attention_heads=own.heads, intermediate_size=4 * own.hidden_size, num_labels=own.num_labels)
    model = ViTForImageClassification(cfg)
    train = DynamicGenDataset(cfg, mode="vision_only", dataset_size=own.dataset_size, image_size=own.image_size)
    evald = DynamicGenDataset(cfg, mode="vision_only", dataset_size=max(8, own.dataset_size // 8),
                              image_size=own.image_size, seed=1)
    args.input_names = ["pixel_values"]
    args.return_logits = True
    trainer = Merak.MerakTrainer(model, args, train_dataset=train, eval_dataset=evald, data_collator=collate,
                                 leaf_modules=(ViTLayer,), compute_metrics=accuracy,
                                 loss_fn=lambda out, labels: F.cross_entropy(out.float(), labels))
    trainer.train()
    trainer.evaluation()          # logs "eval loss: ..., accuracy: ..." (also after every epoch with --do_eval true)


if __name__ == "__main__":
    main()
