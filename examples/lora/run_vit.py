"""LoRA fine-tuning of a Hugging Face ViT classifier with accuracy on the evaluation split: adapters go
into the attention ``query`` / ``value`` projections, only they are trained and saved, and every
evaluation reports loss and accuracy from the last pipeline stage's logits (``--return_logits true`` +
``compute_metrics``).  The counterpart of the reference's examples/lora/run_vit.py:89-316, which does
this on CIFAR-10 with a trainer subclass; here the images are generated (pass your own ``Dataset`` of
``{"pixel_values", "labels"}`` dicts) and the trainer's own evaluation calls the metric function.

    torchrun --nproc-per-node=4 --master-addr 127.0.0.1 examples/lora/run_vit.py \\
        --per_device_train_batch_size 128 --gradient_accumulation_steps 4 --output_dir ./output \\
        --num_train_epochs 5 --learning_rate 5e-3 --do_eval true --return_logits true \\
        --lora_config examples/lora/vit_lora_config.json
    # base weights: --resume_from_checkpoint <Hugging Face directory or a framework checkpoint>
    # ``--tiny 1`` shrinks the model for a CPU run
"""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from _common import degrees, parse

import torch
import torch.nn.functional as F
import transformers as T

import merak_b200 as Merak
from merak_b200.utils.datasets import DynamicGenDataset


def compute_metrics(p):
    """Top-1 accuracy of an evaluation step (``p.predictions``: logits, ``p.label_ids``: classes)."""
    return {"accuracy": (p.predictions.argmax(dim=-1) == p.label_ids).float().mean().item()}


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    args, own = parse({"tiny": 0, "num_labels": 10, "dataset_size": 2048, "return_logits": True,
                       "lora_config": os.path.join(here, "vit_lora_config.json")})
    Merak.init(**degrees())
    shape = dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, intermediate_size=128, image_size=32,
                 patch_size=8, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0) if own.tiny else {}
    config = T.ViTConfig(num_labels=own.num_labels, **shape)
    model = T.ViTForImageClassification(config)
    train = DynamicGenDataset(config, mode="vision_only", dataset_size=own.dataset_size, image_size=config.image_size)
    evald = DynamicGenDataset(config, mode="vision_only", dataset_size=max(8, own.dataset_size // 8),
                              image_size=config.image_size, seed=1)
    args.input_names = ["pixel_values"]
    trainer = Merak.MerakTrainer(model, args, train_dataset=train, eval_dataset=evald, compute_metrics=compute_metrics,
                                 loss_fn=lambda out, labels: F.cross_entropy(out.float(), labels))
    trainer.train()
    trainer.evaluation()
    trainable = sum(p.numel() for p in trainer.engine.module.parameters() if p.requires_grad)
    total = sum(p.numel() for p in trainer.engine.module.parameters())
    if Merak.mpu.get_global_rank() == 0:
        print("trainable parameters on this stage: %d of %d; evaluation metrics: %s" % (trainable, total, trainer.eval_metrics))


if __name__ == "__main__":
    main()
