"""AltCLIP contrastive image-text pre-training (examples/models/altclip): the Hugging Face ``AltCLIPModel`` with random weights on generated data.

    torchrun --nproc_per_node=4 --master-addr 127.0.0.1 examples/models/altclip/run_altclip.py \\
        --output_dir ./out --per_device_train_batch_size 4 --gradient_accumulation_steps 4 --max_steps 50
    PP=2 TP=2 ...   (degrees come from the environment; ``--tiny 1`` shrinks the model for a CPU run)
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import transformers as T  # noqa: E402
from _hf import run  # noqa: E402

TINY_TEXT = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, vocab_size=1024,
                 max_position_embeddings=80, project_dim=32, pad_token_id=1)
TINY_VISION = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=32,
                   patch_size=8, projection_dim=32)


def contrastive_loss(model):
    """The model returns the image-text similarity matrix ``logits_per_image [B, B]`` first; matching pairs sit
    on the diagonal: symmetric cross entropy over rows and columns (what ``return_loss=True`` computes inside
    the Hugging Face model)."""
    import torch
    import torch.nn.functional as F

    def loss(outputs, labels):
        sim = outputs[0] if isinstance(outputs, (tuple, list)) else outputs
        if isinstance(sim, dict):
            sim = sim["logits_per_image"]
        target = torch.arange(sim.shape[0], device=sim.device)
        return 0.5 * (F.cross_entropy(sim.float(), target) + F.cross_entropy(sim.float().t(), target))
    return loss


def tiny_images(sample):
    """The generated images follow the top-level configuration (224 x 224); the tiny towers take 32 x 32."""
    out = dict(sample)
    out["pixel_values"] = sample["pixel_values"][:, :32, :32].contiguous()
    return out


if __name__ == "__main__":
    tiny = "--tiny" in sys.argv and sys.argv[sys.argv.index("--tiny") + 1] not in ("0", "false")
    run(T.AltCLIPConfig, T.AltCLIPModel, mode="multimodal", loss_fn=contrastive_loss,
        tiny_overrides=dict(text_config=TINY_TEXT, vision_config=TINY_VISION, projection_dim=32),
        sample_fn=tiny_images if tiny else None)
