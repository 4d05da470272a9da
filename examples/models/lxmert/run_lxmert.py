"""LXMERT visual question answering (examples/models/lxmert): the Hugging Face ``LxmertForQuestionAnswering`` with random weights on generated data.

    torchrun --nproc_per_node=4 --master-addr 127.0.0.1 examples/models/lxmert/run_lxmert.py \\
        --output_dir ./out --per_device_train_batch_size 4 --gradient_accumulation_steps 4 --max_steps 50
    PP=2 TP=2 ...   (degrees come from the environment; ``--tiny 1`` shrinks the model for a CPU run)
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import torch  # noqa: E402
import transformers as T  # noqa: E402
from _hf import run  # noqa: E402

TINY_LXMERT = dict(l_layers=1, x_layers=1, r_layers=1, visual_feat_dim=32, visual_pos_dim=4, num_qa_labels=10,
                   vocab_size=1024, num_hidden_layers=None)


def with_regions(feat_dim, answers):
    """Adds what the vision stream reads: region features ``[boxes, feat_dim]`` and normalised boxes
    ``[boxes, 4]``, and an answer class as the label (all generated, seeded by the sample's first token)."""
    def fn(sample):
        g = torch.Generator().manual_seed(int(sample["input_ids"][0]))
        return {"input_ids": sample["input_ids"], "visual_feats": torch.randn(8, feat_dim, generator=g),
                "visual_pos": torch.rand(8, 4, generator=g), "labels": sample["input_ids"][0] % answers}
    return fn


if __name__ == "__main__":
    tiny = "--tiny" in sys.argv and sys.argv[sys.argv.index("--tiny") + 1] not in ("0", "false")
    cfg = T.LxmertConfig()
    run(T.LxmertConfig, T.LxmertForQuestionAnswering, mode="text_only", tiny_overrides=TINY_LXMERT,
        sample_fn=with_regions(32 if tiny else cfg.visual_feat_dim, 10 if tiny else cfg.num_qa_labels),
        num_layers=3 if tiny else cfg.l_layers + cfg.x_layers + cfg.r_layers)
