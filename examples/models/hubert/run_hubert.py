"""HuBERT speech recognition (CTC) (examples/models/hubert): the Hugging Face ``HubertForCTC`` with random weights on generated data.

    torchrun --nproc_per_node=4 --master-addr 127.0.0.1 examples/models/hubert/run_hubert.py \\
        --output_dir ./out --per_device_train_batch_size 4 --gradient_accumulation_steps 4 --max_steps 50
    PP=2 TP=2 ...   (degrees come from the environment; ``--tiny 1`` shrinks the model for a CPU run)
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import transformers as T  # noqa: E402
from _hf import run  # noqa: E402


def ctc_loss(model):
    """The model returns frame logits ``[B, T, V]``; the labels are token sequences: connectionist temporal
    classification over all frames (the reference's script builds the same loss in its ``get_loss_fn``
    override, examples/models/wav2vec2/run_wav2vec2.py:72-119)."""
    import torch
    import torch.nn.functional as F

    def loss(outputs, labels):
        logits = outputs[0] if isinstance(outputs, (tuple, list)) else outputs
        if isinstance(labels, dict):
            labels = labels["labels"]
        logp = F.log_softmax(logits.float(), dim=-1).transpose(0, 1)              # [T, B, V]
        frames, batch = logp.shape[0], logp.shape[1]
        in_len = torch.full((batch,), frames, dtype=torch.long)
        tgt_len = torch.full((batch,), labels.shape[1], dtype=torch.long)
        return F.ctc_loss(logp, labels, in_len, tgt_len, blank=model.config.pad_token_id or 0, reduction="mean",
                          zero_infinity=True)
    return loss


TINY_SPEECH = dict(conv_dim=(32, 32), conv_stride=(5, 4), conv_kernel=(10, 8), num_conv_pos_embeddings=16,
                   num_conv_pos_embedding_groups=2, mask_time_prob=0.0, vocab_size=64)

if __name__ == "__main__":
    run(T.HubertConfig, T.HubertForCTC, mode="speech", tiny_overrides=TINY_SPEECH, config_overrides=dict(mask_time_prob=0.0),
        loss_fn=ctc_loss)
