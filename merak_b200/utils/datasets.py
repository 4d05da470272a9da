"""Synthetic datasets for examples, tests and benchmarks: ``DynamicGenDataset`` produces random
samples of the shapes a model config implies, in the seven modes of the reference
(Merak/utils/datasets.py:39-216)."""
from __future__ import annotations

from typing import Optional

import torch
from torch.utils.data import Dataset

MODES = ("text_only", "multimodal", "vision_only", "condition", "speech", "speech2text", "for_qa")
SEQ_LENGTH_KEYS = ("seq_length", "max_position_embeddings", "n_positions", "embed_dim", "max_target_positions")


class DynamicGenDataset(Dataset):

    def __init__(self, model_config, mode: str = "text_only", dataset_size: int = 10000, image_size: Optional[int] = None,
                 seq_length: Optional[int] = None, seed: int = 0, vocab_limit: Optional[int] = 1000):
        # positional order as in the reference (Merak/utils/datasets.py:62-69)
        if mode not in MODES:
            raise ValueError("mode must be one of %s" % (MODES,))
        self.cfg, self.mode, self.size = model_config, mode, int(dataset_size)      # the reference scripts pass 1e6
        # two-tower configurations (CLIP, AltCLIP) keep the text sizes in ``text_config`` and the image sizes in
        # ``vision_config``; the sequence length is the first of the reference's keys the configuration has
        # (Merak/utils/datasets.py:31-37,88-99)
        text = getattr(model_config, "text_config", None) or model_config
        vision = getattr(model_config, "vision_config", None) or model_config
        inferred = next((getattr(text, k) for k in SEQ_LENGTH_KEYS if isinstance(getattr(text, k, None), int)), None)
        self.seq = int(seq_length or inferred or 128)
        img = image_size or getattr(vision, "image_size", None) or getattr(model_config, "image_size", 224)
        self.image_size = img if isinstance(img, int) else img[0]
        self.channels = int(getattr(vision, "num_channels", 3))
        vocab = int(getattr(text, "vocab_size", 1000) or 1000)
        self.vocab = min(vocab, vocab_limit) if vocab_limit else vocab
        self.seed = seed

    def __len__(self):
        return self.size

    def _gen(self, idx):
        g = torch.Generator()
        g.manual_seed(self.seed * 1000003 + idx)
        return g

    def __getitem__(self, idx):
        g = self._gen(idx)
        ids = torch.randint(1, self.vocab, (self.seq,), generator=g)
        if self.mode == "text_only":
            return {"input_ids": ids, "labels": ids.clone()}
        if self.mode == "for_qa":
            if hasattr(self.cfg, "visual_feat_dim"):          # LXMERT: region features and boxes beside the question
                return {"input_ids": ids,
                        "visual_feats": torch.randn(self.seq, int(self.cfg.visual_feat_dim), generator=g),
                        "visual_pos": torch.randn(self.seq, int(self.cfg.visual_pos_dim), generator=g),
                        "labels": torch.zeros(1, dtype=torch.long)}
            return {"input_ids": ids, "start_positions": torch.randint(0, self.seq, (), generator=g),
                    "end_positions": torch.randint(0, self.seq, (), generator=g)}
        if self.mode == "condition":
            return {"input_ids": ids, "decoder_input_ids": ids.clone(), "labels": ids.clone()}
        pixels = torch.randn(self.channels, self.image_size, self.image_size, generator=g)
        if self.mode == "vision_only":
            n_labels = int(getattr(self.cfg, "num_labels", 1000) or 1000)
            return {"pixel_values": pixels, "labels": torch.randint(0, n_labels, (), generator=g)}
        if self.mode == "multimodal":
            return {"input_ids": ids, "pixel_values": pixels, "labels": ids.clone()}
        feats = torch.randn(16000, generator=g)
        if self.mode == "speech":
            return {"input_values": feats, "labels": torch.randint(1, self.vocab, (32,), generator=g)}
        if hasattr(self.cfg, "input_feat_per_channel"):    # Speech2Text: [frames, features] filter banks
            feats = torch.randn(self.seq, int(self.cfg.input_feat_per_channel), generator=g)
            return {"input_features": feats, "decoder_input_ids": ids.clone(), "labels": ids.clone()}
        mel = torch.randn(int(getattr(self.cfg, "num_mel_bins", 80)), 3000, generator=g)
        return {"input_features": mel, "decoder_input_ids": ids.clone(), "labels": ids.clone()}


class SyntheticTokenDataset(Dataset):
    """Uniform random token ids with next-token (``causal``) or masked-LM (``mlm``) labels; the
    workloads the benchmark configurations name."""

    def __init__(self, vocab_size: int, seq_length: int, size: int, task: str = "causal", seed: int = 0,
                 mask_token_id: int = 103, mlm_probability: float = 0.15):
        self.vocab, self.seq, self.size, self.task, self.seed = vocab_size, seq_length, size, task, seed
        self.mask_id, self.p = mask_token_id, mlm_probability

    def __len__(self):
        return self.size

    def __getitem__(self, idx):
        g = torch.Generator()
        g.manual_seed(self.seed * 1000003 + idx)
        ids = torch.randint(0, self.vocab, (self.seq,), generator=g)
        if self.task == "causal":
            return {"input_ids": ids, "labels": ids.clone()}
        labels = ids.clone()
        masked = torch.rand(self.seq, generator=g) < self.p
        labels[~masked] = -100
        roll = torch.rand(self.seq, generator=g)
        inp = ids.clone()
        inp[masked & (roll < 0.8)] = self.mask_id                           # 80%: [MASK]
        rnd = masked & (roll >= 0.8) & (roll < 0.9)                          # 10%: random token
        inp[rnd] = torch.randint(0, self.vocab, (int(rnd.sum()),), generator=g)
        return {"input_ids": inp, "attention_mask": torch.ones(self.seq, dtype=torch.long), "labels": labels}
