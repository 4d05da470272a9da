#!/usr/bin/env python
"""Merge a sharded training checkpoint (one file per tensor-parallel rank and pipeline stage) into
Hugging-Face-style safetensors.

    python tools/convert_safetensor.py --load_path out/2026-01-01_ckpt --save_path merged [--parallel_vocab]

Same contract as the reference tool (tools/convert_safetensor.py:30-320): tp/pp degrees are inferred
from the ``mp_rank_XX[_pp_rank_YYY]`` directory names; per pipeline stage the tensor-parallel shards
are concatenated (``*col_linear*`` on dim 0, ``*row_linear*`` weights on dim 1, vocabulary-sharded
embeddings on dim 0 with ``--parallel_vocab``); the leading shard index and the ``col_linear.`` /
``row_linear.`` components are stripped from the keys; output is ``model.safetensors`` (pp=1) or
``model-0000i-of-00000n.safetensors`` plus ``model.safetensors.index.json`` with
``metadata.total_size``, ``metadata.tp_meta_data`` and ``weight_map``.

Fused projections written by this framework carry their part sizes in the checkpoint's args-free
metadata (``fused_parts`` is recovered from the key: qkv / gate_up), so each part is re-assembled
separately before concatenation.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
from collections import OrderedDict

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

FUSED_PARTS = {"c_attn": 3, "qkv": 3, "gate_up_proj": 2}


def find_latest(load_path: str) -> str:
    tracker = os.path.join(load_path, "latest_checkpointed_iteration.txt")
    if os.path.isfile(tracker):
        it = open(tracker).read().strip()
        return os.path.join(load_path, "release" if it == "release" else "iter_{:07d}".format(int(it)))
    return load_path


def discover(iter_dir: str):
    """Returns (tp, pp, {(tp_rank, pp_rank): file})."""
    files = {}
    single = os.path.join(iter_dir, "model_optim.pt")
    if os.path.isfile(single):
        return 1, 1, {(0, 0): single}
    for d in sorted(os.listdir(iter_dir)):
        m = re.match(r"mp_rank_(\d+)(?:_pp_rank_(\d+))?$", d)
        if m:
            files[(int(m.group(1)), int(m.group(2) or 0))] = os.path.join(iter_dir, d, "partial_model_optim.pt")
    if not files:
        raise FileNotFoundError("no model shards under %s" % iter_dir)
    tp = max(k[0] for k in files) + 1
    pp = max(k[1] for k in files) + 1
    return tp, pp, files


def _fused_parts_of(key: str):
    for frag, n in FUSED_PARTS.items():
        if ("." + frag + ".") in ("." + key + "."):
            return n
    return None


def merge_tp(shards, parallel_vocab: bool):
    """shards: list over tp rank of state dicts of one pipeline stage."""
    out, meta = OrderedDict(), {}
    for key in shards[0]:
        tensors = [s[key] for s in shards]
        if len(tensors) == 1:
            out[key] = tensors[0]
            continue
        if "col_linear" in key:
            parts = _fused_parts_of(key)
            if parts:
                chunks = [t.chunk(parts, 0) for t in tensors]
                merged = torch.cat([torch.cat([c[p] for c in chunks], 0) for p in range(parts)], 0)
            else:
                merged = torch.cat(tensors, 0)
            meta[key] = {"dim": 0, "parts": parts or 1}
        elif "row_linear" in key and key.endswith("weight"):
            merged = torch.cat(tensors, 1)
            meta[key] = {"dim": 1, "parts": 1}
        elif parallel_vocab and ("wte" in key or "tied_modules" in key or "embed_tokens" in key
                                 or "word_embeddings" in key):
            merged = torch.cat(tensors, 0)
            meta[key] = {"dim": 0, "parts": 1}
        else:
            merged = tensors[0]
        out[key] = merged
    return out, meta


def clean_key(key: str) -> str:
    parts = key.split(".")
    if parts[0].isdigit():
        parts = parts[1:]
    return ".".join(p for p in parts if p not in ("col_linear", "row_linear"))


def convert(load_path: str, save_path: str, parallel_vocab: bool = False):
    from safetensors.torch import save_file
    iter_dir = find_latest(load_path)
    tp, pp, files = discover(iter_dir)
    os.makedirs(save_path, exist_ok=True)
    weight_map, tp_meta, total = OrderedDict(), {}, 0
    for stage in range(pp):
        shards = []
        for r in range(tp):
            sd = torch.load(files[(r, stage)], map_location="cpu", weights_only=False)["model"]
            shards.append(sd)
        merged, meta = merge_tp(shards, parallel_vocab)
        clean = OrderedDict()
        for k, v in merged.items():
            if k.startswith("tied_modules."):
                continue
            ck = clean_key(k)
            clean[ck] = v.contiguous().clone()
            if k in meta:
                tp_meta[ck] = meta[k]
        fname = "model.safetensors" if pp == 1 else "model-{:05d}-of-{:06d}.safetensors".format(stage + 1, pp)
        save_file(clean, os.path.join(save_path, fname), metadata={"format": "pt"})
        for k, v in clean.items():
            weight_map[k] = fname
            total += v.numel() * v.element_size()
    with open(os.path.join(save_path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total, "tp_meta_data": tp_meta, "tp": tp, "pp": pp},
                   "weight_map": weight_map}, f, indent=2)
    return tp, pp, list(weight_map)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--load_path", required=True)
    ap.add_argument("--save_path", required=True)
    ap.add_argument("--parallel_vocab", action="store_true")
    a = ap.parse_args()
    tp, pp, keys = convert(a.load_path, a.save_path, a.parallel_vocab)
    print("merged tp=%d pp=%d -> %d tensors in %s" % (tp, pp, len(keys), a.save_path))


if __name__ == "__main__":
    main()
