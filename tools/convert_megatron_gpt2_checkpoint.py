#!/usr/bin/env python
"""Convert a Megatron-LM GPT-2 checkpoint (any tensor-/pipeline-parallel layout) into a Hugging Face
GPT-2 directory (``model.safetensors`` + ``config.json``) that ``resume_from_checkpoint`` loads under
any ``Merak.init(pp, tp, dp)`` layout.

    python tools/convert_megatron_gpt2_checkpoint.py --path_to_checkpoint ckpt/iter_0005000 \
        --path_to_output_checkpoint gpt2_hf [--config_file config.json] [--print-checkpoint-structure]

Role of the reference's tools/convert_megatron_gpt2_checkpoint.py:198-640, which re-shards a Megatron
checkpoint into the framework's per-rank files inside a distributed job (``--dp/--tp/--pp`` are
accepted here for command-line compatibility; re-sharding happens when the result is loaded, so this
tool runs in one process without GPUs).

Layout handled: ``mp_rank_{tp:02d}/model_optim_rng.pt`` (pp = 1) or
``mp_rank_{tp:02d}_{pp:03d}/model_optim_rng.pt``; ``model.language_model.embedding`` and
``.encoder`` (older: ``.transformer``); ``self_attention`` or ``attention`` blocks.  Column-parallel
tensors (word embeddings, ``query_key_value``, ``dense_h_to_4h``) are concatenated on dim 0,
row-parallel weights (``dense``, ``dense_4h_to_h``) on dim 1; the fused QKV rows are re-ordered from
Megatron's per-head interleaving (by ``checkpoint_version``) to ``[q; k; v]``; projection weights are
written transposed because Hugging Face GPT-2 stores them as ``Conv1D``.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
from collections import OrderedDict

import torch

LAYER_RE = re.compile(r"layers\.(\d+)\.([a-z0-9_.]+)\.(weight|bias)$")


def find_shards(path: str):
    """{(tp_rank, pp_rank): file}; a single file counts as tp = pp = 1."""
    if os.path.isfile(path):
        return {(0, 0): path}
    out = {}
    for d in sorted(os.listdir(path)):
        m = re.match(r"mp_rank_(\d+)(?:_(\d+))?$", d)
        f = os.path.join(path, d, "model_optim_rng.pt")
        if m and os.path.isfile(f):
            out[(int(m.group(1)), int(m.group(2) or 0))] = f
    if not out:
        raise FileNotFoundError("no mp_rank_*/model_optim_rng.pt under %r" % path)
    return out


def fix_query_key_value_ordering(param: torch.Tensor, version: float, num_splits: int, heads: int, head_dim: int):
    """Rows of a fused QKV tensor to ``[splits, heads, head_dim]`` order."""
    rest = param.shape[1:]
    if version >= 2.0:            # stored [heads, splits, head_dim]
        param = param.view(heads, num_splits, head_dim, *rest).transpose(0, 1).contiguous()
    elif version >= 1.0:          # stored [heads, head_dim, splits]
        param = param.view(heads, head_dim, num_splits, *rest).transpose(1, 2).transpose(0, 1).contiguous()
    return param.view(num_splits * heads * head_dim, *rest)


def recursive_print(name, val, spaces=0):
    pad = " " * spaces
    if isinstance(val, dict):
        if name is not None:
            print(pad + str(name))
        for k, v in val.items():
            recursive_print(k, v, spaces + 2)
    elif isinstance(val, torch.Tensor):
        print("%s%s : %s" % (pad, name, tuple(val.shape)))
    else:
        print("%s%s : %s" % (pad, name, val))


def _lm(sd):
    model = sd["model"]
    return model["language_model"] if "language_model" in model else model


def convert(shards: dict, config: dict):
    tp = 1 + max(t for t, _ in shards)
    pp = 1 + max(p for _, p in shards)
    loaded = {k: torch.load(f, map_location="cpu", weights_only=False) for k, f in shards.items()}
    first = loaded[(0, 0)]
    version = float(first.get("checkpoint_version", 0.0))
    margs = first.get("args", None)
    if margs is not None:
        g = (lambda n, d=None: getattr(margs, n, d)) if not isinstance(margs, dict) else (lambda n, d=None: margs.get(n, d))
        config.setdefault("vocab_size", g("padded_vocab_size"))
        config.setdefault("n_positions", g("max_position_embeddings"))
        config.setdefault("n_embd", g("hidden_size"))
        config.setdefault("n_layer", g("num_layers"))
        config.setdefault("n_head", g("num_attention_heads"))
        config.setdefault("n_inner", g("ffn_hidden_size"))
    out = OrderedDict()

    def cat(key_fn, dim):
        ts = [key_fn(r) for r in range(tp)]
        return ts[0] if dim is None or tp == 1 else torch.cat(ts, dim=dim)

    # embeddings live on the first pipeline stage
    emb = lambda r: _lm(loaded[(r, 0)])["embedding"]
    wte = cat(lambda r: emb(r)["word_embeddings"]["weight"], 0)
    config.setdefault("vocab_size", wte.shape[0])
    out["transformer.wte.weight"] = wte[:config["vocab_size"]].clone()
    out["transformer.wpe.weight"] = emb(0)["position_embeddings"]["weight"].clone()
    config.setdefault("n_positions", out["transformer.wpe.weight"].shape[0])
    config.setdefault("n_embd", wte.shape[1])
    hidden = config["n_embd"]

    layer_offset = 0
    final_ln = {}
    for stage in range(pp):
        enc = lambda r: (_lm(loaded[(r, stage)]).get("encoder") or _lm(loaded[(r, stage)]).get("transformer"))
        keys = list(enc(0).keys())
        local_layers = 0
        for key in keys:
            m = LAYER_RE.match(key)
            if m is None:
                if key.startswith("final_layernorm."):
                    final_ln[key.split(".")[-1]] = enc(0)[key]
                continue
            idx, op, kind = int(m.group(1)), m.group(2), m.group(3)
            local_layers = max(local_layers, idx + 1)
            name = "transformer.h.%d" % (layer_offset + idx)
            if op.endswith("layernorm"):
                ln = "ln_1" if op.startswith("input") else "ln_2"
                out["%s.%s.%s" % (name, ln, kind)] = enc(0)[key].clone()
            elif op in ("self_attention.query_key_value", "attention.query_key_value"):
                heads = config["n_head"]
                hd = hidden // heads
                per_rank = [fix_query_key_value_ordering(enc(r)[key], version, 3, heads // tp, hd) for r in range(tp)]
                # every rank holds [q_r; k_r; v_r]: gather the q parts of all ranks, then k, then v
                parts = [torch.cat([t.chunk(3, 0)[s] for t in per_rank], 0) for s in range(3)]
                full = torch.cat(parts, 0)
                out["%s.attn.c_attn.%s" % (name, kind)] = full.t().contiguous() if kind == "weight" else full
            elif op in ("self_attention.dense", "attention.dense"):
                t = cat(lambda r: enc(r)[key], 1) if kind == "weight" else enc(0)[key]
                out["%s.attn.c_proj.%s" % (name, kind)] = t.t().contiguous() if kind == "weight" else t.clone()
            elif op == "mlp.dense_h_to_4h":
                t = cat(lambda r: enc(r)[key], 0)
                out["%s.mlp.c_fc.%s" % (name, kind)] = t.t().contiguous() if kind == "weight" else t
            elif op == "mlp.dense_4h_to_h":
                t = cat(lambda r: enc(r)[key], 1) if kind == "weight" else enc(0)[key]
                out["%s.mlp.c_proj.%s" % (name, kind)] = t.t().contiguous() if kind == "weight" else t.clone()
        layer_offset += local_layers
    out["transformer.ln_f.weight"] = final_ln["weight"].clone()
    out["transformer.ln_f.bias"] = final_ln["bias"].clone()
    out["lm_head.weight"] = out["transformer.wte.weight"]
    config.setdefault("n_layer", layer_offset)
    if config.get("n_inner") is None:
        config["n_inner"] = out["transformer.h.0.mlp.c_fc.bias"].shape[0]
    return out, config


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--print-checkpoint-structure", action="store_true")
    ap.add_argument("--config_file", default="", type=str, help="optional GPT-2 config json")
    ap.add_argument("--path_to_checkpoint", type=str, required=True,
                    help="iteration directory holding mp_rank_* sub-directories, or one .pt file")
    ap.add_argument("--path_to_output_checkpoint", type=str, required=True)
    for flag in ("--dp", "--tp", "--pp", "--overlap_level", "--local_rank"):
        ap.add_argument(flag, default=-1, type=int, help="accepted for compatibility; not needed")
    ap.add_argument("--distributed_backend", default="none")
    o = ap.parse_args(argv)
    config = {}
    if o.config_file:
        with open(o.config_file) as f:
            config = json.load(f)
    shards = find_shards(o.path_to_checkpoint)
    state, config = convert(shards, config)
    if o.print_checkpoint_structure:
        recursive_print(None, state)
    config.update({"model_type": "gpt2", "architectures": ["GPT2LMHeadModel"], "activation_function": "gelu_new",
                   "tie_word_embeddings": True})
    config.setdefault("layer_norm_epsilon", 1e-5)
    os.makedirs(o.path_to_output_checkpoint, exist_ok=True)
    with open(os.path.join(o.path_to_output_checkpoint, "config.json"), "w") as f:
        json.dump(config, f, indent=2)
    from safetensors.torch import save_file
    tensors = {k: v.contiguous() for k, v in state.items() if k != "lm_head.weight"}   # tied to wte
    save_file(tensors, os.path.join(o.path_to_output_checkpoint, "model.safetensors"), metadata={"format": "pt"})
    print("wrote %d tensors to %s" % (len(tensors), o.path_to_output_checkpoint))
    return 0


if __name__ == "__main__":
    sys.exit(main())
