"""The LoRA fine-tuning example on a Hugging Face checkpoint directory (the reference's
examples/deepseek-r1/finetune.py:125-227): config.json + model.safetensors are written here with a
tiny Llama, the script builds the model on the meta device, loads the base weights per stage,
injects the adapters, trains over two pipeline stages and saves adapter-only checkpoints."""
import math
import os
import re
import socket
import subprocess
import sys

import pytest
import torch

transformers = pytest.importorskip("transformers")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_lora_sft_from_hf_safetensors_pp2(tmp_path):
    T = transformers
    torch.manual_seed(0)
    cfg = T.LlamaConfig(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                        intermediate_size=128, vocab_size=256, max_position_embeddings=64, tie_word_embeddings=False)
    base = T.LlamaForCausalLM(cfg)
    with torch.no_grad():
        base.lm_head.weight.zero_()       # uniform logits: the first loss is ln(vocab) iff these weights were loaded
    hf_dir = str(tmp_path / "hf")
    base.save_pretrained(hf_dir, safe_serialization=True)
    out_dir = str(tmp_path / "out")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "examples", "deepseek-r1", "finetune.py"),
           "--model_path", hf_dir, "--output_dir", out_dir, "--max_length", "32", "--dataset_size", "32",
           "--per_device_train_batch_size", "2", "--gradient_accumulation_steps", "2", "--max_steps", "3",
           "--logging_steps", "1", "--no_cuda", "true", "--report_to", "none", "--save", "true", "--save_steps", "3",
           "--learning_rate", "1e-2"]
    env = dict(os.environ, PP="2", TP="1", DP="1", OMP_NUM_THREADS="1")
    env.pop("MERAK_QUIET", None)
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    text = res.stdout + res.stderr
    assert res.returncode == 0, text[-3000:]
    losses = [float(m) for m in re.findall(r"steps: \d+ loss: ([0-9.]+)", text)]
    assert len(losses) >= 3
    assert abs(losses[0] - math.log(256)) < 2e-3, losses          # base weights came from the safetensors file
    assert all(math.isfinite(l) for l in losses)    # (adapter learning itself: tests/test_examples_cpu.py, run_lora)
    ckpt = [os.path.join(d, f) for d, _, fs in os.walk(out_dir) for f in fs]
    lora_files = [f for f in ckpt if f.endswith("lora_partial_model_optim.pt")]
    assert len(lora_files) == 2, ckpt                               # one adapter file per pipeline stage
    assert any(f.endswith("lora_config.json") for f in ckpt)
    sd = torch.load(lora_files[0], map_location="cpu", weights_only=False)["model"]
    assert sd and all("lora_" in k for k in sd), list(sd)[:5]
