"""The example scripts run end to end on CPU with tiny sizes (framework models, the generic
torch.fx path for a plain nn.Module, and the torch.export capture path)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COMMON = ["--per_device_train_batch_size", "2", "--gradient_accumulation_steps", "2", "--max_steps", "2",
          "--logging_steps", "1", "--no_cuda", "true", "--report_to", "none"]


@pytest.mark.parametrize("script,extra", [
    ("models/gpt2/run_gpt.py", ["--model_size", "gpt2-tiny", "--seq_length", "32", "--dataset_size", "32"]),
    ("image-classification/run_vit.py", ["--image_size", "32", "--hidden_size", "64", "--layers", "2", "--heads", "2",
                                         "--num_labels", "10", "--dataset_size", "32"]),
    ("unet/run_unet.py", ["--image_size", "32", "--width", "8", "--dataset_size", "32"]),
    ("lora/run_lora.py", ["--model_size", "llama-tiny", "--seq_length", "32", "--dataset_size", "32"]),
    # Hugging Face model families through torch.export tracing (tiny random configurations)
    ("models/albert/run_albert.py", ["--tiny", "1", "--dataset_size", "32"]),
    ("models/opt/run_opt.py", ["--tiny", "1", "--dataset_size", "32"]),
    ("models/bart/run_bart.py", ["--tiny", "1", "--dataset_size", "32"]),
    ("models/resnet/run_resnet.py", ["--tiny", "1", "--dataset_size", "32"]),
    ("models/convnext/run_convnext.py", ["--tiny", "1", "--dataset_size", "32"]),
    ("models/marianmt/run_marianmt.py", ["--tiny", "1", "--dataset_size", "32"]),
    ("models/wav2vec2/run_wav2vec2.py", ["--tiny", "1", "--dataset_size", "32"]),      # speech input, CTC loss hook
    ("models/clip/run_clip.py", ["--tiny", "1", "--dataset_size", "32"]),              # two towers, contrastive loss hook
])
def test_example_runs(tmp_path, script, extra):
    cmd = [sys.executable, os.path.join(ROOT, "examples", script), "--output_dir", str(tmp_path)] + extra + COMMON
    env = dict(os.environ, MERAK_QUIET="1", OMP_NUM_THREADS="2", MASTER_PORT="29%03d" % (os.getpid() % 1000))
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stderr[-3000:]
    assert "steps: 2 loss:" in (res.stdout + res.stderr)


def test_lora_vit_example_reports_accuracy(tmp_path):
    """LoRA on a traced Hugging Face ViT over two pipeline stages; the evaluation reports the accuracy
    of the last stage's logits through ``compute_metrics`` (with the batch size the graph was traced for)."""
    import re
    port = 29000 + (os.getpid() + 17) % 1000
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "examples", "lora", "run_vit.py"), "--output_dir",
           str(tmp_path), "--tiny", "1", "--dataset_size", "32", "--do_eval", "true"] + COMMON
    env = dict(os.environ, MERAK_QUIET="1", OMP_NUM_THREADS="2", PP="2")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-3000:]
    m = re.search(r"eval loss: ([0-9.]+), accuracy: ([0-9.]+)", out)
    assert m, out[-2000:]
    assert 0.0 <= float(m.group(2)) <= 1.0
    assert "trainable parameters on this stage: 2048 of" in out      # only the adapters of this stage's layer train
