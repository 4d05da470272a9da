"""Text generation through the pipeline engine (Merak/inference/text_generation_inference.py:
35-274): greedy decoding under pipeline and tensor parallelism equals the single-process
result, and the logits filter keeps what top-k / top-p say it keeps."""
import json
import os
import socket
import subprocess
import sys

import torch

from merak_b200.inference.text_generation import sample_next_token, top_k_top_p_filter

HERE = os.path.dirname(os.path.abspath(__file__))
SCRIPT = os.path.join(HERE, "dist_scripts", "generate_small.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(tmp_path, name, world, extra):
    out = os.path.join(str(tmp_path), name + ".json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), SCRIPT, "--out", out] + extra
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, OMP_NUM_THREADS="1", MERAK_QUIET="1"))
    assert res.returncode == 0, "%s failed:\n%s\n%s" % (name, res.stdout[-3000:], res.stderr[-3000:])
    with open(out) as f:
        return json.load(f)


def test_greedy_generation_pp2_and_tp2_match_single(tmp_path):
    single = _run(tmp_path, "single", 1, [])
    assert all(len(seq) == 8 + 6 for seq in single["greedy"])
    assert single["greedy"][0][:8] == [5, 17, 99, 256, 3, 44, 7, 120]
    assert all(0 <= t < 512 for seq in single["sampled"] for t in seq)
    pp2 = _run(tmp_path, "pp2", 2, ["--pp", "2"])
    assert pp2["greedy"] == single["greedy"]
    tp2 = _run(tmp_path, "tp2", 2, ["--tp", "2"])            # vocabulary-parallel head: shards gathered per token
    assert tp2["greedy"] == single["greedy"]


def test_top_k_top_p_filter():
    logits = torch.tensor([[1.0, 3.0, 2.0, 0.0, -1.0]])
    kept = top_k_top_p_filter(logits, top_k=2)
    assert torch.isinf(kept[0, [0, 3, 4]]).all() and kept[0, 1] == 3.0 and kept[0, 2] == 2.0
    probs = torch.tensor([[0.5, 0.3, 0.15, 0.05]])
    kept = top_k_top_p_filter(probs.log(), top_p=0.7)
    # the smallest prefix of the sorted distribution whose mass exceeds 0.7: {0.5, 0.3}
    assert torch.isfinite(kept[0, :2]).all() and torch.isinf(kept[0, 2:]).all()
    g = torch.Generator().manual_seed(0)
    draws = {int(sample_next_token(probs.log(), temperature=1.0, top_k=0, top_p=0.7, generator=g)) for _ in range(50)}
    assert draws <= {0, 1}
    assert int(sample_next_token(logits, greedy=True)) == 1
