"""Hugging Face model classes (``transformers`` 5.x, tiny random configurations) go through
``torch.export`` + module folding + graph sharding and train under pipeline and tensor parallelism
to the single-process loss curve (CPU / gloo).  The reference covers the same model families with
its Hugging Face fx tracer (Merak/core/fx/tracer/_symbolic_trace.py:32-127, examples/models/*)."""
import json
import os
import socket
import subprocess
import sys

import pytest

transformers = pytest.importorskip("transformers")

HERE = os.path.dirname(os.path.abspath(__file__))
SCRIPT = os.path.join(HERE, "dist_scripts", "train_hf.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run(tmp_path, name, world, extra):
    out = os.path.join(str(tmp_path), name + ".json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), SCRIPT, "--out", out] + extra
    env = dict(os.environ, OMP_NUM_THREADS="1", MERAK_QUIET="1")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert res.returncode == 0, "%s failed:\n%s\n%s" % (name, res.stdout[-3000:], res.stderr[-3000:])
    with open(out) as f:
        return json.load(f)


_SINGLE = {}


def single_run(tmp_path, model):
    if model not in _SINGLE:
        _SINGLE[model] = run(tmp_path, model + "_single", 1, ["--model", model])
    return _SINGLE[model]


def close(a, b, tol=3e-4):
    assert len(a) == len(b)
    for x, y in zip(a, b):
        assert abs(x - y) < tol * max(1.0, abs(y)), (a, b)


@pytest.mark.parametrize("model", ["gpt2", "bert", "llama", "vit", "t5"])
def test_hf_model_pp2_matches_single(tmp_path, model):
    single = single_run(tmp_path, model)
    assert single["shards"] >= 4, single            # the graph was cut into several shards
    assert single["losses"][-1] < single["losses"][0]
    pp2 = run(tmp_path, model + "_pp2", 2, ["--model", model, "--pp", "2"])
    close(pp2["losses"], single["losses"])


@pytest.mark.parametrize("model", ["gpt2", "llama", "t5"])        # t5: the relative position bias is cut by heads
def test_hf_model_tp2_matches_single(tmp_path, model):
    single = single_run(tmp_path, model)
    tp2 = run(tmp_path, model + "_tp2", 2, ["--model", model, "--tp", "2"])
    close(tp2["losses"], single["losses"])


def test_hf_model_layer_split_pp2_dp2(tmp_path):
    single = single_run(tmp_path, "gpt2")
    got = run(tmp_path, "gpt2_pp2dp2", 4, ["--model", "gpt2", "--pp", "2", "--dp", "2", "--gas", "2", "--split",
                                            "layer_split"])
    close(got["losses"], single["losses"])
