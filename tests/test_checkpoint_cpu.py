"""Checkpoint format, resume and conversion: a pp=2 x tp=2 run saves per-(tp,pp) shards in the
reference layout, resumes to the same loss curve, and the merged safetensors equal the weights of
a single-process run that took the same steps."""
import glob
import json
import os
import subprocess
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from test_parallel_cpu import assert_close, run_layout  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_save_resume_convert(tmp_path):
    d4 = os.path.join(str(tmp_path), "run4")
    d1 = os.path.join(str(tmp_path), "run1")
    full = run_layout(tmp_path, "full", 1, ["--steps", "6"])
    first = run_layout(tmp_path, "first", 4, ["--pp", "2", "--tp", "2", "--steps", "3", "--save_dir", d4])
    assert_close(first, full[:3])
    ck_root = glob.glob(os.path.join(d4, "*_ckpt"))[0]
    assert open(os.path.join(ck_root, "latest_checkpointed_iteration.txt")).read().strip() == "3"
    it_dir = os.path.join(ck_root, "iter_0000003")
    names = sorted(os.listdir(it_dir))
    assert names == ["mp_rank_00_pp_rank_000", "mp_rank_00_pp_rank_001", "mp_rank_01_pp_rank_000",
                     "mp_rank_01_pp_rank_001"]
    sd = torch.load(os.path.join(it_dir, names[0], "partial_model_optim.pt"), map_location="cpu", weights_only=False)
    assert sd["checkpoint_version"] == 3.0 and sd["iteration"] == 3
    for key in ("args", "model", "optimizer", "lr_scheduler", "torch_rng_state", "rng_tracker_states"):
        assert key in sd
    keys = list(sd["model"])
    assert any(".attn.c_attn.col_linear.weight" in k for k in keys)
    assert any(".mlp.c_proj.row_linear.weight" in k for k in keys)
    assert all(k.split(".")[0].isdigit() or k.startswith("tied_modules.") for k in keys)

    # resume: three more steps continue the single-process curve
    resumed = run_layout(tmp_path, "resumed", 4, ["--pp", "2", "--tp", "2", "--steps", "3", "--resume", ck_root])
    assert_close(resumed, full[3:6], tol=5e-4)

    # convert and compare with a single-process run saved at the same step
    run_layout(tmp_path, "single3", 1, ["--steps", "3", "--save_dir", d1])
    merged = os.path.join(str(tmp_path), "merged")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "tools", "convert_safetensor.py"), "--load_path", ck_root,
                          "--save_path", merged], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    from safetensors.torch import load_file
    index = json.load(open(os.path.join(merged, "model.safetensors.index.json")))
    got = {}
    for fn in sorted(set(index["weight_map"].values())):
        got.update(load_file(os.path.join(merged, fn)))
    ref_root = glob.glob(os.path.join(d1, "*_ckpt"))[0]
    ref = torch.load(os.path.join(ref_root, "iter_0000003", "model_optim.pt"), map_location="cpu", weights_only=False)
    ref_model = {".".join(k.split(".")[1:]): v for k, v in ref["model"].items() if not k.startswith("tied_modules.")}
    assert set(got) == set(ref_model)
    for k, v in ref_model.items():
        assert got[k].shape == v.shape, k
        assert torch.allclose(got[k].float(), v.float(), atol=2e-4), k
