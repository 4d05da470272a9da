"""fp16 loss scaling, master-weight wrapping of user optimizers and the ZeRO-1 shard arithmetic
(reference: Merak/core/amp/fp16_optimizer.py:36-358, Merak/core/zero/stage1.py:42-757,
Merak/core/zero/utils.py:232-384).  Overflows are injected on the host."""
import json
import os
import subprocess
import sys

import pytest
import torch

from merak_b200.amp import FP16_Optimizer, MixedPrecisionConfig
from merak_b200.amp.loss_scaler import DynamicLossScaler
from merak_b200.zero import ZeroOptimizer_Stage1, is_zero_supported_optimizer

HERE = os.path.dirname(os.path.abspath(__file__))


def test_dynamic_loss_scaler_hysteresis_and_growth():
    s = DynamicLossScaler(init_scale=1024.0, scale_window=2, min_scale=1.0, hysteresis=2)
    s.update_scale(True)                 # first overflow is absorbed by the hysteresis
    assert s.cur_scale == 1024.0
    s.update_scale(True)                 # second one halves
    assert s.cur_scale == 512.0
    s.update_scale(False)
    s.update_scale(False)                # scale_window clean steps since the last overflow: doubles
    assert s.cur_scale == 1024.0
    t = DynamicLossScaler(init_scale=2.0, min_scale=1.0, hysteresis=1)
    for _ in range(5):
        t.update_scale(True)
    assert t.cur_scale == 1.0            # never below min_scale
    static = DynamicLossScaler(init_scale=128.0, static=True)
    static.update_scale(True)
    assert static.cur_scale == 128.0
    clone = DynamicLossScaler()
    clone.load_state_dict(s.state_dict())
    assert clone.cur_scale == s.cur_scale and clone.cur_hysteresis == s.cur_hysteresis


def _pair(dtype):
    torch.manual_seed(0)
    ref = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
    low = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
    low.load_state_dict(ref.state_dict())
    return ref, low.to(dtype)


def test_fp16_optimizer_tracks_fp32_and_skips_on_overflow():
    ref, low = _pair(torch.float16)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    opt = FP16_Optimizer(torch.optim.SGD(low.parameters(), lr=0.1, momentum=0.9), dynamic_loss_scale=True,
                         dynamic_loss_args=dict(init_scale=256.0, hysteresis=1, scale_window=1000))
    x = torch.randn(6, 8)
    for step in range(6):
        loss = low(x.half()).float().pow(2).mean()
        opt.backward(loss)
        if step == 2:
            low[0].weight.grad[0, 0] = float("inf")
            before = [p.detach().clone() for p in low.parameters()]
        ok = opt.step()
        if step == 2:
            assert not ok and opt.overflow and opt.cur_scale == 128.0
            for p, b in zip(low.parameters(), before):
                assert torch.equal(p, b)
            continue
        assert ok
        rl = ref(x).pow(2).mean()
        rl.backward()
        ropt.step()
        ropt.zero_grad()
        assert abs(float(loss) - float(rl)) < 5e-3 * max(1.0, abs(float(rl)))
    for p, q in zip(low.parameters(), ref.parameters()):
        assert torch.allclose(p.float(), q, atol=2e-3, rtol=2e-2)
    sd = opt.state_dict()
    opt.load_state_dict(sd)


def test_zero1_shards_compose_to_the_unsharded_step():
    """Two emulated data-parallel ranks step their halves of the flat buffers; gathered, the result is
    the unsharded optimizer's."""
    x = torch.randn(6, 8)
    models, opts = [], []
    for rank in range(2):
        _, m = _pair(torch.bfloat16)
        o = ZeroOptimizer_Stage1(torch.optim.AdamW([{"params": [m[0].weight, m[2].weight], "weight_decay": 0.1},
                                                    {"params": [m[0].bias, m[2].bias], "weight_decay": 0.0}], lr=1e-2),
                                 dp_rank=rank, dp_size=2, shard=True, max_grad_norm=0.5)
        models.append(m)
        opts.append(o)
    _, whole = _pair(torch.bfloat16)
    wopt = ZeroOptimizer_Stage1(torch.optim.AdamW([{"params": [whole[0].weight, whole[2].weight], "weight_decay": 0.1},
                                                   {"params": [whole[0].bias, whole[2].bias], "weight_decay": 0.0}],
                                                  lr=1e-2), shard=False, max_grad_norm=0.5, pad_to=128)
    assert opts[0].flat.numel % 2 == 0 and opts[0].end == opts[1].start
    for _ in range(3):
        for m, o in zip(models + [whole], opts + [wopt]):
            m(x.bfloat16()).float().pow(2).mean().backward()
            for p in o.flat.params:
                p.main_grad.add_(p.grad.float())
                p.grad = None
        ss = opts[0].grad_sumsq().clone() + opts[1].grad_sumsq()      # the data-parallel all-reduce
        for o in opts:
            o.step(sumsq=ss)
        wopt.step()
        gathered = torch.cat([o.flat.model[o.start:o.end] for o in opts])  # the parameter all-gather
        for o in opts:
            o.flat.model.copy_(gathered)
            o.zero_grad()
        wopt.zero_grad()
        assert torch.equal(gathered, wopt.flat.model)
    assert not is_zero_supported_optimizer(torch.optim.LBFGS(whole.parameters()))
    with pytest.raises(ValueError):
        _, m = _pair(torch.bfloat16)
        ZeroOptimizer_Stage1(torch.optim.LBFGS(m.parameters()), dp_rank=0, dp_size=2, shard=True)


def test_mixed_precision_config_builds_the_scaler():
    from merak_b200.args import MerakArguments
    a = MerakArguments(output_dir="/tmp/x", fp16=True, initial_scale_power=10, hysteresis=3, report_to="none")
    s = MixedPrecisionConfig(a).make_loss_scaler()
    assert s.cur_scale == 1024.0 and s.delayed_shift == 3 and not s.static
    a = MerakArguments(output_dir="/tmp/x", fp16=True, loss_scale=64.0, report_to="none")
    assert MixedPrecisionConfig(a).make_loss_scaler().static
    a = MerakArguments(output_dir="/tmp/x", bf16=True, report_to="none")
    assert MixedPrecisionConfig(a).make_loss_scaler() is None
    a = MerakArguments(output_dir="/tmp/x", fp16=True, half_precision_backend="apex", report_to="none")
    with pytest.raises(ValueError):
        MixedPrecisionConfig(a)


def test_engine_fp16_skips_the_overflowed_step_and_rescales(tmp_path):
    """The engine's fp16 path end to end: an inf written into the gradient buffer of step 2 makes the
    optimizer skip that step, the loss scale halves (hysteresis 1) and grows back after the window."""
    out = os.path.join(str(tmp_path), "fp16.json")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29700 + os.getpid() % 200), RANK="0",
               WORLD_SIZE="1", LOCAL_RANK="0", MERAK_QUIET="1", OMP_NUM_THREADS="2")
    res = subprocess.run([sys.executable, os.path.join(HERE, "dist_scripts", "train_small.py"), "--dtype", "fp16",
                          "--steps", "8", "--inject_overflow", "2", "--out", out], capture_output=True, text=True,
                         timeout=600, env=env)
    assert res.returncode == 0, res.stderr[-3000:]
    r = json.load(open(out))
    assert r["skipped"] == [False, False, True, False, False, False, False, False]
    assert r["scales"][1] == 256.0 and r["scales"][2] == 128.0 and r["scales"][-1] == 256.0
    assert r["losses"][-1] < r["losses"][0]
