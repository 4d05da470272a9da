"""Fused data-parallel kernels (gradient reduce-scatter + AdamW + parameter all-gather over
peer-mapped memory).  On one GPU the ranks are emulated: all ranks' buffers live on the same device
and the kernels run rank after rank with the cross-rank barriers switched off; the two-process
test needs two GPUs."""
import ctypes
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
SCRIPT = os.path.join(HERE, "dist_scripts", "train_small.py")


def _table(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def _adam_ref(p, m, v, g, lr, b1, b2, eps, wd, t):
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    p = p * (1 - lr * wd) - lr * (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + eps)
    return p, m, v


@pytest.mark.parametrize("n", [1, 2, 3, 4])
def test_dp_kernels_emulated_ranks(n):
    from merak_b200.ops import _lib
    lib = _lib.kernels()
    dev = torch.device("cuda")
    torch.manual_seed(n)
    numel = 64 * n * 37
    per = numel // n
    grads = [torch.randn(numel, device=dev) * 0.1 for _ in range(n)]
    grads_in = [g.clone() for g in grads]
    models = [torch.zeros(numel, dtype=torch.bfloat16, device=dev) for _ in range(n)]
    ctrl_bytes = lib.mrk_symm_ctrl_bytes()
    ctrls = [torch.zeros(ctrl_bytes, dtype=torch.uint8, device=dev) for _ in range(n)]
    flags = torch.zeros(numel // 64 + 1, dtype=torch.uint8, device=dev)
    flags[: numel // 128] = 1                     # first half decays
    flags[numel // 64 - 3: numel // 64] |= 2      # last three granules are not counted in the norm
    master_full = torch.randn(numel, device=dev)
    masters = [master_full[r * per:(r + 1) * per].clone() for r in range(n)]
    ms = [torch.zeros(per, device=dev) for _ in range(n)]
    vs = [torch.zeros(per, device=dev) for _ in range(n)]
    lr, b1, b2, eps, wd, t = 1e-2, 0.9, 0.999, 1e-8, 0.1, 1
    hp = torch.tensor([lr, b1, b2, eps, wd, 1 - b1 ** t, 1 - b2 ** t], device=dev)
    norm_out = torch.zeros(1, device=dev)
    skip_out = torch.zeros(1, dtype=torch.int32, device=dev)
    gt, mt, ct = _table([g.data_ptr() for g in grads]), _table([m.data_ptr() for m in models]), \
        _table([c.data_ptr() for c in ctrls])
    st = _lib.stream_ptr()
    for r in range(n):
        _lib.check(lib.mrk_dp_reduce_scatter(gt, ct, n, r, r * per, per, flags.data_ptr(), 1, 0, 100, st), "rs")
    grad_scale, max_norm = 1.0 / n, 0.5
    for r in range(n):
        _lib.check(lib.mrk_dp_adamw_allgather(mt, ct, n, r, r * per, per, grads[r].data_ptr() + 4 * r * per,
                                              masters[r].data_ptr(), ms[r].data_ptr(), vs[r].data_ptr(),
                                              flags.data_ptr(), hp.data_ptr(), grad_scale, max_norm, None,
                                              norm_out.data_ptr(), skip_out.data_ptr(), 1, 0, 1, 100, st), "ag")
    torch.cuda.synchronize()
    assert _lib.status() == 0
    total = torch.stack(grads_in).sum(0)
    counted = total.clone()
    counted[(numel // 64 - 3) * 64:] = 0
    norm = counted.double().pow(2).sum().sqrt().item() * grad_scale
    assert abs(norm_out.item() - norm) < 1e-4 * norm
    assert skip_out.item() == 0
    coef = grad_scale * (max_norm / (norm + 1e-6) if norm > max_norm else 1.0)
    wd_vec = torch.zeros(numel, device=dev)
    wd_vec[: (numel // 128) * 64] = wd
    p_ref, m_ref, v_ref = _adam_ref(master_full, torch.zeros_like(total), torch.zeros_like(total), total * coef,
                                    lr, b1, b2, eps, wd_vec, t)
    for r in range(n):
        sl = slice(r * per, (r + 1) * per)
        torch.testing.assert_close(grads[r][sl], total[sl], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(masters[r], p_ref[sl], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(ms[r], m_ref[sl], rtol=1e-5, atol=1e-7)
        torch.testing.assert_close(vs[r], v_ref[sl], rtol=1e-5, atol=1e-9)
    for k in range(n):
        torch.testing.assert_close(models[k].float(), p_ref.bfloat16().float(), rtol=0, atol=0)


@pytest.mark.parametrize("n", [2, 3, 4])
def test_dp_staged_reduce_emulated_ranks(n):
    """Overlapped reduction: every rank copies the pieces of its gradient buffer that other ranks own
    into the owners' staging slots (device-to-device copies, piece after piece from the end of the
    buffer), then the reduce-scatter kernel sums its own buffer and its staging slots."""
    from merak_b200.ops import _lib
    lib = _lib.kernels()
    dev = torch.device("cuda")
    torch.manual_seed(10 + n)
    numel = 64 * n * 41
    per = numel // n
    grads = [torch.randn(numel, device=dev) * 0.1 for _ in range(n)]
    total = torch.stack(grads).sum(0)
    stages = [torch.zeros(n * per, device=dev) for _ in range(n)]
    ctrls = [torch.zeros(lib.mrk_symm_ctrl_bytes(), dtype=torch.uint8, device=dev) for _ in range(n)]
    flags = torch.zeros(numel // 64 + 1, dtype=torch.uint8, device=dev)
    flags[numel // 64 - 2: numel // 64] |= 2                          # not counted in the norm
    ct = _table([c.data_ptr() for c in ctrls])
    st = _lib.stream_ptr()
    cuts = sorted({0, numel, 64 * 7, per + 64 * 3, numel - 64 * 9, (numel // 2) // 64 * 64})
    for lo, hi in list(zip(cuts, cuts[1:]))[::-1]:
        for src in range(n):
            for own in range(n):
                a, b = max(lo, own * per), min(hi, (own + 1) * per)
                if own != src and a < b:
                    dst = stages[own].data_ptr() + 4 * (src * per + a - own * per)
                    _lib.check(lib.mrk_memcpy_d2d_async(dst, grads[src].data_ptr() + 4 * a, 4 * (b - a), st), "copy")
    for r in range(n):
        table = _table([grads[r].data_ptr() if k == r else stages[r].data_ptr() + 4 * (k * per - r * per)
                        for k in range(n)])
        _lib.check(lib.mrk_dp_reduce_scatter(table, ct, n, r, r * per, per, flags.data_ptr(), 1, 0, 100, st), "sum")
    torch.cuda.synchronize()
    assert _lib.status() == 0
    counted = total.clone()
    counted[(numel // 64 - 2) * 64:] = 0
    want = counted.double().pow(2).sum().item()
    for r in range(n):
        sl = slice(r * per, (r + 1) * per)
        torch.testing.assert_close(grads[r][sl], total[sl], rtol=1e-5, atol=1e-6)
        slots = ctrls[r].view(torch.float32)[16 * 16: 16 * 16 + 4 * n].view(n, 4)   # posted (sumsq, bad) per source
        got = slots[:, 0].double().sum().item()
        assert abs(got - want) < 1e-4 * want, (got, want)
        assert slots[:, 1].abs().sum().item() == 0


def test_nonfinite_gradient_skips_update():
    from merak_b200.ops import _lib
    lib = _lib.kernels()
    dev = torch.device("cuda")
    numel = 64 * 8
    grad = torch.ones(numel, device=dev)
    grad[5] = float("inf")
    model = torch.zeros(numel, dtype=torch.bfloat16, device=dev)
    ctrl = torch.zeros(lib.mrk_symm_ctrl_bytes(), dtype=torch.uint8, device=dev)
    master = torch.ones(numel, device=dev)
    m, v = torch.zeros(numel, device=dev), torch.zeros(numel, device=dev)
    hp = torch.tensor([1e-2, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001], device=dev)
    norm_out, skip_out = torch.zeros(1, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    gt, mt, ct = _table([grad.data_ptr()]), _table([model.data_ptr()]), _table([ctrl.data_ptr()])
    st = _lib.stream_ptr()
    _lib.check(lib.mrk_dp_reduce_scatter(gt, ct, 1, 0, 0, numel, None, 1, 0, 100, st), "rs")
    _lib.check(lib.mrk_dp_adamw_allgather(mt, ct, 1, 0, 0, numel, grad.data_ptr(), master.data_ptr(), m.data_ptr(),
                                          v.data_ptr(), None, hp.data_ptr(), 1.0, 1.0, None, norm_out.data_ptr(),
                                          skip_out.data_ptr(), 1, 0, 1, 100, st), "ag")
    torch.cuda.synchronize()
    assert skip_out.item() == 1
    assert torch.equal(master, torch.ones_like(master)) and torch.equal(m, torch.zeros_like(m))


def test_barrier_wait_runs_out_and_reports():
    """A flag that nothing sets: the bounded wait gives up, the status word says so, and the
    context stays usable."""
    from merak_b200.ops import _lib
    lib = _lib.kernels()
    dev = torch.device("cuda")
    ctrls = [torch.zeros(lib.mrk_symm_ctrl_bytes(), dtype=torch.uint8, device=dev) for _ in range(2)]
    ct = _table([c.data_ptr() for c in ctrls])
    torch.cuda.synchronize()
    _lib.status(clear=True)
    # rank 0 signals and waits for rank 1, which never runs
    _lib.check(lib.mrk_symm_barrier(ct, 2, 0, 3, 1, 1, 20, _lib.stream_ptr()), "barrier")
    torch.cuda.synchronize()
    assert _lib.status(clear=True) & 2, "the flag wait should have timed out"
    # rank 1 arrives later: both flags are now set and the wait of rank 1 completes at once
    _lib.check(lib.mrk_symm_barrier(ct, 2, 1, 3, 1, 1, 20, _lib.stream_ptr()), "barrier")
    torch.cuda.synchronize()
    assert _lib.status(clear=True) == 0
    x = torch.ones(1024, device=dev)
    assert float((x * 2).sum()) == 2048.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(tmp, name, world, extra):
    import json
    out = os.path.join(str(tmp), name + ".json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), SCRIPT, "--out", out,
           "--device", "cuda", "--dtype", "bf16"] + extra
    env = dict(os.environ, MERAK_QUIET="1", NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, "%s failed:\n%s\n%s" % (name, res.stdout[-3000:], res.stderr[-3000:])
    with open(out) as f:
        return json.load(f)["losses"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("model", ["gpt2", "bert"])
def test_tp2_dropout_keeps_replicated_parameters_identical(tmp_path, model):
    """Tensor parallelism with dropout switched on (hidden, embedding, attention probabilities): activations
    every rank holds get the same mask on every rank, so parameters that are not sharded (norms, row-parallel
    biases, position embeddings) receive identical gradients and stay bit-identical; the script checks that
    after the last step and fails otherwise."""
    losses = _run(tmp_path, "tp2_dropout", 2, ["--model", model, "--tp", "2", "--steps", "5", "--gas", "2",
                                               "--dropout", "0.1", "--check_replicated", "1"])
    assert all(l == l for l in losses) and losses[-1] < losses[0] + 0.5


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("model", ["gpt2", "bert"])
def test_fused_dp_matches_nccl_two_gpus(tmp_path, model):
    base = ["--model", model, "--dp", "2", "--steps", "6", "--gas", "2"]
    ref = _run(tmp_path, "nccl", 2, base + ["--comm", "nccl"])
    fused = _run(tmp_path, "fused", 2, base + ["--comm", "fused"])
    assert fused[-1] < fused[0]
    for a, b in zip(fused, ref):
        assert abs(a - b) < 2e-2 * max(1.0, abs(b)), (fused, ref)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("graph,gas", [(0, 2), (1, 1)])
def test_fused_dp_overlapped_with_backward_two_gpus(tmp_path, graph, gas):
    """Pieces of the gradient buffer travel to their owners while the backward pass runs (eagerly on
    the last micro-batch, or as a side branch of the captured graph): same losses as the serial
    reduction."""
    base = ["--model", "gpt2", "--dp", "2", "--steps", "6", "--gas", str(gas), "--comm", "fused",
            "--cuda_graph", str(graph)]
    serial = _run(tmp_path, "serial", 2, base + ["--dp_overlap", "0"])
    overlapped = _run(tmp_path, "overlap", 2, base + ["--dp_overlap", "1", "--dp_bucket", "4096"])
    assert overlapped[-1] < overlapped[0]
    for a, b in zip(overlapped, serial):
        assert abs(a - b) < 2e-3 * max(1.0, abs(b)), (overlapped, serial)


# ---- tensor-parallel fused GEMMs, ranks emulated on one GPU --------------------------------------
def _preset_flags(ctrls, which, epoch):
    """Marks barrier `which` as already reached by every source (the emulated ranks run one after
    the other, so nobody could signal in time)."""
    for c in ctrls:
        c.view(torch.int32)[which * 16: which * 16 + 16] = epoch


@pytest.mark.parametrize("n,B,seg,N", [(2, 2, 128, 512), (4, 1, 256, 256), (3, 3, 64, 160)])
def test_reduce_pull_and_gather_rows_emulated(n, B, seg, N):
    from merak_b200.ops import _lib
    lib = _lib.kernels()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    L = seg * n
    M = B * L
    parts = [torch.randn(M, N, device=dev, dtype=torch.bfloat16) for _ in range(n)]
    bias = torch.randn(N, device=dev, dtype=torch.bfloat16)
    ctrls = [torch.zeros(lib.mrk_symm_ctrl_bytes(), dtype=torch.uint8, device=dev) for _ in range(n)]
    pt, ct = _table([a.data_ptr() for a in parts]), _table([c.data_ptr() for c in ctrls])
    st = _lib.stream_ptr()
    ref = sum(p_.float() for p_ in parts) + bias.float()
    ref3 = ref.view(B, n, seg, N)
    reds = [torch.empty(M // n, N, dtype=torch.bfloat16, device=dev) for _ in range(n)]
    for r in range(n):
        _lib.check(lib.mrk_tp_reduce_pull(pt, ct, n, r, reds[r].data_ptr(), M // n, N, seg, bias.data_ptr(), 1, 0, 50,
                                          st), "pull")
    rt = _table([a.data_ptr() for a in reds])
    outs = []
    for r in range(n):
        o = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        _lib.check(lib.mrk_tp_gather_rows(rt, ct, n, r, o.data_ptr(), M, N, seg, 1, 0, 50, st), "gather")
        outs.append(o)
    torch.cuda.synchronize()
    assert _lib.status() == 0
    for r in range(n):
        torch.testing.assert_close(reds[r].float().view(B, seg, N), ref3[:, r].bfloat16().float(), rtol=0, atol=0)
        torch.testing.assert_close(outs[r].float(), ref.bfloat16().float(), rtol=0, atol=0)


@pytest.mark.parametrize("n,B,seg,K,N", [(2, 2, 128, 256, 512), (4, 1, 256, 128, 384), (2, 1, 64, 64, 96)])
def test_allgather_gemm_emulated(n, B, seg, K, N):
    from merak_b200.ops import _lib
    lib = _lib.kernels()
    dev = torch.device("cuda")
    torch.manual_seed(1)
    L = seg * n
    M = B * L
    x = torch.randn(B, L, K, device=dev, dtype=torch.bfloat16)
    shards = [x[:, r * seg:(r + 1) * seg].contiguous().view(-1, K) for r in range(n)]
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.1
    bias = torch.randn(N, device=dev, dtype=torch.bfloat16)
    ctrls = [torch.zeros(lib.mrk_symm_ctrl_bytes(), dtype=torch.uint8, device=dev) for _ in range(n)]
    _preset_flags(ctrls, 4, 1)
    stt, ct = _table([s.data_ptr() for s in shards]), _table([c.data_ptr() for c in ctrls])
    ref = x.view(M, K).float() @ w.float().t() + bias.float()
    G = 4
    for r in range(n):
        flags = torch.zeros(M // seg, dtype=torch.int32, device=dev)
        gathered = torch.zeros(M, K, dtype=torch.bfloat16, device=dev)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        _lib.check(lib.mrk_gemm_bf16_ag(gathered.data_ptr(), stt, w.data_ptr(), y.data_ptr(), M, N, K, K, N,
                                        bias.data_ptr(), None, 0, 0, 0, 1.0, ct, flags.data_ptr(), G, G, n, r, seg,
                                        1, 200, _lib.stream_ptr()), "ag")
        torch.cuda.synchronize()
        assert _lib.status() == 0
        assert torch.equal(gathered, x.view(M, K))
        assert int(flags.min()) == int(flags.max()) and int(flags.min()) % G == 0 and int(flags.min()) >= G   # every gather worker counted once
        torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("sp", [0, 1])
def test_fused_tp_matches_nccl_two_gpus(tmp_path, sp):
    base = ["--model", "gpt2", "--tp", "2", "--steps", "6", "--gas", "2", "--megatron_sp", str(sp)]
    ref = _run(tmp_path, "nccl", 2, base + ["--comm", "nccl"])
    fused = _run(tmp_path, "fused", 2, base + ["--comm", "fused"])
    assert fused[-1] < fused[0]
    for a, b in zip(fused, ref):
        assert abs(a - b) < 2e-2 * max(1.0, abs(b)), (fused, ref)


def test_moe_alltoall_push_emulated():
    """Rows of every emulated rank land in the destination's buffer at the offset reserved for the
    source (ranks run one after the other on one GPU, barriers off)."""
    from merak_b200.ops import _lib
    lib = _lib.kernels()
    dev = torch.device("cuda")
    torch.manual_seed(3)
    n, H = 3, 64
    C = [[5, 0, 7], [2, 9, 1], [4, 4, 0]]          # rows source -> destination
    sends = [torch.randn(sum(C[s]), H, device=dev, dtype=torch.bfloat16) for s in range(n)]
    recvs = [torch.zeros(sum(C[s][d] for s in range(n)), H, device=dev, dtype=torch.bfloat16) for d in range(n)]
    ctrls = [torch.zeros(lib.mrk_symm_ctrl_bytes(), dtype=torch.uint8, device=dev) for _ in range(n)]
    rt, ct = _table([r.data_ptr() for r in recvs]), _table([c.data_ptr() for c in ctrls])
    for s in range(n):
        begin = [0]
        for d in range(n):
            begin.append(begin[-1] + C[s][d])
        dst_row = [sum(C[q][d] for q in range(s)) for d in range(n)]
        sb = (ctypes.c_longlong * (n + 1))(*begin)
        dr = (ctypes.c_longlong * n)(*dst_row)
        _lib.check(lib.mrk_moe_alltoall_push(rt, ct, n, s, sends[s].data_ptr(), sb, dr, H, 2, 1, 0, 50,
                                             _lib.stream_ptr()), "push")
    torch.cuda.synchronize()
    assert _lib.status() == 0
    for d in range(n):
        want = torch.cat([sends[s][sum(C[s][:d]):sum(C[s][:d + 1])] for s in range(n)])
        assert torch.equal(recvs[d], want)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_moe_expert_parallel_fused_matches_nccl_two_gpus(tmp_path):
    base = ["--model", "moe", "--dp", "2", "--ep", "2", "--steps", "6", "--gas", "2"]
    ref = _run(tmp_path, "nccl", 2, base + ["--comm", "nccl"])
    fused = _run(tmp_path, "fused", 2, base + ["--comm", "fused"])
    assert fused[-1] < fused[0]
    for a, b in zip(fused, ref):
        assert abs(a - b) < 3e-2 * max(1.0, abs(b)), (fused, ref)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ulysses_sequence_parallel_fused_matches_nccl_two_gpus(tmp_path):
    """Ulysses head/sequence all-to-all through the peer-store kernel against all_to_all_single."""
    base = ["--model", "llama", "--sp", "2", "--steps", "6", "--gas", "2"]
    ref = _run(tmp_path, "nccl", 2, base + ["--comm", "nccl"])
    fused = _run(tmp_path, "fused", 2, base + ["--comm", "fused"])
    assert fused[-1] < fused[0]
    for a, b in zip(fused, ref):
        assert abs(a - b) < 2e-2 * max(1.0, abs(b)), (fused, ref)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_flag_barriers_with_skewed_ranks_two_gpus(tmp_path):
    """Signal-flag protocol with one rank arriving 0.4 s late at every step: no timeout, right sums."""
    import json
    out = str(tmp_path / "skew.json")
    script = os.path.join(HERE, "dist_scripts", "symm_barrier_skew.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), script, out]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert res.returncode == 0, res.stderr[-3000:]
    with open(out) as f:
        r = json.load(f)
    assert r["ok"] == 1 and r["status"] == 0, r


@pytest.mark.parametrize("n,B,L,N,K", [(2, 1, 512, 512, 256), (4, 2, 512, 384, 192), (2, 3, 256, 1600, 128)])
def test_gemm_reduce_scatter_one_launch_emulated(n, B, L, N, K):
    """GEMM -> reduce-scatter kernel with the ranks emulated on one GPU: first every rank multiplies
    and publishes its sub-tile flags (phase 1), then every rank reduces the sub-tiles it owns
    (phase 2); in production both phases are one launch per rank.  Oracle: fp32 PyTorch."""
    from merak_b200.ops import _lib
    lib = _lib.kernels()
    dev = torch.device("cuda")
    torch.manual_seed(n * 100 + N)
    M, seg = B * L, L // n
    xs = [torch.randn(M, K, device=dev, dtype=torch.bfloat16) * 0.5 for _ in range(n)]
    ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.5 for _ in range(n)]
    bias = torch.randn(N, device=dev, dtype=torch.bfloat16)
    parts = [torch.zeros(M, N, device=dev, dtype=torch.bfloat16) for _ in range(n)]
    units = int(lib.mrk_gemm_bf16_rs_units(M, N))
    flags = [torch.zeros(n * units, dtype=torch.int32, device=dev) for _ in range(n)]
    outs = [torch.zeros(M // n, N, device=dev, dtype=torch.bfloat16) for _ in range(n)]
    queue = torch.zeros(1, dtype=torch.int32, device=dev)
    pt, ft = _table([p_.data_ptr() for p_ in parts]), _table([f.data_ptr() for f in flags])
    st = _lib.stream_ptr()
    torch.cuda.synchronize()
    _lib.status(clear=True)
    for epoch in (1, 2):                       # twice: flags of the first call must not satisfy the second
        if epoch == 2:
            xs = [x * 0.5 for x in xs]
        for phase in (1, 2):
            for r in range(n):
                _lib.check(lib.mrk_gemm_bf16_rs(xs[r].data_ptr(), ws[r].data_ptr(), pt, ft, outs[r].data_ptr(),
                                                bias.data_ptr(), M, N, K, K, K, 0, n, r, seg, epoch, phase, 8,
                                                queue.data_ptr(), 200, st),
                           "gemm_rs")
        torch.cuda.synchronize()
        assert _lib.status(clear=True) == 0
        full = sum(x.float() @ w.float().t() for x, w in zip(xs, ws)) + bias.float()
        ref = full.view(B, n, seg, N)
        for r in range(n):
            want = ref[:, r].reshape(M // n, N)
            torch.testing.assert_close(outs[r].float(), want, rtol=3e-2, atol=3e-1)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_gemm_reduce_scatter_one_launch_two_gpus(tmp_path):
    """The one-launch GEMM -> reduce-scatter on real peers: sub-tile flags cross NVLink, owners pull the
    partial products while the other rank is still multiplying."""
    import json
    out = str(tmp_path / "rs.json")
    script = os.path.join(HERE, "dist_scripts", "tp_gemm_rs.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), script, "--out", out, "--shapes",
           "1x1024x512x256,2x512x1600x320,4x1024x4096x512"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert res.returncode == 0, res.stderr[-3000:]
    with open(out) as f:
        r = json.load(f)
    assert r["status"] == 0 and all(x["ok"] for x in r["results"]), r
