"""Norm / cross-entropy / AdamW / embedding / RoPE / SwiGLU / linear kernels vs PyTorch fp32."""
import math

import pytest
import torch
import torch.nn.functional as F

from merak_b200.ops import _lib
from merak_b200.ops import gemm as G
from merak_b200.ops.cross_entropy import softmax_cross_entropy
from merak_b200.ops.elementwise import apply_rope, colsum, dropout, embedding_sum, rope_reference, rope_tables, swiglu
from merak_b200.ops.linear import linear, mlp
from merak_b200.ops.norm import fused_norm
from merak_b200.ops.optim import FlatBuffers, FusedAdamW

pytestmark = pytest.mark.gpu


def rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


@pytest.mark.parametrize("H", [256, 1024, 1600, 4096, 8192])
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("residual", [False, True])
def test_norm_fwd_bwd(H, rms, residual):
    torch.manual_seed(0)
    M = 300
    x = torch.randn(M, H, device="cuda").bfloat16().requires_grad_()
    r = torch.randn(M, H, device="cuda").bfloat16().requires_grad_() if residual else None
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_()
    b = None if rms else (0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_()
    y, z = fused_norm(x, w, b, r, 1e-5, rms)
    dy, dz = torch.randn_like(y), torch.randn_like(z)
    (y.float() * dy.float()).sum().add((z.float() * dz.float()).sum()).backward()
    torch.cuda.synchronize()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    rr = r.detach().float().requires_grad_() if residual else None
    br = b.detach().float().requires_grad_() if b is not None else None
    zr = xr + rr if residual else xr
    zr_b = zr + (zr.bfloat16().float() - zr).detach()           # forward on rounded values
    if rms:
        yr = zr_b * torch.rsqrt(zr_b.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    else:
        yr = F.layer_norm(zr_b, (H,), wr, br, 1e-5)
    ((yr * dy.float()).sum() + (zr * dz.float()).sum()).backward()
    assert rel(y, yr) < 2e-2
    assert rel(x.grad, xr.grad) < 2e-2
    if residual:
        assert rel(r.grad, rr.grad) < 2e-2
    assert rel(w.grad, wr.grad) < 3e-2
    if b is not None:
        assert rel(b.grad, br.grad) < 3e-2


def test_norm_dropout_mask_consistency():
    torch.manual_seed(0)
    M, H, p = 256, 1024, 0.25
    x = torch.ones(M, H, device="cuda").bfloat16().requires_grad_()
    w = torch.ones(H, device="cuda").bfloat16().requires_grad_()
    b = torch.zeros(H, device="cuda").bfloat16().requires_grad_()
    y, z = fused_norm(x, w, b, None, 1e-5, False, p_drop=p, training=True)
    keep = (z != 0).float()
    frac = keep.mean().item()
    assert abs(frac - (1 - p)) < 0.02
    assert torch.allclose(z[z != 0].float(), torch.full_like(z[z != 0].float(), 1 / (1 - p)), atol=1e-2)
    z.float().sum().backward()        # gradient only through z: dx = mask / (1-p)
    torch.cuda.synchronize()
    assert torch.allclose(x.grad.float(), keep / (1 - p), atol=1e-2)


@pytest.mark.parametrize("V", [30522, 50257, 32000])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cross_entropy(V, dtype):
    torch.manual_seed(0)
    M = 257
    logits = (torch.randn(M, V, device="cuda") * 2).to(dtype).requires_grad_()
    labels = torch.randint(0, V, (M,), device="cuda")
    labels[::5] = -100
    loss = softmax_cross_entropy(logits, labels)
    loss.backward()
    torch.cuda.synchronize()
    lr = logits.detach().float().requires_grad_()
    ref = F.cross_entropy(lr, labels, ignore_index=-100)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1.0, abs(ref.item()))
    assert (logits.grad.float() - lr.grad).abs().max().item() < (1e-4 if dtype == torch.float32 else 2e-4)


def test_adamw_matches_torch():
    torch.manual_seed(0)
    shapes = [(64, 128), (128,), (33, 7), (256, 256)]
    params = [torch.nn.Parameter(torch.randn(s, device="cuda").bfloat16()) for s in shapes]
    ref = [torch.nn.Parameter(p.detach().float().clone()) for p in params]
    flat = FlatBuffers(params)
    opt = FusedAdamW(flat, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0)
    decay = [p for p in ref if p.dim() > 1]
    nodecay = [p for p in ref if p.dim() <= 1]
    topt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": nodecay, "weight_decay": 0.0}],
                             lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    for step in range(5):
        for p, r in zip(params, ref):
            g = torch.randn_like(r)
            p.main_grad.copy_(g)
            r.grad = g.clone()
        torch.nn.utils.clip_grad_norm_(ref, 1.0)
        topt.step()
        opt.step()
        flat.zero_grad()
    torch.cuda.synchronize()
    for p, r, o in zip(params, ref, flat.offsets):
        m = opt.master[o:o + r.numel()].view(r.shape)
        assert (m - r).abs().max().item() < 1e-4
        assert (p.float() - r).abs().max().item() < 2e-2


def test_embedding_rope_swiglu_colsum_dropout():
    torch.manual_seed(0)
    V, P, H, B, L = 1000, 64, 256, 4, 48
    wt = torch.nn.Parameter(torch.randn(V, H, device="cuda").bfloat16())
    pt = torch.nn.Parameter(torch.randn(P, H, device="cuda").bfloat16())
    ids = torch.randint(0, V, (B, L), device="cuda")
    pos = torch.arange(L, device="cuda")[None].expand(B, L)
    out = embedding_sum([ids, pos], [wt, pt])
    ref = F.embedding(ids, wt.float()) + F.embedding(pos, pt.float())
    assert rel(out, ref) < 1e-2
    g = torch.randn_like(out)
    out.backward(g)
    rw = torch.zeros(V, H, device="cuda").index_add_(0, ids.reshape(-1), g.float().reshape(-1, H))
    assert rel(wt.grad, rw) < 2e-2
    # vocab-parallel style range restriction
    out2 = embedding_sum([ids], [wt[500:].detach().contiguous()], [500])
    ref2 = F.embedding((ids - 500).clamp(min=0), wt[500:].float()) * (ids >= 500).unsqueeze(-1)
    assert rel(out2, ref2) < 1e-2
    # rope
    D, Hh = 128, 4
    x = torch.randn(B, L, Hh, D, device="cuda").bfloat16().requires_grad_()
    cos, sin = rope_tables(L, D, device="cuda")
    y = apply_rope(x, cos, sin)
    assert rel(y, rope_reference(x.detach(), cos, sin)) < 1e-2
    gy = torch.randn_like(y)
    y.backward(gy)
    assert rel(x.grad, rope_reference(gy, cos, sin, inverse=True)) < 1e-2
    # swiglu
    gu = torch.randn(B * L, 2 * 512, device="cuda").bfloat16().requires_grad_()
    o = swiglu(gu)
    gr = gu.detach().float().requires_grad_()
    orf = F.silu(gr[:, :512]) * gr[:, 512:]
    go = torch.randn_like(o)
    o.backward(go)
    orf.backward(go.float())
    assert rel(o, orf) < 1e-2 and rel(gu.grad, gr.grad) < 2e-2
    # colsum
    xx = torch.randn(1000, 770, device="cuda").bfloat16()
    assert rel(colsum(xx), xx.float().sum(0)) < 1e-3
    # dropout
    xd = torch.ones(1024, 512, device="cuda").bfloat16().requires_grad_()
    yd = dropout(xd, 0.5)
    yd.sum().backward()
    assert abs((yd != 0).float().mean().item() - 0.5) < 0.02
    assert torch.equal(xd.grad != 0, yd != 0)
    torch.cuda.synchronize()
    _lib.assert_status_ok("elementwise")


def test_linear_and_mlp_autograd():
    torch.manual_seed(0)
    B, L, K, F1, N = 4, 96, 256, 1024, 256
    x = torch.randn(B, L, K, device="cuda").bfloat16().requires_grad_()
    res = torch.randn(B, L, N, device="cuda").bfloat16().requires_grad_()
    w1 = torch.nn.Parameter((torch.randn(F1, K, device="cuda") * 0.05).bfloat16())
    b1 = torch.nn.Parameter((torch.randn(F1, device="cuda") * 0.05).bfloat16())
    w2 = torch.nn.Parameter((torch.randn(N, F1, device="cuda") * 0.05).bfloat16())
    b2 = torch.nn.Parameter((torch.randn(N, device="cuda") * 0.05).bfloat16())
    y = mlp(x, w1, b1, w2, b2, G.ACT_GELU_ERF, res)
    gy = torch.randn_like(y)
    y.backward(gy)
    torch.cuda.synchronize()
    xr, rr = x.detach().float().requires_grad_(), res.detach().float().requires_grad_()
    p = [t.detach().float().requires_grad_() for t in (w1, b1, w2, b2)]
    yr = F.linear(F.gelu(F.linear(xr, p[0], p[1])), p[2], p[3]) + rr
    yr.backward(gy.float())
    assert rel(y, yr) < 2e-2
    assert rel(x.grad, xr.grad) < 3e-2 and rel(res.grad, rr.grad) < 1e-2
    for t, r in zip((w1, b1, w2, b2), p):
        assert rel(t.grad, r.grad) < 3e-2
    # plain linear with main_grad accumulation
    w = torch.nn.Parameter((torch.randn(N, K, device="cuda") * 0.05).bfloat16())
    w.main_grad = torch.zeros(N, K, device="cuda")
    x2 = torch.randn(B, L, K, device="cuda").bfloat16().requires_grad_()
    for _ in range(2):
        linear(x2, w).backward(gy)
    torch.cuda.synchronize()
    ref = 2 * (gy.float().reshape(-1, N).t() @ x2.detach().float().reshape(-1, K))
    assert w.grad is None and rel(w.main_grad, ref) < 2e-2
    _lib.assert_status_ok("linear")


@pytest.mark.parametrize("act", ["gelu_erf", "gelu_tanh", "relu", "silu"])
@pytest.mark.parametrize("M,N", [(1000, 4096), (37, 264)])
def test_activation_passes_between_the_mlp_gemms(act, M, N):
    """act(h) and d * act'(h) with the bias-gradient column sums in the same pass, against fp32 PyTorch."""
    from merak_b200.ops.elementwise import act_backward, act_forward
    code = {"gelu_erf": G.ACT_GELU_ERF, "gelu_tanh": G.ACT_GELU_TANH, "relu": G.ACT_RELU, "silu": G.ACT_SILU}[act]
    torch.manual_seed(0)
    h = (torch.randn(M, N, device="cuda") * 2.5).bfloat16()
    d = torch.randn(M, N, device="cuda").bfloat16()
    hr = h.float().requires_grad_()
    yr = G.act_forward(code, hr)
    yr.backward(d.float())
    y = act_forward(code, h)
    torch.testing.assert_close(y.float(), yr.detach(), rtol=1e-2, atol=2e-3)
    acc = torch.ones(N, device="cuda")
    dh = act_backward(code, d.clone(), h, acc)
    torch.testing.assert_close(dh.float(), hr.grad, rtol=1e-2, atol=3e-3)
    torch.testing.assert_close(acc, 1.0 + dh.float().sum(0), rtol=1e-3, atol=1e-2)
    # the tails of the erf polynomial: exact zero / identity far from the origin
    far = torch.tensor([[-30.0, -6.0, 6.0, 30.0] * 2], device="cuda").bfloat16()
    if act == "gelu_erf":
        torch.testing.assert_close(act_forward(code, far).float(), F.gelu(far.float()), rtol=1e-2, atol=1e-3)
    torch.cuda.synchronize()
    _lib.assert_status_ok("activation")


@pytest.mark.parametrize("M,N,pitch", [(1000, 4096, 4096), (777, 30522, 30528), (513, 250, 256), (64, 30, 30)])
def test_colsum_vector_and_ragged(M, N, pitch):
    """Column sums (bias gradients): 16-byte path for full and ragged widths with a padded pitch, scalar
    path otherwise; garbage in the padding columns must not leak into the result."""
    from merak_b200.ops.elementwise import colsum
    torch.manual_seed(0)
    buf = torch.full((M, pitch), float("nan"), device="cuda", dtype=torch.bfloat16)
    buf[:, :N] = torch.randn(M, N, device="cuda").bfloat16()
    x = buf[:, :N]
    out = colsum(x)
    ref = x.float().sum(0)
    torch.testing.assert_close(out, ref, rtol=2e-3, atol=2e-2)
