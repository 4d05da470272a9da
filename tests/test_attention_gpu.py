"""tcgen05 flash attention forward/backward against fp32 PyTorch autograd."""
import math

import pytest
import torch

from merak_b200.ops import _lib
from merak_b200.ops.attention import attention_reference, flash_attention

pytestmark = pytest.mark.gpu

CASES = [
    # B, H, Hkv, Lq, Lk, D, causal, bias
    (1, 1, 1, 128, 128, 64, False, False),
    (2, 4, 4, 512, 512, 64, False, False),
    (2, 4, 4, 512, 512, 64, True, False),
    (2, 4, 2, 384, 384, 128, True, False),
    (1, 3, 3, 200, 333, 64, False, False),
    (1, 3, 3, 333, 333, 64, True, False),
    (1, 2, 2, 300, 300, 128, False, False),
    (2, 2, 2, 256, 256, 128, False, True),
    (2, 2, 2, 256, 256, 64, False, True),
    (1, 8, 2, 256, 256, 64, True, False),
]


@pytest.mark.parametrize("case", CASES)
def test_attention_fwd_bwd(case):
    B, H, Hkv, Lq, Lk, D, causal, bias = case
    torch.manual_seed(0)
    q = torch.randn(B, Lq, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, Lk, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, Lk, Hkv, D, device="cuda").bfloat16().requires_grad_()
    kb = None
    if bias:
        kb = torch.zeros(B, Lk, device="cuda")
        kb[:, Lk - Lk // 3:] = -30000.0
    out = flash_attention(q, k, v, key_bias=kb, causal=causal)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.assert_status_ok("attention")
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, kb, causal, 1.0 / math.sqrt(D))
    ref.backward(dout.float())
    def close(a, b, what, tol):
        err = (a.float() - b.float()).abs().max().item()
        scale = b.float().abs().max().item() + 1e-6
        assert err / scale < tol, "%s: err %g (scale %g)" % (what, err, scale)
    close(out, ref, "out", 2e-2)
    close(q.grad, qr.grad, "dq", 3e-2)
    close(k.grad, kr.grad, "dk", 3e-2)
    close(v.grad, vr.grad, "dv", 3e-2)


def test_attention_strided_qkv():
    """Q, K, V as views of one fused projection output [B, L, 3, H, D]."""
    B, L, H, D = 2, 256, 4, 64
    torch.manual_seed(1)
    qkv = torch.randn(B, L, 3, H, D, device="cuda").bfloat16()
    q, k, v = qkv.unbind(2)
    out = flash_attention(q, k, v, causal=True)
    ref = attention_reference(q, k, v, None, True, None)
    torch.cuda.synchronize()
    _lib.assert_status_ok("attention")
    assert (out.float() - ref.float()).abs().max().item() < 3e-2


@pytest.mark.parametrize("hq,hkv,D,causal", [(4, 4, 64, False), (8, 2, 64, True), (4, 4, 128, True)])
def test_attention_packed(hq, hkv, D, causal):
    from merak_b200.ops.attention import flash_attention_packed
    B, L = 2, 256
    torch.manual_seed(2)
    qkv = torch.randn(B, L, hq + 2 * hkv, D, device="cuda").bfloat16().requires_grad_()
    out = flash_attention_packed(qkv, hq, hkv, causal=causal)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.assert_status_ok("attention")
    r = qkv.detach().float().requires_grad_()
    ref = attention_reference(r[:, :, :hq], r[:, :, hq:hq + hkv], r[:, :, hq + hkv:], None, causal, None)
    ref.backward(dout.float())
    assert (out.float() - ref).abs().max().item() < 3e-2
    err = (qkv.grad.float() - r.grad).abs().max().item() / (r.grad.abs().max().item() + 1e-6)
    assert err < 3e-2, err


@pytest.mark.parametrize("case", [
    # B, H, Hkv, Lq, Lk, D, causal, bias, p
    (2, 4, 4, 512, 512, 64, False, False, 0.1),
    (1, 3, 3, 200, 333, 64, False, True, 0.25),
    (2, 4, 2, 384, 384, 128, True, False, 0.1),
    (1, 8, 2, 256, 256, 64, True, False, 0.5),
])
def test_attention_probability_dropout_against_the_same_mask(case):
    """Dropout on the probabilities inside the kernels: forward and backward regenerate the mask from
    a stateless hash; the fp32 reference applies the identical mask (evaluated on the host side with
    int64 tensors) between softmax and the value product."""
    from merak_b200.ops.attention import dropout_keep_mask
    from merak_b200.ops.rng import dropout_state
    B, H, Hkv, Lq, Lk, D, causal, bias, p = case
    torch.manual_seed(3)
    st = dropout_state()
    st.manual_seed(987654321012345)
    q = torch.randn(B, Lq, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, Lk, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, Lk, Hkv, D, device="cuda").bfloat16().requires_grad_()
    kb = None
    if bias:
        kb = torch.zeros(B, Lk, device="cuda")
        kb[:, Lk - Lk // 3:] = -30000.0
    out = flash_attention(q, k, v, key_bias=kb, causal=causal, dropout_p=p)
    seed, offset = (int(x) for x in st.tensor(q.device, sharded=True).tolist())
    call_id = st.get_call_id()
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.assert_status_ok("attention dropout")
    keep = dropout_keep_mask(seed, offset + call_id, B, H, Lq, Lk, p, q.device)
    assert abs(keep.float().mean().item() - (1.0 - p)) < 0.01
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    qf, kf, vf = (t.permute(0, 2, 1, 3) for t in (qr, kr, vr))
    if Hkv != H:
        kf = kf.repeat_interleave(H // Hkv, dim=1)
        vf = vf.repeat_interleave(H // Hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) / math.sqrt(D)
    if kb is not None:
        s = s + kb[:, None, None, :]
    if causal:
        s = s.masked_fill(~torch.ones(Lq, Lk, dtype=torch.bool, device="cuda").tril(Lk - Lq), float("-inf"))
    prob = torch.softmax(s, dim=-1) * keep.float() / (1.0 - p)
    ref = torch.matmul(prob, vf).permute(0, 2, 1, 3)
    ref.backward(dout.float())

    def close(a, b, what, tol):
        err = (a.float() - b.float()).abs().max().item()
        scale = b.float().abs().max().item() + 1e-6
        assert err / scale < tol, "%s: err %g (scale %g)" % (what, err, scale)
    close(out, ref, "out", 2e-2)
    close(q.grad, qr.grad, "dq", 3e-2)
    close(k.grad, kr.grad, "dk", 3e-2)
    close(v.grad, vr.grad, "dv", 3e-2)
    # another call draws another mask; p = 0 is the plain kernel
    out2 = flash_attention(q, k, v, key_bias=kb, causal=causal, dropout_p=p)
    assert not torch.equal(out2, out)
