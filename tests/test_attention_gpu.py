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
