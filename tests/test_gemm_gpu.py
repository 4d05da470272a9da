"""tcgen05 GEMM against an fp32 PyTorch evaluation of the same formula."""
import pytest
import torch

from merak_b200.ops import _lib, gemm as G

pytestmark = pytest.mark.gpu


def _rand(shape, scale=1.0):
    return (torch.randn(shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _check(out, ref, K, what):
    tol = 2e-2 * (K ** 0.5) * 0.05 + 2e-2
    err = (out.float() - ref.float()).abs().max().item()
    rel = err / (ref.float().abs().max().item() + 1e-6)
    assert rel < 2e-2 or err < tol, "%s: max abs err %g rel %g" % (what, err, rel)


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (384, 768, 320), (1024, 1024, 1024),
                                   (200, 264, 72), (77, 40, 24), (4096, 3072, 1024)])
@pytest.mark.parametrize("block_n", [0, 128, 256, 512])
def test_gemm_layouts(shape, a_mn, b_mn, block_n):
    M, N, K = shape
    torch.manual_seed(0)
    a = _rand((K, M) if a_mn else (M, K))
    b = _rand((K, N) if b_mn else (N, K))
    out, _ = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=block_n)
    torch.cuda.synchronize()
    _lib.assert_status_ok("gemm")
    ref, _ = G._reference(a.cpu(), b.cpu(), a_mn, b_mn, None, 0, None, 0, 1.0, None, False, torch.float32, False)
    _check(out.cpu(), ref, K, "gemm %s a_mn=%s b_mn=%s" % (shape, a_mn, b_mn))


@pytest.mark.parametrize("act", [G.ACT_NONE, G.ACT_GELU_ERF, G.ACT_GELU_TANH, G.ACT_RELU, G.ACT_SILU])
@pytest.mark.parametrize("bias_dtype", [None, torch.bfloat16, torch.float32])
def test_gemm_bias_act_preact(act, bias_dtype):
    M, N, K = 512, 640, 256
    torch.manual_seed(1)
    a, b = _rand((M, K)), _rand((N, K), 0.05)
    bias = None if bias_dtype is None else torch.randn(N, device="cuda").to(bias_dtype)
    out, pre = G.gemm(a, b, bias=bias, act=act, want_preact=True)
    torch.cuda.synchronize()
    _lib.assert_status_ok("gemm")
    ref, rpre = G._reference(a.cpu(), b.cpu(), False, False, None if bias is None else bias.cpu(), act, None, 0,
                             1.0, None, False, torch.float32, True)
    _check(out.cpu(), ref, K, "act")
    _check(pre.cpu(), rpre, K, "preact")


@pytest.mark.parametrize("aux_mode", [G.AUX_ADD, G.AUX_DACT])
@pytest.mark.parametrize("N", [512, 520, 100])
def test_gemm_aux(aux_mode, N):
    M, K = 300, 192
    torch.manual_seed(2)
    a, b = _rand((M, K)), _rand((N, K), 0.05)
    aux = _rand((M, N))
    out, _ = G.gemm(a, b, act=G.ACT_GELU_ERF, aux_in=aux, aux_mode=aux_mode)
    torch.cuda.synchronize()
    _lib.assert_status_ok("gemm")
    ref, _ = G._reference(a.cpu(), b.cpu(), False, False, None, G.ACT_GELU_ERF, aux.cpu(), aux_mode, 1.0, None,
                          False, torch.float32, False)
    _check(out.cpu(), ref, K, "aux")


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_accumulate(out_dtype):
    M, N, K = 256, 384, 512
    torch.manual_seed(3)
    a, b = _rand((K, M)), _rand((K, N), 0.05)
    out = torch.randn(M, N, device="cuda").to(out_dtype)
    base = out.clone()
    G.gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True, alpha=0.5)
    torch.cuda.synchronize()
    _lib.assert_status_ok("gemm")
    ref = base.float().cpu() + 0.5 * (a.float().cpu().t() @ b.float().cpu())
    _check(out.cpu(), ref, K, "accumulate")


@pytest.mark.parametrize("shape", [(1024, 1024, 16384), (1024, 4096, 16384), (3072, 1024, 8192), (256, 256, 4096)])
def test_gemm_split_k_wgrad(shape):
    """Small fp32-accumulate outputs with a long contraction take the split-K path."""
    M, N, K = shape
    torch.manual_seed(4)
    a, b = _rand((K, M), 0.1), _rand((K, N), 0.1)
    out = torch.randn(M, N, device="cuda")
    base = out.clone()
    G.gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True)
    torch.cuda.synchronize()
    _lib.assert_status_ok("gemm")
    ref = base + a.float().t() @ b.float()
    _check(out, ref, K, "split-k")


def test_linear_and_mlp_fork_sum_input_gradients_in_the_gemm():
    """``linear_fork`` / ``mlp_fork`` hand the input through as a second output; the two gradients of
    the input are added in the data-gradient GEMM's epilogue."""
    from merak_b200.ops import gemm as G
    from merak_b200.ops.linear import linear, linear_fork, mlp, mlp_fork
    torch.manual_seed(0)
    dev = torch.device("cuda")
    M, K, N, F = 384, 256, 320, 512
    x = (torch.randn(3, M // 3, K, device=dev) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=dev) * 0.05).bfloat16().requires_grad_(True)
    b = torch.randn(N, device=dev).bfloat16().requires_grad_(True)
    gy = torch.randn(3, M // 3, N, device=dev).bfloat16()
    gx = torch.randn(3, M // 3, K, device=dev).bfloat16()
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    y, xr = linear_fork(xa, w, b)
    ((y.float() * gy.float()).sum() + (xr.float() * gx.float()).sum()).backward()
    dw_fork, w.grad = w.grad.clone(), None
    y2 = linear(xb, w, b)
    ((y2.float() * gy.float()).sum() + (xb.float() * gx.float()).sum()).backward()
    torch.testing.assert_close(y.float(), y2.float(), rtol=0, atol=0)
    torch.testing.assert_close(xa.grad.float(), xb.grad.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dw_fork.float(), w.grad.float(), rtol=0, atol=0)
    # only the pass-through output used
    xc = x.clone().requires_grad_(True)
    _, xr = linear_fork(xc, w, b)
    (xr.float() * gx.float()).sum().backward()
    torch.testing.assert_close(xc.grad.float(), gx.float(), rtol=0, atol=0)
    # MLP
    w1 = (torch.randn(F, K, device=dev) * 0.05).bfloat16().requires_grad_(True)
    b1 = torch.zeros(F, device=dev).bfloat16().requires_grad_(True)
    w2 = (torch.randn(K, F, device=dev) * 0.05).bfloat16().requires_grad_(True)
    b2 = torch.zeros(K, device=dev).bfloat16().requires_grad_(True)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    y, xr = mlp_fork(xa, w1, b1, w2, b2, G.ACT_GELU_ERF)
    ((y.float() * gx.float()).sum() + (xr.float() * gx.float()).sum()).backward()
    y2 = mlp(xb, w1, b1, w2, b2, G.ACT_GELU_ERF)
    ((y2.float() * gx.float()).sum() + (xb.float() * gx.float()).sum()).backward()
    torch.testing.assert_close(xa.grad.float(), xb.grad.float(), rtol=2e-2, atol=2e-2)
