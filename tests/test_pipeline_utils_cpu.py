"""Output pseudo-deallocation + direct autograd-engine backward, the uneven channel split, the
channel-parallel conv wrapper (single rank) and the norm-clipping helper."""
import torch
import torch.nn as nn

from merak_b200.parallel.utils import channels_uniform
from merak_b200.pipeline.utils import clip_grad_norm_, custom_backward, deallocate_output_tensor


def test_deallocate_then_custom_backward_matches_plain_backward():
    torch.manual_seed(0)
    w = torch.randn(8, 8, requires_grad=True)
    x = torch.randn(4, 8)
    y = (x @ w).relu()
    g = torch.randn_like(y)
    (gw_ref,) = torch.autograd.grad(y, w, g, retain_graph=True)
    deallocate_output_tensor(y)
    assert y.numel() == 1 and y.grad_fn is not None
    custom_backward(y, g)
    torch.testing.assert_close(w.grad, gw_ref)


def test_channels_uniform():
    assert channels_uniform(10, 4) == [0, 3, 6, 8, 10]
    assert channels_uniform(8, 2) == [0, 4, 8]


def test_clip_grad_norm_single_rank():
    p = nn.Parameter(torch.ones(4))
    p.grad = torch.full((4,), 3.0)
    norm = clip_grad_norm_([p], max_norm=1.0)
    assert abs(norm - 6.0) < 1e-5
    assert abs(p.grad.norm().item() - 1.0) < 1e-4


def test_conv_para_single_rank_is_the_plain_conv():
    from merak_b200.parallel.tp_transform import ConvPara
    torch.manual_seed(1)
    conv = nn.Conv2d(4, 6, 3, padding=1)
    x = torch.randn(2, 4, 5, 5)
    torch.testing.assert_close(ConvPara(conv)(x), conv(x))
