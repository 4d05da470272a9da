"""FlopsProfiler totals against analytic counts, and the AutoPipe partition driven by it
(Merak/core/pipeline/profiler.py:21-960, Merak/core/pipeline/layers_partition.py:102-139)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from merak_b200.models.gpt2 import GPT2LMHeadModel, gpt2_config
from merak_b200.pipeline.profiler import FlopsProfiler, profile_layer_costs


def test_gpt2_tiny_total_matches_the_analytic_count():
    cfg = gpt2_config("gpt2-tiny", vocab_size=512)
    model = GPT2LMHeadModel(cfg).eval()
    B, L, H, V, nl, nh = 2, 32, cfg.n_embd, cfg.vocab_size, cfg.n_layer, cfg.n_head
    T = B * L
    prof = FlopsProfiler(model)
    prof.start_profile()
    with torch.no_grad():
        model(torch.randint(0, V, (B, L)))
    prof.end_profile()
    gemm = nl * (2 * T * H * 3 * H + 2 * T * H * H + 2 * 2 * T * H * 4 * H) + 2 * T * H * V
    attn = nl * B * nh * (2 * 2 * L * L * (H // nh))
    total = prof.get_total_flops()
    # matmuls dominate; norms, GELU, softmax and residual adds come on top (a few per cent)
    assert gemm + attn <= total <= 1.10 * (gemm + attn), (total, gemm + attn)
    # attribution: the head's share is its GEMM, a block's share is a quarter of the blocks' total
    assert prof.module_flops(model.lm_head) == 2 * T * H * V
    per_block = [prof.module_flops(b) for b in model.transformer.h]
    assert max(per_block) == min(per_block) > 0
    assert prof.get_total_macs() == total // 2
    assert prof.get_total_params() == sum(p.numel() for p in model.parameters())


class _Mixed(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(3, 8, 3, padding=1)
        self.bn = nn.BatchNorm2d(8)
        self.fc = nn.Linear(8, 5)

    def forward(self, x):
        y = F.relu(self.bn(self.conv(x)))
        y = F.interpolate(y, scale_factor=2, mode="bilinear", align_corners=False)
        y = F.max_pool2d(y, 2)
        y = y.mean(dim=(2, 3))
        a = torch.bmm(y.unsqueeze(1), y.unsqueeze(2)).squeeze()          # tensor-method / functional calls
        return F.softmax(self.fc(y), dim=-1) * a[:, None]


def test_functional_and_tensor_method_calls_are_counted():
    m = _Mixed().eval()
    x = torch.randn(2, 3, 16, 16)
    prof = FlopsProfiler(m)
    prof.start_profile()
    with torch.no_grad():
        m(x)
    prof.end_profile()
    conv = 2 * (2 * 8 * 16 * 16) * (3 * 3 * 3) + 2 * 8 * 16 * 16          # multiply-adds + bias
    assert prof.module_flops(m.conv) == conv
    assert prof.module_flops(m.fc) == 2 * 2 * 8 * 5 + 2 * 5
    total = prof.get_total_flops()
    # interpolate (8 per output element), pooling (4), bmm, softmax, mean, relu, batch norm all add up
    extra = total - conv - prof.module_flops(m.fc) - prof.module_flops(m.bn)
    assert extra >= 8 * 2 * 8 * 32 * 32 + 4 * 2 * 8 * 16 * 16 + 2 * 2 * 8
    assert prof.module_flops(m.bn) == 5 * 2 * 8 * 16 * 16


def test_layer_costs_feed_autopipe():
    from merak_b200.pipeline.partition import partition_layers
    layers = [nn.Linear(64, 64) for _ in range(6)] + [nn.Linear(64, 1024), nn.Linear(1024, 64)]
    x = torch.randn(4, 64)

    def run_all():
        y = x
        for l in layers:
            y = l(y)

    fwd = profile_layer_costs(layers, run_all, unit=1000)
    assert fwd[6] > 10 * fwd[0] and fwd[7] > 10 * fwd[0]
    parts = partition_layers("autopipe", len(layers), 2, fwd_costs=fwd, bwd_costs=[3 * f for f in fwd])
    assert parts[0] == 0 and parts[-1] == len(layers) and 0 < parts[1] < len(layers)
    # the two wide layers outweigh the six narrow ones: the cut falls at or after the sixth layer
    assert parts[1] >= 6
