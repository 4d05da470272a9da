"""Dropout masks of the PyTorch fallback paths: a pure function of (generator seed, step offset + call
number, element index), like the kernels' masks."""
import torch

from merak_b200.ops.attention import dropout_keep_mask
from merak_b200.ops.rng import DropoutState


def test_host_masks_are_counter_based():
    st = DropoutState()
    st.manual_seed(1234, replicated_seed=99)
    a = st.host_keep_mask((64, 128), 0.25, "cpu")
    b = st.host_keep_mask((64, 128), 0.25, "cpu")                 # next call number: another mask
    assert abs(a.float().mean().item() - 0.75) < 0.02
    assert not torch.equal(a, b)
    # consuming a torch generator in between changes nothing; restoring the call number regenerates the mask
    torch.rand(1000)
    st.set_call_id(0)
    assert torch.equal(st.host_keep_mask((64, 128), 0.25, "cpu"), a)
    # the two generators differ, and a step moves both
    st.set_call_id(0)
    sharded = st.host_keep_mask((64, 128), 0.25, "cpu", sharded=True)
    assert not torch.equal(sharded, a)
    st.advance_step()
    assert not torch.equal(st.host_keep_mask((64, 128), 0.25, "cpu"), a)
    # two states with the same replicated seed agree whatever their sharded seeds are (tensor-parallel ranks)
    r0, r1 = DropoutState(), DropoutState()
    r0.manual_seed(5, replicated_seed=77)
    r1.manual_seed(6, replicated_seed=77)
    assert torch.equal(r0.host_keep_mask((32, 32), 0.1, "cpu"), r1.host_keep_mask((32, 32), 0.1, "cpu"))
    assert not torch.equal(r0.host_keep_mask((32, 32), 0.1, "cpu", sharded=True),
                           r1.host_keep_mask((32, 32), 0.1, "cpu", sharded=True))


def test_host_dropout_scales_and_zeroes():
    st = DropoutState()
    st.manual_seed(3)
    x = torch.ones(1000, 16)
    y = st.host_dropout(x, 0.5)
    kept = y != 0
    assert torch.allclose(y[kept], torch.full_like(y[kept], 2.0))
    assert abs(kept.float().mean().item() - 0.5) < 0.03


def test_attention_mask_replica_statistics_and_determinism():
    m1 = dropout_keep_mask(42, 7, 2, 3, 64, 96, 0.1, "cpu")
    m2 = dropout_keep_mask(42, 7, 2, 3, 64, 96, 0.1, "cpu")
    m3 = dropout_keep_mask(42, 8, 2, 3, 64, 96, 0.1, "cpu")
    assert m1.shape == (2, 3, 64, 96) and torch.equal(m1, m2) and not torch.equal(m1, m3)
    assert abs(m1.float().mean().item() - 0.9) < 0.01
    # rows and heads are decorrelated: no two query rows share their mask
    flat = m1.reshape(-1, 96)
    assert len({tuple(r.tolist()) for r in flat}) == flat.shape[0]
