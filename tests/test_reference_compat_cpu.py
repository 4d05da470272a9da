"""Pieces that let scripts written for the reference run unchanged: values that are not tensors crossing a
pipeline boundary, in-place operations on shard inputs, the generated dataset's layouts for nested
configurations, depth lookup for unusual configurations, and the tracing-time handling of configurations
written for older ``transformers`` (``return_dict=False``)."""
import torch
import torch.fx as fx
import torch.nn as nn

import pytest


def test_scalars_and_devices_travel_as_tagged_tensors():
    from merak_b200.parallel import p2p
    values = [torch.randn(2, 3), 7, 0.25, True, torch.device("cpu"), torch.arange(4)]
    tensors, kinds = p2p.to_wire(values, "cpu")
    assert kinds == [0, p2p.KIND_INT, p2p.KIND_FLOAT, p2p.KIND_BOOL, p2p.KIND_DEVICE, 0]
    assert all(isinstance(t, torch.Tensor) for t in tensors)
    meta = p2p.decode_meta(p2p.encode_meta(tensors, kinds))
    assert [m[1] for m in meta] == [1, p2p.KIND_INT, p2p.KIND_FLOAT, p2p.KIND_BOOL, p2p.KIND_DEVICE, 0]
    assert meta[0][2] == (2, 3) and meta[1][2] == ()
    back = p2p.from_wire(tensors, meta, "cpu")
    assert back[1] == 7 and isinstance(back[1], int) and back[2] == 0.25 and back[3] is True
    assert back[4] == torch.device("cpu") and torch.equal(back[5], values[5]) and back[0] is values[0]
    with pytest.raises(TypeError):
        p2p.to_wire(["text"], "cpu")


def test_inplace_on_a_shard_input_runs_out_of_place():
    """A cut right before ``nn.ReLU(inplace=True)`` (torchvision / Hugging Face ResNets): the next shard's input
    is a leaf that requires grad, on which the in-place form is an autograd error."""
    from merak_b200.fx.split import split_graph

    class Net(nn.Module):
        def __init__(self, method: bool):
            super().__init__()
            self.a, self.relu, self.b, self.method = nn.Linear(4, 4), nn.ReLU(inplace=True), nn.Linear(4, 2), method

        def forward(self, x):
            h = self.a(x)
            h = h.add_(1.0) if self.method else self.relu(h)
            return self.b(h)

    for method in (False, True):           # nn.ReLU(inplace=True) as a module call; Tensor.add_ as a method call
        torch.manual_seed(0)
        net = Net(method)
        gm = fx.symbolic_trace(net)
        nodes = [n for n in gm.graph.nodes if n.op not in ("placeholder", "output")]
        assignment = {n: (0 if n.target == "a" else 1) for n in nodes}
        shards, _ = split_graph(gm, assignment, 2)
        x = torch.randn(3, 4)
        want = net(x.clone())
        mid = shards[0](x)
        mid = mid[0] if isinstance(mid, tuple) else mid
        leaf = mid.detach().requires_grad_(True)
        before = leaf.detach().clone()
        out = shards[1](leaf)
        out = out[0] if isinstance(out, tuple) else out
        out.sum().backward()                                   # no "leaf Variable ... in-place" error
        assert torch.allclose(out, want, atol=1e-6) and leaf.grad is not None
        assert torch.equal(leaf.detach(), before)               # the received activation itself is left alone
        assert net.relu.inplace is True                         # the model's own module is untouched


def test_generated_dataset_layouts():
    import transformers as T
    from merak_b200.utils.datasets import DynamicGenDataset
    clip = T.CLIPConfig()
    ds = DynamicGenDataset(clip, mode="multimodal", dataset_size=1e6)       # the reference scripts pass a float
    s = ds[0]
    assert len(ds) == 1000000 and s["input_ids"].shape == (clip.text_config.max_position_embeddings,)
    assert s["pixel_values"].shape == (3, clip.vision_config.image_size, clip.vision_config.image_size)
    s2t = T.Speech2TextConfig()
    s = DynamicGenDataset(s2t, mode="speech2text", dataset_size=4, seq_length=40)[1]
    assert s["input_features"].shape == (40, s2t.input_feat_per_channel) and s["decoder_input_ids"].shape == (40,)
    lx = T.LxmertConfig()
    s = DynamicGenDataset(lx, mode="for_qa", dataset_size=4, seq_length=12)[0]
    assert s["visual_feats"].shape == (12, lx.visual_feat_dim) and s["visual_pos"].shape == (12, lx.visual_pos_dim)
    bert = T.BertConfig()
    s = DynamicGenDataset(bert, mode="for_qa", dataset_size=4, seq_length=12)[0]
    assert set(s) == {"input_ids", "start_positions", "end_positions"}


def test_depth_lookup_for_unusual_configs():
    import transformers as T
    from merak_b200.args import MerakArguments, mergeargs
    lx = T.LxmertConfig()
    a = mergeargs(MerakArguments(no_cuda=True), lx)
    assert a.num_layers == lx.l_layers + lx.x_layers + lx.r_layers and a.shard_count == 2 * a.num_layers + 4
    b = mergeargs(MerakArguments(no_cuda=True), T.BertConfig(num_hidden_layers=5))
    assert b.num_layers == 5

    class Odd:           # nothing that states a depth: left to the trainer's fallback, not an error
        hidden_size = 8
    assert mergeargs(MerakArguments(no_cuda=True), Odd()).num_layers is None


def test_export_with_return_dict_false_config_and_lifted_constants():
    """Configurations of the reference's examples say ``return_dict=False``; in transformers 5.x the inner model
    then returns a tuple that the head cannot read.  The export path traces with dictionaries inside and a tuple
    outside, restores the configuration, and leaves no in-place detach of a lifted constant in the graph."""
    import transformers as T
    from merak_b200.fx.export_trace import export_flat
    cfg = T.T5Config(d_model=32, d_kv=8, num_heads=4, d_ff=64, num_layers=1, vocab_size=128, use_cache=False,
                     return_dict=False, dropout_rate=0.0)
    model = T.T5ForConditionalGeneration(cfg)
    ids = torch.randint(1, 100, (2, 8))
    gm = export_flat(model, {"input_ids": ids, "decoder_input_ids": ids.clone()})
    assert cfg.return_dict is False
    assert not any(n.op == "call_function" and n.target is torch.ops.aten.detach_.default for n in gm.graph.nodes)
    out = gm(ids, ids.clone())
    assert out[0].shape == (2, 8, 128)
