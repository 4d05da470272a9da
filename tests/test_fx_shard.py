"""Tracing + sharding: composing the shards reproduces the model, for every split method."""
import pytest
import torch
import torch.nn as nn

from merak_b200.fx.shard import shard_model
from merak_b200.fx.split import run_shards
from merak_b200.fx.tracer import trace_model
from merak_b200.models.bert import BertForMaskedLM, bert_config
from merak_b200.models.gpt2 import GPT2LMHeadModel, gpt2_config
from merak_b200.models.llama import LlamaForCausalLM, llama_config


def _models():
    g = GPT2LMHeadModel(gpt2_config("gpt2-tiny", vocab_size=512, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0))
    b = BertForMaskedLM(bert_config("bert-tiny", vocab_size=512, hidden_dropout_prob=0.0))
    l = LlamaForCausalLM(llama_config("llama-tiny"))
    return {"gpt2": (g, ["input_ids"]), "bert": (b, ["input_ids", "attention_mask"]), "llama": (l, ["input_ids"])}


@pytest.mark.parametrize("name", ["gpt2", "bert", "llama"])
@pytest.mark.parametrize("method", ["layer_split", "nearest_min_deps", "farthest_min_deps"])
def test_shards_compose_to_model(name, method):
    torch.manual_seed(0)
    model, input_names = _models()[name]
    model.eval()
    gm = trace_model(model, input_names)
    shards, input_to_shard = shard_model(gm, method, shard_count=4, model_type=model.config.model_type)
    assert len(shards) >= 2
    ids = torch.randint(0, 512, (2, 16))
    inputs = {"input_ids": ids, "attention_mask": torch.ones(2, 16, dtype=torch.long)}
    want = model(**{k: inputs[k] for k in input_names})
    got = run_shards(shards, inputs)
    assert torch.allclose(got, want, atol=1e-5)
    assert set(input_to_shard) == set(input_names)
    # every parameter lives in exactly the shards that use it; together they cover the model
    covered = set()
    for sh in shards:
        covered |= {p.data_ptr() for p in sh.parameters()}
    assert covered == {p.data_ptr() for p in model.parameters()}


class _Skip(nn.Module):
    """A value produced early and used three layers later must be forwarded through the shards."""

    def __init__(self):
        super().__init__()
        self.a, self.b, self.c, self.d = (nn.Linear(8, 8) for _ in range(4))

    def forward(self, x, y):
        h0 = self.a(x)
        h1 = self.b(h0)
        h2 = self.c(h1) + y
        return self.d(h2) + h0


def test_multi_hop_forwarding_and_late_inputs():
    torch.manual_seed(0)
    m = _Skip()
    gm = trace_model(m, ["x", "y"])
    shards, input_to_shard = shard_model(gm, "nearest_min_deps")
    assert len(shards) == 4
    assert input_to_shard["x"] == 0 and input_to_shard["y"] == 2
    # h0 crosses shards 1 and 2 untouched
    assert any("a" in n for n in shards[1].input_names) and any("a" in n for n in shards[2].output_names)
    x, y = torch.randn(3, 8), torch.randn(3, 8)
    assert torch.allclose(run_shards(shards, {"x": x, "y": y}), m(x, y), atol=1e-6)
