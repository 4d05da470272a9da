"""tools/convert_megatron_gpt2_checkpoint.py: a Megatron-LM layout (tp=2, pp=2, checkpoint version 3:
per-head interleaved QKV) synthesised from known full tensors converts back to exactly those tensors
in Hugging Face GPT-2 naming, and the framework's GPT-2 loads the result."""
import importlib.util
import os
import sys
import types

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tool():
    spec = importlib.util.spec_from_file_location("convert_megatron", os.path.join(ROOT, "tools",
                                                                                   "convert_megatron_gpt2_checkpoint.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _megatron_qkv(full, heads, hd, tp, r):
    """[q; k; v] rows ([3*H, ...]) -> Megatron v3 shard of rank r: [heads/tp, 3, hd, ...]."""
    rest = full.shape[1:]
    t = full.view(3, heads, hd, *rest)[:, r * heads // tp:(r + 1) * heads // tp]      # [3, hl, hd]
    return t.transpose(0, 1).contiguous().view(3 * heads // tp * hd, *rest)


def test_megatron_gpt2_roundtrip(tmp_path):
    torch.manual_seed(0)
    L, H, heads, V, P, tp, pp = 4, 32, 4, 64, 16, 2, 2
    hd = H // heads
    ref = {}
    for i in range(L):
        ref[i] = {"ln1.w": torch.randn(H), "ln1.b": torch.randn(H), "qkv.w": torch.randn(3 * H, H),
                  "qkv.b": torch.randn(3 * H), "dense.w": torch.randn(H, H), "dense.b": torch.randn(H),
                  "ln2.w": torch.randn(H), "ln2.b": torch.randn(H), "fc.w": torch.randn(4 * H, H),
                  "fc.b": torch.randn(4 * H), "proj.w": torch.randn(H, 4 * H), "proj.b": torch.randn(H)}
    wte, wpe = torch.randn(V, H), torch.randn(P, H)
    lnf_w, lnf_b = torch.randn(H), torch.randn(H)
    margs = types.SimpleNamespace(padded_vocab_size=V, max_position_embeddings=P, hidden_size=H, num_layers=L,
                                  num_attention_heads=heads, ffn_hidden_size=4 * H)
    for r in range(tp):
        for s in range(pp):
            enc = {}
            for j in range(L // pp):
                w = ref[s * (L // pp) + j]
                pre = "layers.%d." % j
                enc[pre + "input_layernorm.weight"], enc[pre + "input_layernorm.bias"] = w["ln1.w"], w["ln1.b"]
                enc[pre + "self_attention.query_key_value.weight"] = _megatron_qkv(w["qkv.w"], heads, hd, tp, r)
                enc[pre + "self_attention.query_key_value.bias"] = _megatron_qkv(w["qkv.b"], heads, hd, tp, r)
                enc[pre + "self_attention.dense.weight"] = w["dense.w"].chunk(tp, 1)[r].clone()
                enc[pre + "self_attention.dense.bias"] = w["dense.b"]
                enc[pre + "post_attention_layernorm.weight"], enc[pre + "post_attention_layernorm.bias"] = w["ln2.w"], w["ln2.b"]
                enc[pre + "mlp.dense_h_to_4h.weight"] = w["fc.w"].chunk(tp, 0)[r].clone()
                enc[pre + "mlp.dense_h_to_4h.bias"] = w["fc.b"].chunk(tp, 0)[r].clone()
                enc[pre + "mlp.dense_4h_to_h.weight"] = w["proj.w"].chunk(tp, 1)[r].clone()
                enc[pre + "mlp.dense_4h_to_h.bias"] = w["proj.b"]
            if s == pp - 1:
                enc["final_layernorm.weight"], enc["final_layernorm.bias"] = lnf_w, lnf_b
            lm = {"encoder": enc}
            if s == 0:
                lm["embedding"] = {"word_embeddings": {"weight": wte.chunk(tp, 0)[r].clone()},
                                   "position_embeddings": {"weight": wpe}}
            d = tmp_path / "iter_0000010" / ("mp_rank_%02d_%03d" % (r, s))
            d.mkdir(parents=True)
            torch.save({"model": {"language_model": lm}, "checkpoint_version": 3.0, "args": margs, "iteration": 10},
                       str(d / "model_optim_rng.pt"))
    out_dir = tmp_path / "hf"
    tool = _tool()
    assert tool.main(["--path_to_checkpoint", str(tmp_path / "iter_0000010"), "--path_to_output_checkpoint",
                      str(out_dir), "--tp", "2", "--pp", "2", "--dp", "1"]) == 0
    from safetensors.torch import load_file
    got = load_file(str(out_dir / "model.safetensors"))
    assert torch.equal(got["transformer.wte.weight"], wte) and torch.equal(got["transformer.wpe.weight"], wpe)
    for i in range(L):
        w = ref[i]
        pre = "transformer.h.%d." % i
        assert torch.equal(got[pre + "attn.c_attn.weight"], w["qkv.w"].t())
        assert torch.equal(got[pre + "attn.c_attn.bias"], w["qkv.b"])
        assert torch.equal(got[pre + "attn.c_proj.weight"], w["dense.w"].t())
        assert torch.equal(got[pre + "mlp.c_fc.weight"], w["fc.w"].t())
        assert torch.equal(got[pre + "mlp.c_proj.weight"], w["proj.w"].t())
        assert torch.equal(got[pre + "ln_2.bias"], w["ln2.b"])
    assert torch.equal(got["transformer.ln_f.weight"], lnf_w)

    # the framework's GPT-2 reads the directory as a release checkpoint
    sys.path.insert(0, ROOT)
    import merak_b200 as Merak
    from merak_b200.checkpoint.checkpoint import CheckpointLoader
    from merak_b200.models.gpt2 import GPT2LMHeadModel, gpt2_config
    model = GPT2LMHeadModel(gpt2_config("gpt2-tiny", vocab_size=V, n_positions=P, n_embd=H, n_layer=L, n_head=heads))
    args = Merak.MerakArguments(output_dir=str(tmp_path / "o"), resume_from_checkpoint=str(out_dir))
    CheckpointLoader(args).load_checkpoint(model, path=str(out_dir))
    sd = model.state_dict()
    assert torch.equal(sd["transformer.h.2.attn.c_attn.weight"], ref[2]["qkv.w"])
    assert torch.equal(sd["transformer.h.3.mlp.c_proj.weight"], ref[3]["proj.w"])
    assert torch.equal(sd["transformer.wte.weight"], wte)
