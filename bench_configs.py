"""Throughput of the larger workloads on one 8-GPU node (tokens/s, CUDA-event timed, max over ranks):

    gpt2-1.5b   GPT-2 1.5B (48L d1600 h25), dp2 x tp2 x pp2, seq 1024, global batch 64, micro-batch 4,
                activation recomputation, ZeRO-1
    llama-7b    Llama-2-7B shape, tp4 x pp2 + Megatron sequence parallelism, seq 4096, global batch 32,
                micro-batch 1
    moe         DeepSeek-V2-Lite shape, dp8 with expert parallel 8, seq 4096, micro-batch 1 per GPU

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \\
        bench_configs.py --config llama-7b --steps 3 --warmup 2 [--comm nccl] [--layers N]

Models are built under ``init_empty_weights`` (every rank allocates only its own stage / tensor-parallel
slices, directly on its GPU), data are uniform random token ids, weights random.  Rank 0 prints one
JSON line in the format of ``bench.py``.  ``--layers`` shrinks the depth for a quick run and is
recorded in the output.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

os.environ.setdefault("MERAK_QUIET", "1")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from bench import ClockSampler  # noqa: E402

CONFIGS = {
    "gpt2-1.5b": dict(pp=2, tp=2, dp=2, ep=1, seq=1024, mbs=4, gbs=64, recompute=True, zero=1, sp=False),
    "llama-7b": dict(pp=2, tp=4, dp=1, ep=1, seq=4096, mbs=1, gbs=32, recompute=False, zero=0, sp=True),
    "moe": dict(pp=1, tp=1, dp=8, ep=8, seq=4096, mbs=1, gbs=8, recompute=False, zero=0, sp=False),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=sorted(CONFIGS))
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--gbs", type=int, default=0)
    ap.add_argument("--dp-overlap", type=int, default=1, help="reduce data-parallel gradients while the backward pass runs")
    for k in ("pp", "tp", "dp", "ep"):
        ap.add_argument("--" + k, type=int, default=0, help="override the layout (smaller boxes)")
    o = ap.parse_args()
    c = dict(CONFIGS[o.config])
    if o.gbs:
        c["gbs"] = o.gbs
    for k in ("pp", "tp", "dp", "ep"):
        if getattr(o, k):
            c[k] = getattr(o, k)

    import torch
    import torch.distributed as dist

    import merak_b200 as Merak
    from merak_b200.ops import _lib
    from merak_b200.utils.datasets import SyntheticTokenDataset

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    Merak.init(pp=c["pp"], tp=c["tp"], dp=c["dp"], ep=c["ep"])
    torch.manual_seed(0)
    over = {}
    with Merak.init_empty_weights():
        if o.config == "gpt2-1.5b":
            from merak_b200.models.gpt2 import GPT2LMHeadModel, gpt2_config
            if o.layers:
                over["n_layer"] = o.layers
            cfg = gpt2_config("gpt2-xl", resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0, **over)
            model = GPT2LMHeadModel(cfg)
            name = "GPT-2 1.5B (%dL d%d h%d)" % (cfg.n_layer, cfg.n_embd, cfg.n_head)
        elif o.config == "llama-7b":
            from merak_b200.models.llama import LlamaForCausalLM, llama_config
            if o.layers:
                over["num_hidden_layers"] = o.layers
            cfg = llama_config("llama-7b", max_position_embeddings=c["seq"], **over)
            model = LlamaForCausalLM(cfg)
            name = "Llama-2-7B shape (%dL d%d)" % (cfg.num_hidden_layers, cfg.hidden_size)
        else:
            from merak_b200.models.moe import DeepseekV2ForCausalLM, deepseek_v2_config
            if o.layers:
                over["num_hidden_layers"] = o.layers
            cfg = deepseek_v2_config("deepseek-v2-lite", **over)
            model = DeepseekV2ForCausalLM(cfg)
            name = "DeepSeek-V2-Lite shape (%dL, %d routed experts top-%d)" % (cfg.num_hidden_layers, cfg.n_routed_experts,
                                                                              cfg.num_experts_per_tok)
    gas = max(1, c["gbs"] // (c["mbs"] * c["dp"]))
    args = Merak.MerakArguments(
        output_dir="/tmp/merak_b200_bench_configs", bf16=True, per_device_train_batch_size=c["mbs"],
        gradient_accumulation_steps=gas, max_steps=10 ** 9, learning_rate=1e-4, weight_decay=0.01, max_grad_norm=1.0,
        lr_scheduler_type="constant", logging_steps=0, wall_clock_breakdown=False, report_to="none",
        activation_checkpointing=c["recompute"], zero_stage=c["zero"] or None, megatron_sequence_parallel=c["sp"],
        split_method="layer_split", comm_mode=o.comm, seed=0, overlap_dp_reduce=bool(o.dp_overlap))
    ds = SyntheticTokenDataset(cfg.vocab_size, c["seq"], 1 << 16, task="causal", seed=1)
    trainer = Merak.MerakTrainer(model, args, train_dataset=ds)
    engine = trainer.init_engine()
    data_iter = trainer._batch_iter(trainer.train_dataloader)
    world, rank = dist.get_world_size(), dist.get_rank()

    def sync_all():
        dist.barrier()
        torch.cuda.synchronize()

    for i in range(o.warmup):
        engine.train_batch(data_iter)
        if rank == 0 and os.environ.get("BENCH_PROGRESS") == "1":
            torch.cuda.synchronize()
            print("warm-up step %d done" % i, file=sys.stderr, flush=True)
    sync_all()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loss = None
    for _ in range(o.steps):
        loss = engine.train_batch(data_iter)
    e1.record()
    sync_all()
    clocks = sampler.stop()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    mem = torch.tensor([torch.cuda.max_memory_allocated() / 2 ** 30], dtype=torch.float64, device=device)
    dist.all_reduce(mem, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    tokens = c["mbs"] * gas * c["dp"] * c["seq"] * o.steps
    if rank == 0:
        print(json.dumps({
            "metric": "train tokens/s (device-timed, max over ranks)", "value": tokens / (ms / 1000.0), "unit": "tokens/s",
            "n_gpus": world, "steps": o.steps, "warmup": o.warmup, "ms_per_step": ms / o.steps, "higher_is_better": True,
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights", "impl": "ours",
            "config": {"model": name, "global_batch": c["mbs"] * gas * c["dp"], "seq_len": c["seq"],
                       "micro_batch_per_gpu": c["mbs"], "gradient_accumulation": gas,
                       "parallelism": "pp%d tp%d dp%d ep%d%s" % (c["pp"], c["tp"], c["dp"], c["ep"], " +sp" if c["sp"] else ""),
                       "activation_recompute": c["recompute"], "zero": c["zero"], "comm": o.comm,
                       "layers_override": o.layers or None},
            "clocks": clocks, "gpu_launches": int(_lib.launch_count() - launches0), "final_loss": float(loss),
            "max_memory_allocated_gib": float(mem.item()), "device_status_word": _lib.status()}), flush=True)
    sync_all()
    import merak_b200.initialize as ini
    ini.destroy()


if __name__ == "__main__":
    main()
