"""Reference arm of the benchmark: the unmodified reference package (installed under
``baseline/_ref``) trains a plain-PyTorch BERT-large through its own public API.

The path taken is the reference's stock one: ``Merak.init(pp, tp, dp)``
(Merak/initialize.py:36-85), ``MerakArguments`` (Merak/merak_args/args.py:37), ``MerakTrainer``
(Merak/merak_trainer.py:49-146) which traces the model with ``torch.fx``
(Merak/core/fx/convert.py:72-85), shards the graph, wraps it in its ``PipelineModule``, then
``trainer.init_engine()`` and ``engine.train_batch`` (Merak/core/merak_engine.py:1192-1269) with
the bucketed NCCL gradient all-reduce (``:552-621``) and ``torch.optim.AdamW``
(Merak/merak_trainer.py:225-257).  Nothing of this repository's framework, models or kernels is
imported here: the model below is ``nn.Linear`` / ``nn.LayerNorm`` / ``nn.Embedding`` /
``F.scaled_dot_product_attention`` only.

The model, data, precision, optimizer and timing protocol are the ones of the repository's own
arm: BERT-large masked LM (24 layers, hidden 1024, 16 heads, feed-forward 4096, vocabulary 30522,
tied decoder), sequence 512, micro-batch 32 per GPU, bf16, hidden dropout 0.1, attention dropout 0,
AdamW lr 1e-4 weight decay 0.01, gradient clipping 1.0, constant learning rate.
"""
from __future__ import annotations

import json
import math
import os
import sys
import tempfile
import types

import torch
import torch.nn as nn
import torch.nn.functional as F


# ----------------------------------------------------------------------------------------------
# plain-PyTorch BERT (masked LM)
# ----------------------------------------------------------------------------------------------
class PlainBertLayer(nn.Module):
    def __init__(self, hidden, heads, ff, p_drop, eps):
        super().__init__()
        self.heads, self.head_dim = heads, hidden // heads
        self.query = nn.Linear(hidden, hidden)
        self.key = nn.Linear(hidden, hidden)
        self.value = nn.Linear(hidden, hidden)
        self.attn_out = nn.Linear(hidden, hidden)
        self.attn_norm = nn.LayerNorm(hidden, eps=eps)
        self.fc1 = nn.Linear(hidden, ff)
        self.fc2 = nn.Linear(ff, hidden)
        self.out_norm = nn.LayerNorm(hidden, eps=eps)
        self.drop = nn.Dropout(p_drop)

    def forward(self, x, bias):
        b, l = x.size(0), x.size(1)
        q = self.query(x).view(b, l, self.heads, self.head_dim).transpose(1, 2)
        k = self.key(x).view(b, l, self.heads, self.head_dim).transpose(1, 2)
        v = self.value(x).view(b, l, self.heads, self.head_dim).transpose(1, 2)
        ctx = F.scaled_dot_product_attention(q, k, v, attn_mask=bias)
        ctx = ctx.transpose(1, 2).reshape(b, l, self.heads * self.head_dim)
        x = self.attn_norm(x + self.drop(self.attn_out(ctx)))
        return self.out_norm(x + self.drop(self.fc2(F.gelu(self.fc1(x)))))


class PlainBertForMaskedLM(nn.Module):
    def __init__(self, vocab=30522, hidden=1024, layers=24, heads=16, ff=4096, max_pos=512,
                 p_drop=0.1, eps=1e-12, std=0.02, seq=512):
        super().__init__()
        # read by the reference's ``mergeargs`` (Merak/merak_args/args.py:598-657)
        self.config = types.SimpleNamespace(num_hidden_layers=layers, hidden_size=hidden,
                                            num_attention_heads=heads, max_position_embeddings=max_pos,
                                            tie_word_embeddings=True, vocab_size=vocab)
        self.std = std
        self.word_embeddings = nn.Embedding(vocab, hidden)
        self.position_embeddings = nn.Embedding(max_pos, hidden)
        self.token_type_embeddings = nn.Embedding(2, hidden)
        self.emb_norm = nn.LayerNorm(hidden, eps=eps)
        self.drop = nn.Dropout(p_drop)
        # plain torch.fx cannot slice a buffer by a traced length: positions are fixed to ``seq``
        self.register_buffer("position_ids", torch.arange(seq).unsqueeze(0), persistent=False)
        self.layer = nn.ModuleList([PlainBertLayer(hidden, heads, ff, p_drop, eps) for _ in range(layers)])
        self.head_dense = nn.Linear(hidden, hidden)
        self.head_norm = nn.LayerNorm(hidden, eps=eps)
        self.decoder = nn.Linear(hidden, vocab)
        self.apply(self._init_weights)
        self.decoder.weight = self.word_embeddings.weight

    def _init_weights(self, m):
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, mean=0.0, std=self.std)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=self.std)
        elif isinstance(m, nn.LayerNorm):
            nn.init.ones_(m.weight)
            nn.init.zeros_(m.bias)

    def forward(self, input_ids, attention_mask):
        x = self.word_embeddings(input_ids) + self.position_embeddings(self.position_ids) \
            + self.token_type_embeddings(torch.zeros_like(input_ids))
        x = self.drop(self.emb_norm(x))
        # additive key-padding bias, as Hugging Face's BERT builds it for its SDPA path
        bias = (1.0 - attention_mask[:, None, None, :].to(x.dtype)) * -30000.0
        for blk in self.layer:
            x = blk(x, bias)
        x = self.head_norm(F.gelu(self.head_dense(x)))
        return self.decoder(x)


# ----------------------------------------------------------------------------------------------
# synthetic masked-LM data (uniform token ids, 15 % masked with the 80/10/10 rule)
# ----------------------------------------------------------------------------------------------
class MlmDataset(torch.utils.data.Dataset):
    def __init__(self, vocab, seq, size, seed=0, mask_id=103, p=0.15):
        self.vocab, self.seq, self.size, self.seed, self.mask_id, self.p = vocab, seq, size, seed, mask_id, p

    def __len__(self):
        return self.size

    def __getitem__(self, idx):
        g = torch.Generator()
        g.manual_seed(self.seed * 1000003 + idx)
        ids = torch.randint(0, self.vocab, (self.seq,), generator=g)
        labels = ids.clone()
        masked = torch.rand(self.seq, generator=g) < self.p
        labels[~masked] = -100
        roll = torch.rand(self.seq, generator=g)
        inp = ids.clone()
        inp[masked & (roll < 0.8)] = self.mask_id
        rnd = masked & (roll >= 0.8) & (roll < 0.9)
        inp[rnd] = torch.randint(0, self.vocab, (int(rnd.sum()),), generator=g)
        return {"input_ids": inp, "attention_mask": torch.ones(self.seq, dtype=torch.long), "labels": labels}


def _batches(ds, mbs, n, device, pinned):
    out = []
    for b in range(n):
        items = [ds[b * mbs + i] for i in range(mbs)]
        batch = {k: torch.stack([it[k] for it in items]) for k in items[0]}
        if pinned:
            batch = {k: (v.pin_memory() if torch.cuda.is_available() else v) for k, v in batch.items()}
        else:
            batch = {k: v.to(device) for k, v in batch.items()}
        out.append(batch)
    return out


class _Cycle:
    """An endless iterable of fresh dict copies (the reference's ``prepare_data`` pops the keys
    of the batch it is given, Merak/merak_trainer.py:329-353)."""

    def __init__(self, batches):
        self.batches = batches

    def __iter__(self):
        i = 0
        while True:
            yield dict(self.batches[i % len(self.batches)])
            i += 1


def run(o, ref_dir: str, clock_sampler_cls, metric: str, small: dict | None = None) -> None:
    """Train and time; rank 0 prints the JSON line.  ``small`` overrides the model shape (used by
    the CPU test of this runner)."""
    import torch.distributed as dist

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    sys.path.insert(0, ref_dir)
    import compat
    compat.install()

    cuda = torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("LOCAL_RANK", str(local))
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    if cuda:
        torch.cuda.set_device(local)
    elif not dist.is_initialized():
        # no GPU (the CPU test of this runner): the reference would insist on NCCL
        # (Merak/initialize.py:48-56); it keeps a process group that already exists.
        dist.init_process_group("gloo")
    device = torch.device("cuda", local) if cuda else torch.device("cpu")

    import Merak
    assert os.path.abspath(Merak.__file__).startswith(os.path.abspath(ref_dir)), Merak.__file__
    from Merak import MerakArguments, MerakTrainer

    world = int(os.environ["WORLD_SIZE"])
    Merak.init(1, 1, world)                      # (pp, tp, dp)
    rank = dist.get_rank()

    shape = dict(vocab=30522, hidden=1024, layers=24, heads=16, ff=4096, max_pos=max(512, o.seq), p_drop=o.dropout, seq=o.seq)
    if small:
        shape.update(small)
    torch.manual_seed(0)
    model = PlainBertForMaskedLM(**shape)
    args = MerakArguments(
        output_dir=os.path.join(tempfile.gettempdir(), "merak_ref_bench"), bf16=cuda, use_cpu=not cuda,
        per_device_train_batch_size=o.mbs, gradient_accumulation_steps=1, max_steps=10 ** 6,
        learning_rate=1e-4, weight_decay=0.01, max_grad_norm=1.0, lr_scheduler_type="constant",
        logging_steps=10 ** 9, wall_clock_breakdown=False, report_to="none", activation_checkpointing=False,
        save=False, seed=1234, input_names=["input_ids", "attention_mask"], dataloader_pin_memory=False)
    # ``adafactor`` left ``TrainingArguments`` in transformers 5.x; the reference's
    # ``create_optimizer`` still reads it (Merak/merak_trainer.py:242)
    if not hasattr(args, "adafactor"):
        args.adafactor = False
    ds = MlmDataset(shape["vocab"], o.seq, 1 << 16, seed=0)
    trainer = MerakTrainer(model=model, args=args, train_dataset=ds)
    trainer.init_engine()
    engine = trainer.engine
    engine.batch_fn = trainer.prepare_data
    trainer.tuning_params.global_steps = 1

    bench_ds = MlmDataset(shape["vocab"], o.seq, 1 << 30, seed=1 + rank)
    n_distinct = 4

    def sync_all():
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    def timed(batches, read_loss):
        data = _Cycle(batches)
        engine.reset_dataiterator(iter(data))
        for _ in range(o.warmup):
            loss = engine.train_batch(data)
            if read_loss:
                float(loss)
        sync_all()
        sampler = clock_sampler_cls(local)
        if cuda:
            sampler.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        else:
            import time
            t0 = time.perf_counter()
        last = None
        for _ in range(o.steps):
            last = engine.train_batch(data)
            if read_loss:
                last = float(last)
        if cuda:
            e1.record()
            sync_all()
            clocks = sampler.stop()
            ms = e0.elapsed_time(e1)
        else:
            clocks = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
            ms = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), clocks, float(last)

    ms_dev, clocks, _ = timed(_batches(bench_ds, o.mbs, n_distinct, device, pinned=False), read_loss=False)
    host = _batches(bench_ds, o.mbs, n_distinct, device, pinned=True)
    ms_e2e, _, loss = timed(host, read_loss=True)
    h2d = sum(v.numel() * v.element_size() for v in host[0].values())
    tokens = o.mbs * o.seq * world * o.steps
    if rank == 0:
        print(json.dumps({
            "metric": metric, "value": tokens / (ms_dev / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": o.steps, "warmup": o.warmup, "ms_per_step": ms_dev / o.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if cuda else "fp32",
            "data": "synthetic (uniform token ids, 15% MLM masking 80/10/10), random-init weights N(0,0.02)",
            "impl": "reference",
            "config": {"model": "BERT-large MLM (24L d1024 h16 ff4096 vocab30522)" if not small else "small test shape",
                       "global_batch": o.mbs * world, "seq_len": o.seq, "micro_batch_per_gpu": o.mbs,
                       "parallelism": "dp%d" % world, "hidden_dropout": o.dropout, "attention_dropout": 0.0,
                       "optimizer": "torch.optim.AdamW on bf16 parameters (the reference keeps no fp32 master "
                                    "copy without ZeRO), clip 1.0",
                       "model_code": "plain PyTorch (nn.Linear, nn.LayerNorm, scaled_dot_product_attention) "
                                     "traced and run by the reference's engine",
                       "l2_policy": "no flush: one step touches >20 GB, far more than the 126 MB L2"},
            "clocks": clocks, "gpu_launches": 0,
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / o.steps,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4},
            "final_loss": loss,
        }), flush=True)
    sync_all()
    if dist.is_initialized():
        dist.destroy_process_group()
