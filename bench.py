"""Headline benchmark: BERT-large masked-LM pre-training throughput (tokens/s), bf16, sequence 512,
micro-batch 32 per GPU, data parallel over N GPUs of one node (weak scaling), synthetic data and
random-init weights, through the framework's public API (``init`` / ``MerakArguments`` /
``MerakTrainer``).

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...     # the reference implementation, if it can run here

Rank 0 prints one JSON line.  ``value`` is timed on the device (CUDA events around exactly K
steps, max over ranks) with inputs already resident; ``e2e.value`` repeats the measurement with,
per step, the host->device copy of that step's batch from pinned memory and a device->host read of
the loss inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

os.environ.setdefault("MERAK_QUIET", "1")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

SEQ, MBS = 512, 32
METRIC = "train tokens/s (device-timed, max over ranks)"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="bert-large")
    ap.add_argument("--mbs", type=int, default=MBS)
    ap.add_argument("--seq", type=int, default=SEQ)
    ap.add_argument("--dropout", type=float, default=0.1)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--cuda-graph", type=int, default=1)
    ap.add_argument("--dp-overlap", type=int, default=1, help="reduce gradients while the backward pass runs")
    ap.add_argument("--check", action="store_true",
                    help="before timing, train 5 steps from the same seed with --comm as given and with NCCL "
                         "collectives and require the two loss curves to agree")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons during the timed region."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx = device_index
        self.proc, self.path = None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def build_ours(o, device, comm=None):
    import torch

    import merak_b200 as Merak
    from merak_b200.models.bert import BertForMaskedLM, bert_config
    from merak_b200.utils.datasets import SyntheticTokenDataset

    comm = comm or o.comm
    import torch.distributed as dist
    if not dist.is_initialized():
        Merak.init(pp=1, tp=1, dp=o.gpus)
    torch.manual_seed(0)
    cfg = bert_config(o.model, hidden_dropout_prob=o.dropout, attention_probs_dropout_prob=0.0)
    model = BertForMaskedLM(cfg)
    args = Merak.MerakArguments(
        output_dir=os.path.join(tempfile.gettempdir(), "merak_b200_bench"), bf16=True,
        per_device_train_batch_size=o.mbs, gradient_accumulation_steps=1, max_steps=10 ** 9,
        learning_rate=1e-4, weight_decay=0.01, max_grad_norm=1.0, lr_scheduler_type="constant",
        logging_steps=0, wall_clock_breakdown=False, report_to="none", activation_checkpointing=False,
        split_method="layer_split", comm_mode=comm, cuda_graph=bool(o.cuda_graph), seed=0,
        overlap_dp_reduce=bool(o.dp_overlap))
    ds = SyntheticTokenDataset(cfg.vocab_size, o.seq, 1 << 20, task="mlm", seed=0)
    trainer = Merak.MerakTrainer(model, args, train_dataset=ds)
    engine = trainer.init_engine()
    return cfg, trainer, engine


def make_batches(cfg, o, n, device, pinned: bool):
    """n synthetic MLM batches (uniform token ids, 15% masked with the 80/10/10 rule)."""
    import torch
    from merak_b200.utils.datasets import SyntheticTokenDataset
    rank = int(os.environ.get("RANK", "0"))
    ds = SyntheticTokenDataset(cfg.vocab_size, o.seq, 1 << 30, task="mlm", seed=1 + rank)
    out = []
    for b in range(n):
        items = [ds[b * o.mbs + i] for i in range(o.mbs)]
        batch = {k: torch.stack([it[k] for it in items]) for k in items[0]}
        if pinned:
            batch = {k: v.pin_memory() for k, v in batch.items()}
        else:
            batch = {k: v.to(device) for k, v in batch.items()}
        out.append(batch)
    return out


def run_ours(o):
    import torch
    import torch.distributed as dist
    from merak_b200.ops import _lib

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    check = None
    if o.check:
        # the same five steps from the same seed through both communication back ends
        curves = {}
        for comm in dict.fromkeys([o.comm, "nccl"]):
            cfg, trainer, engine = build_ours(o, device, comm=comm)
            it = iter(make_batches(cfg, o, 5, device, pinned=False))
            curves[comm] = [float(engine.train_batch(it)) for _ in range(5)]
            del trainer, engine, it
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
        a, b = curves[o.comm], curves["nccl"]
        worst = max(abs(x - y) / max(1.0, abs(y)) for x, y in zip(a, b))
        check = {"steps": 5, "losses": a, "losses_nccl": b, "max_rel_diff": worst, "tolerance": 2e-3}
        assert worst < 2e-3, "loss curves differ between comm=%s and comm=nccl: %s vs %s" % (o.comm, a, b)
    cfg, trainer, engine = build_ours(o, device)
    rank = dist.get_rank()
    world = dist.get_world_size()
    n_distinct = 4

    def cycle(batches):
        i = 0
        while True:
            yield batches[i % len(batches)]
            i += 1

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(data_iter, read_loss: bool):
        loss = None
        for _ in range(o.warmup):
            loss = engine.train_batch(data_iter)
            if read_loss:
                float(loss)
        after_warmup = float(loss) if loss is not None else None
        sync_all()
        launches0 = _lib.launch_count()
        sampler = ClockSampler(local)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = None
        for _ in range(o.steps):
            last = engine.train_batch(data_iter)
            if read_loss:
                last = float(last)
        e1.record()
        sync_all()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        launches = _lib.launch_count() - launches0 + getattr(engine, "graph_replay_launches", 0)
        engine.graph_replay_launches = 0
        return float(t.item()), clocks, launches, float(last), after_warmup

    # device-timed: batches already on the device
    dev_iter = cycle(make_batches(cfg, o, n_distinct, device, pinned=False))
    ms_dev, clocks, launches, loss_dev, loss_warm = timed(dev_iter, read_loss=False)
    # end to end: pinned host batches copied every step, loss read back every step
    host_batches = make_batches(cfg, o, n_distinct, device, pinned=True)
    ms_e2e, _, _, loss_e2e, _ = timed(cycle(host_batches), read_loss=True)
    h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values())

    tokens = o.mbs * o.seq * world * o.steps
    value = tokens / (ms_dev / 1000.0)
    e2e = tokens / (ms_e2e / 1000.0)
    status = _lib.status()
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": o.steps,
            "warmup": o.warmup, "ms_per_step": ms_dev / o.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform token ids, 15% MLM masking 80/10/10), "
            "random-init weights N(0,0.02)", "impl": "ours",
            "config": {"model": "BERT-large MLM (24L d1024 h16 ff4096 vocab30522)", "global_batch": o.mbs * world,
                       "seq_len": o.seq, "micro_batch_per_gpu": o.mbs, "parallelism": "dp%d" % world,
                       "hidden_dropout": o.dropout, "attention_dropout": 0.0, "optimizer": "AdamW fp32 master, clip 1.0",
                       "comm": o.comm, "cuda_graph": bool(o.cuda_graph),
                       "dp_reduce": "overlapped with the backward pass" if (o.dp_overlap and world > 1) else "after backward",
                       "l2_policy": "no flush: one step touches >20 GB (weights, activations, optimizer state), "
                                    "far more than the 126 MB L2"},
            "clocks": clocks, "gpu_launches": int(launches),
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / o.steps,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4},
            "loss_after_warmup": loss_warm, "final_loss": loss_e2e, "device_status_word": status,
            **({"check": check} if check is not None else {}),
        }), flush=True)
    sync_all()
    import merak_b200.initialize as ini
    ini.destroy()


def run_reference(o, small=None):
    """The reference arm: the unmodified reference package under ``baseline/_ref`` drives a
    plain-PyTorch BERT-large through its own trainer and engine (``baseline/ref_bench.py``).  The
    names it needs from ``transformers`` 4.x are registered from outside its tree
    (``baseline/compat.py``).  Any failure is reported as the ``unavailable`` line with the
    location of the failing frame."""
    here = os.path.dirname(os.path.abspath(__file__))
    ref = os.path.join(here, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "Merak")):
        why = "baseline/_ref is not installed"
    else:
        # this repository's ``Merak`` alias package must not shadow the reference
        sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != here]
        sys.path.insert(0, os.path.join(here, "baseline"))
        try:
            import ref_bench
            ref_bench.run(o, ref, ClockSampler, METRIC, small=small)
            return
        except Exception as exc:   # pragma: no cover - depends on the image
            import traceback
            tb = traceback.extract_tb(exc.__traceback__)
            where = "%s:%d" % (os.path.relpath(tb[-1].filename, here), tb[-1].lineno) if tb else "?"
            why = "%s at %s: %s" % (type(exc).__name__, where, (str(exc).splitlines() or [""])[0][:200])
            traceback.print_exc(file=sys.stderr)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def main():
    o = parse()
    if o.impl == "reference":
        # BENCH_REFERENCE_SMALL=1 shrinks the model so that the arm's plumbing can be exercised on a CPU box
        # in a test; the printed config then says "small test shape" and the number means nothing
        small = None
        if os.environ.get("BENCH_REFERENCE_SMALL") == "1":
            small = dict(vocab=512, hidden=64, layers=2, heads=4, ff=128)
            o.mbs, o.seq = 2, 32
        run_reference(o, small=small)
        return
    run_ours(o)


if __name__ == "__main__":
    main()
