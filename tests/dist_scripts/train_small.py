"""Trains a small model for a few steps under a given parallel layout and writes the loss curve.
Launched by the tests through torch.distributed.run (gloo on CPU, nccl on GPUs)."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ.setdefault("MERAK_QUIET", "1")

import torch

import merak_b200 as Merak
from merak_b200.models.bert import BertForMaskedLM, bert_config
from merak_b200.models.gpt2 import GPT2LMHeadModel, gpt2_config
from merak_b200.models.llama import LlamaForCausalLM, llama_config
from merak_b200.utils.datasets import SyntheticTokenDataset


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--sp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--tp_overlap", type=int, default=0)
    ap.add_argument("--model", default="gpt2")
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--mbs", type=int, default=2)
    ap.add_argument("--gas", type=int, default=4)
    ap.add_argument("--schedule", default="1f1b")
    ap.add_argument("--recompute", type=int, default=0)
    ap.add_argument("--ratio", default=None)
    ap.add_argument("--zero", type=int, default=0)
    ap.add_argument("--parallel_vocab", type=int, default=0)
    ap.add_argument("--megatron_sp", type=int, default=0)
    ap.add_argument("--split", default="nearest_min_deps")
    ap.add_argument("--dtype", default="fp32")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--save_dir", default=None)
    ap.add_argument("--resume", default=None)
    ap.add_argument("--n_head", type=int, default=0)
    ap.add_argument("--meta", type=int, default=0)
    ap.add_argument("--dealloc", type=int, default=0)
    ap.add_argument("--comm", default="nccl")
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--vocab", type=int, default=512)
    ap.add_argument("--seq", type=int, default=32)
    ap.add_argument("--lr", type=float, default=0.0)
    ap.add_argument("--data_seed", type=int, default=7)
    ap.add_argument("--data_size", type=int, default=16)
    ap.add_argument("--cuda_graph", type=int, default=0)
    ap.add_argument("--dp_overlap", type=int, default=1)
    ap.add_argument("--dp_bucket", type=int, default=8 << 20)
    ap.add_argument("--inject_overflow", type=int, default=-1, help="step whose gradients get an inf written in")
    ap.add_argument("--user_opt", default="", help="sgd | adamw: a torch.optim optimizer built by the trainer hook")
    ap.add_argument("--dropout", type=float, default=0.0, help="hidden, embedding and attention dropout of the model")
    ap.add_argument("--attn_dropout", type=float, default=-1.0, help="attention dropout alone (default: --dropout)")
    ap.add_argument("--check_replicated", type=int, default=0,
                    help="after training: parameters that are not tensor-parallel must be bit-identical on every "
                         "rank of the tensor-parallel group")
    ap.add_argument("--out", required=True)
    o = ap.parse_args()
    if o.attn_dropout < 0:
        o.attn_dropout = o.dropout

    Merak.init(o.pp, o.tp, o.dp, sp=o.sp, ep=o.ep, backend="gloo" if o.device == "cpu" else "nccl")
    torch.manual_seed(1234)
    V, L = o.vocab, o.seq
    import contextlib
    build_ctx = Merak.init_empty_weights() if o.meta else contextlib.nullcontext()
    build_ctx.__enter__()
    if o.model == "gpt2":
        over = dict(n_head=o.n_head, n_embd=32 * o.n_head) if o.n_head else {}
        model = GPT2LMHeadModel(gpt2_config("gpt2-tiny", vocab_size=V, resid_pdrop=o.dropout, embd_pdrop=o.dropout,
                                            attn_pdrop=o.attn_dropout, **over))
        task = "causal"
    elif o.model == "bert":
        model = BertForMaskedLM(bert_config("bert-tiny", vocab_size=V, hidden_dropout_prob=o.dropout,
                                            attention_probs_dropout_prob=o.attn_dropout))
        task = "mlm"
    elif o.model == "moe":
        from merak_b200.models.moe import DeepseekV2ForCausalLM, deepseek_v2_config
        model = DeepseekV2ForCausalLM(deepseek_v2_config("deepseek-tiny", vocab_size=V, aux_loss_alpha=0.01))
        task = "causal"
    else:
        model = LlamaForCausalLM(llama_config("llama-tiny", vocab_size=V))
        task = "causal"
    build_ctx.__exit__(None, None, None)
    args = Merak.MerakArguments(
        output_dir=o.save_dir or "/tmp/merak_b200_test", per_device_train_batch_size=o.mbs,
        gradient_accumulation_steps=o.gas, max_steps=o.steps, logging_steps=0, learning_rate=o.lr or (1e-3 if o.model == "gpt2" else 3e-3),
        lr_scheduler_type="constant", weight_decay=0.01, wall_clock_breakdown=False, report_to="none",
        no_cuda=(o.device == "cpu"), train_schedule=o.schedule, activation_checkpointing=bool(o.recompute),
        activation_checkpoint_ratio=[o.ratio] if o.ratio else None, zero_stage=1 if o.zero else None,
        parallel_vocab=bool(o.parallel_vocab), sequence_parallel=o.sp > 1, tp_overlapping_level=o.tp_overlap, megatron_sequence_parallel=bool(o.megatron_sp),
        split_method=o.split, bf16=(o.dtype == "bf16"), fp16=(o.dtype == "fp16"), initial_scale_power=8, hysteresis=1,
        loss_scale_window=3, seed=1234, save=bool(o.save_dir), save_steps=o.steps,
        resume_from_checkpoint=o.resume, comm_mode=o.comm, max_grad_norm=o.clip,
        deallocate_pipeline_outputs=bool(o.dealloc), cuda_graph=bool(o.cuda_graph),
        overlap_dp_reduce=bool(o.dp_overlap), dp_overlap_bucket_elems=o.dp_bucket)
    # every data-parallel layout must see the same global batch per step: dataset order is by index
    ds = SyntheticTokenDataset(V, L, o.data_size, task=task, seed=o.data_seed)   # default: two global batches, revisited
    FixedOrderTrainer.user_opt = o.user_opt
    trainer = FixedOrderTrainer(model, args, train_dataset=ds)
    losses = []
    engine = trainer.init_engine()
    if o.resume:
        it = trainer.load_checkpoint(o.resume)
        trainer.params.resume(it)
    data_iter = trainer._batch_iter(trainer.train_dataloader)
    if o.resume:
        for _ in range(it * o.gas):        # the fixed-order loader restarts at 0: skip what was consumed
            next(data_iter)
    scales, skipped = [], []
    reduce_grads = engine._exec_reduce_grads
    for step in range(o.steps):
        if step == o.inject_overflow:
            def poisoned():
                engine.flat.grad[3] = float("inf")        # host-injected overflow
                reduce_grads()
            engine._exec_reduce_grads = poisoned
        else:
            engine._exec_reduce_grads = reduce_grads
        before = engine.flat.model.clone() if engine.flat is not None else None
        losses.append(float(engine.train_batch(data_iter)))
        if engine.loss_scaler is not None:
            scales.append(engine.loss_scaler.cur_scale)
            skipped.append(bool(torch.equal(before, engine.flat.model)))
        trainer.params.step()
    if o.check_replicated:
        from merak_b200.parallel import mpu
        group = mpu.get_model_parallel_group()
        n = torch.distributed.get_world_size(group)
        for name, prm in engine.module.named_parameters():
            if getattr(prm, "model_parallel", False):
                continue
            mine = prm.detach().float().contiguous()
            every = [torch.empty_like(mine) for _ in range(n)]
            torch.distributed.all_gather(every, mine, group=group)
            for r, other in enumerate(every):
                assert torch.equal(other, every[0]), "replicated parameter %s differs on tensor-parallel rank %d" % (name, r)
    if o.save_dir:
        trainer.save_checkpoint()
    if torch.distributed.get_rank() == 0:
        with open(o.out, "w") as f:
            json.dump({"losses": losses, "scales": scales, "skipped": skipped}, f)
    torch.distributed.barrier()
    Merak.initialize.destroy()


class _SequentialSampler:
    """Global micro-batch g of step s goes to dp rank (g % dp): any dp degree consumes the same
    samples per optimizer step."""

    def __init__(self, n, mbs, gas, dp_rank, dp_size):
        self.n, self.mbs, self.gas, self.r, self.d = n, mbs, gas, dp_rank, dp_size

    def __len__(self):
        return 1 << 30

    def __iter__(self):
        per_step = self.gas * self.d                  # micro-batches per optimizer step, globally
        step = 0
        while True:
            for k in range(self.gas):
                g = step * per_step + k * self.d + self.r
                yield [i % self.n for i in range(g * self.mbs, (g + 1) * self.mbs)]
            step += 1


class FixedOrderTrainer(Merak.MerakTrainer):
    user_opt = ""

    def _wants_custom_optimizer(self):
        return bool(self.user_opt)

    def create_optimizer(self, params):
        params = list(params)
        decay = [p for p in params if p.dim() > 1]
        rest = [p for p in params if p.dim() <= 1]
        groups = [{"params": decay, "weight_decay": 0.01}, {"params": rest, "weight_decay": 0.0}]
        if self.user_opt == "sgd":
            return torch.optim.SGD(groups, lr=0.05, momentum=0.9)
        return torch.optim.AdamW(groups, lr=self.args.learning_rate)

    def create_dataloader(self, dataset, batch_size, train=True):
        from torch.utils.data import DataLoader
        from merak_b200.parallel import mpu
        s = _SequentialSampler(len(dataset), batch_size, self.args.gradient_accumulation_steps,
                               mpu.get_data_parallel_rank(), mpu.get_data_parallel_world_size())
        return DataLoader(dataset, batch_sampler=s, collate_fn=self.data_collator)


if __name__ == "__main__":
    main()
