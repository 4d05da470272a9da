"""``MerakTrainer``: the user-facing training loop (Merak/merak_trainer.py:49-496).

Builds the pipeline module (trace -> shard -> stage assignment -> tensor-parallel layers), the data
loaders (data-parallel sharded sampler), the optimizer / scheduler / loss, and drives
``PipelineEngine.train_batch``.  The hooks of the reference are kept overridable:
``create_dataloader``, ``create_optimizer``, ``create_lr_scheduler``, ``get_loss_fn``,
``prepare_data``; so are ``evaluation``, ``save_checkpoint`` and ``load_checkpoint``.  With
``args.return_logits`` and a ``compute_metrics`` callable the evaluation also reports metrics of the
logits (accuracy and the like), averaged over the data-parallel group.
"""
from __future__ import annotations

import math
import os
import time
from typing import Callable, Dict, Iterable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.data import DataLoader, Dataset

from . import initialize
from .args import MerakArguments, manual_set_args, mergeargs, print_args
from .ops.cross_entropy import softmax_cross_entropy
from .parallel import mpu
from .pipeline.engine import PipelineEngine
from .pipeline.module import PipelineModule
from .printer import AccMetric, log_dist, logger
from .recompute import checkpoint, model_parallel_manual_seed
from .utils.trainer_utils import BaseParams, MegatronPretrainingRandomSampler, RepeatingLoader, WorkerInitObj


def default_collate(features):
    if isinstance(features[0], dict):
        return {k: torch.stack([torch.as_tensor(f[k]) for f in features]) for k in features[0]}
    if isinstance(features[0], (tuple, list)):
        return tuple(torch.stack([torch.as_tensor(f[i]) for f in features]) for i in range(len(features[0])))
    return torch.stack([torch.as_tensor(f) for f in features])


def get_scheduler_lambda(name: str, warmup: int, total: int) -> Callable[[int], float]:
    name = (name or "linear").lower()

    def fn(step: int) -> float:
        if warmup > 0 and step < warmup:
            return float(step) / float(max(1, warmup))
        if name == "constant" or name == "constant_with_warmup":
            return 1.0
        progress = float(step - warmup) / float(max(1, total - warmup))
        progress = min(max(progress, 0.0), 1.0)
        if name == "cosine":
            return 0.5 * (1.0 + math.cos(math.pi * progress))
        if name == "polynomial":
            return (1.0 - progress) ** 2
        return 1.0 - progress      # linear
    return fn


class LambdaLR:
    """Learning-rate schedule over any optimizer exposing ``param_groups`` (the fused AdamW included)."""

    def __init__(self, optimizer, lr_lambda: Callable[[int], float]):
        self.optimizer, self.fn = optimizer, lr_lambda
        self.base_lrs = [g["lr"] for g in optimizer.param_groups]
        self.last_step = 0
        self._apply()

    def _apply(self):
        for g, base in zip(self.optimizer.param_groups, self.base_lrs):
            g["lr"] = base * self.fn(self.last_step)

    def step(self):
        self.last_step += 1
        self._apply()

    def get_last_lr(self):
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self):
        return {"last_step": self.last_step, "base_lrs": self.base_lrs}

    def load_state_dict(self, sd):
        self.last_step, self.base_lrs = sd["last_step"], sd["base_lrs"]
        self._apply()


class MerakTrainer:

    def __init__(self, model: nn.Module, args: Optional[MerakArguments] = None, train_dataset: Optional[Dataset] = None,
                 eval_dataset: Optional[Dataset] = None, data_collator: Optional[Callable] = None,
                 leaf_modules: Iterable[type] = (), optimizers=(None, None), loss_fn: Optional[Callable] = None,
                 tokenizer=None, compute_metrics: Optional[Callable] = None, **kwargs):
        if not mpu.is_initialized():
            initialize.init(1, 1, 1)
        self.args = args or MerakArguments()
        self.model = model
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        self.data_collator = data_collator or default_collate
        self.leaf_modules = tuple(leaf_modules)
        self.tokenizer = tokenizer
        self.optimizer, self.lr_scheduler = optimizers
        config = getattr(model, "config", None)
        if config is not None:
            mergeargs(self.args, config)
        if self.args.num_layers is None:        # no configuration, or one that does not state the depth
            self.args.num_layers = max(1, sum(1 for _ in model.children()))
            if self.args.shard_count is None:
                self.args.shard_count = 2 * self.args.num_layers + 4
        manual_set_args(self.args)
        model_parallel_manual_seed(self.args.seed)
        if dist.is_initialized() and dist.get_rank() == 0:
            print_args(self.args, printer=lambda s: None if os.environ.get("MERAK_QUIET") else print(s))
        self.params = BaseParams(self.args, mpu.get_data_parallel_world_size())
        self.summary_writer = None
        self._user_loss_fn = loss_fn
        # ``compute_metrics(EvalPrediction) -> {name: value}`` on the evaluation logits (needs ``return_logits``)
        self.compute_metrics = compute_metrics
        self.eval_metrics: Dict[str, float] = {}
        self.loss_fn = self.get_loss_fn()
        self.engine: Optional[PipelineEngine] = None
        self.pipe_model: Optional[PipelineModule] = None
        self.train_dataloader = None
        self.eval_dataloader = None
        self.create_pipeline_module()

    # ------------------------------------------------------------------------------------------
    # hooks
    # ------------------------------------------------------------------------------------------
    def get_loss_fn(self) -> Callable:
        """Loss applied to the last stage's output and the labels.  Default: token cross entropy
        (next-token shift for causal LMs, ``ignore_index=-100``); the vocab-parallel form when the
        output projection is vocabulary-sharded (Merak/merak_trainer.py:291-327)."""
        if self._user_loss_fn is not None:
            return self._user_loss_fn
        causal = self._is_causal()
        parallel_vocab = self.args.parallel_vocab and mpu.get_model_parallel_world_size() > 1

        def loss_fn(outputs, labels):
            logits = outputs[0] if isinstance(outputs, (tuple, list)) else outputs
            if isinstance(logits, dict):          # a model output object that survived tracing as a mapping
                logits = logits["logits"] if "logits" in logits else next(iter(logits.values()))
            if isinstance(labels, dict):
                labels = labels.get("labels", next(iter(labels.values())))
            if causal:
                logits, labels = logits[:, :-1, :], labels[:, 1:]
            if parallel_vocab:
                start = mpu.get_model_parallel_rank() * logits.shape[-1]
                return softmax_cross_entropy(logits, labels, vocab_start=start,
                                             tp_group=mpu.get_model_parallel_group())
            if logits.dim() == 2 and labels.dim() == 1:
                return softmax_cross_entropy(logits, labels)
            return softmax_cross_entropy(logits, labels)
        return loss_fn

    def _is_causal(self) -> bool:
        mt = getattr(getattr(self.model, "config", None), "model_type", "") or ""
        name = type(self.model).__name__.lower()
        return "causal" in name or "lmhead" in name or mt in ("gpt2", "llama", "opt", "gptj", "qwen2", "mistral")

    def create_dataloader(self, dataset: Optional[Dataset], batch_size: int, train: bool = True):
        if dataset is None:
            return None
        sampler = MegatronPretrainingRandomSampler(
            total_samples=len(dataset), consumed_samples=0, micro_batch_size=batch_size,
            data_parallel_rank=mpu.get_data_parallel_rank(), data_parallel_size=mpu.get_data_parallel_world_size(),
            seed=self.args.seed)
        return DataLoader(dataset, batch_sampler=sampler, num_workers=self.args.dataloader_num_workers,
                          collate_fn=self.data_collator, pin_memory=torch.cuda.is_available(),
                          worker_init_fn=WorkerInitObj(self.args.seed))

    def create_optimizer(self, params):
        """Return a ``torch.optim`` optimizer to override the built-in fused AdamW (which is used
        when this returns ``None``)."""
        if self.args.adafactor:
            from transformers.optimization import Adafactor
            return Adafactor(params, lr=self.args.learning_rate, scale_parameter=False, relative_step=False)
        return None

    def create_lr_scheduler(self, optimizer):
        total = self.params.max_steps if self.params.max_steps and self.params.max_steps > 0 else 1000000
        warm = self.args.get_warmup_steps(total)
        return LambdaLR(optimizer, get_scheduler_lambda(self.args.lr_scheduler_type, warm, total))

    def prepare_data(self, batch):
        """Maps a loader batch to what the engine consumes (a dict keyed by input name plus
        ``labels``, or a tuple in ``input_names + labels`` order)."""
        return batch

    # ------------------------------------------------------------------------------------------
    def get_dummy_inputs(self) -> Optional[Dict[str, torch.Tensor]]:
        dataset = self.train_dataset if self.train_dataset is not None else self.eval_dataset
        if dataset is None:
            return None
        # one micro-batch of real samples: a graph exported with static shapes bakes this batch size in
        size = self.args.per_device_train_batch_size if self.train_dataset is not None else self.args.per_device_eval_batch_size
        n = max(1, min(int(size), len(dataset)))
        sample = self.data_collator([dataset[i] for i in range(n)])
        if isinstance(sample, dict):
            names = self.args.input_names or [k for k in sample if k not in ("labels", "label")]
            return {k: sample[k] for k in names if k in sample}
        return None

    def create_pipeline_module(self):
        a = self.args
        if a.trace_method in ("fx", "dynamo"):
            dummy = self.get_dummy_inputs()
            if a.input_names is None and dummy is not None:
                import inspect
                sig = inspect.signature(self.model.forward).parameters
                a.input_names = [k for k in dummy if k in sig]
                dummy = {k: dummy[k] for k in a.input_names}
            self.pipe_model = PipelineModule(self.model, a, loss_fn=self.loss_fn,
                                             activation_checkpoint_func=checkpoint, leaf_modules=self.leaf_modules,
                                             dummy_inputs=dummy)
        else:
            if mpu.get_pipe_parallel_world_size() * mpu.get_model_parallel_world_size() != 1:
                raise ValueError("trace_method='none' supports data parallelism only")
            wrapped = _WholeModel(self.model, a.input_names or ["input_ids"])
            self.pipe_model = PipelineModule(self.model, a, loss_fn=self.loss_fn, layers=[wrapped])
        if dist.is_initialized():
            dist.barrier()

    def init_engine(self):
        if self.engine is not None:
            return self.engine
        a = self.args
        self.train_dataloader = self._make_dataloader(self.train_dataset, a.per_device_train_batch_size, True)
        n_mb = len(self.train_dataloader) if self.train_dataloader is not None and hasattr(self.train_dataloader, "__len__") else None
        self.params.train(n_mb)
        self.engine = PipelineEngine(self.pipe_model, a, optimizer=self.optimizer, lr_scheduler=self.lr_scheduler,
                                     loss_fn=self.loss_fn,
                                     optimizer_factory=self._make_optimizer if self._wants_custom_optimizer() else None,
                                     lr_scheduler_factory=self.create_lr_scheduler)
        self.optimizer, self.lr_scheduler = self.engine.optimizer, self.engine.lr_scheduler
        # Tracing, sharding and the tensor-parallel rebuild have drawn from the default generators since the
        # seeds were set, and not the same amount on every rank (a rank builds the layers of its own stage,
        # rank 0 writes caches).  Training starts from the seeded state again, so that ranks of one
        # tensor-parallel group draw the same dropout masks for the activations they all hold.
        model_parallel_manual_seed(a.seed)
        return self.engine

    # The hooks may be overridden with this class's signatures or with the reference's
    # (``create_dataloader(self)`` sets / returns the training loader, Merak/merak_trainer.py:189-223;
    # ``create_optimizer(self, model)`` reads ``model.named_parameters()``, :225-257): both forms are called
    # the way they were written.
    @staticmethod
    def _positional_count(fn) -> int:
        import inspect
        return sum(1 for p in inspect.signature(fn).parameters.values()
                   if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD, p.VAR_POSITIONAL))

    def _make_dataloader(self, dataset, batch_size: int, train: bool):
        if self._positional_count(self.create_dataloader) == 0:       # reference-style override, training data only
            if not train:
                return MerakTrainer.create_dataloader(self, dataset, batch_size, False)
            made = self.create_dataloader()
            return made if made is not None else self.train_dataloader
        return self.create_dataloader(dataset, batch_size, train)

    def _make_optimizer(self, params):
        if self._positional_count(self.create_optimizer) == 0:
            return self.create_optimizer()
        return self.create_optimizer(_OptimizerTarget(params, self.pipe_model))

    def _wants_custom_optimizer(self) -> bool:
        return self.args.adafactor or type(self).create_optimizer is not MerakTrainer.create_optimizer

    def _writer(self):
        if self.summary_writer is None and (not dist.is_initialized() or dist.get_rank() == 0) and \
                self.args.report_to == "tensorboard":
            try:
                from torch.utils.tensorboard import SummaryWriter
                import socket
                log_dir = self.args.logging_dir or os.path.join(self.args.output_dir, "runs", "%s_%s" % (
                    time.strftime("%b%d_%H-%M-%S"), socket.gethostname()))
                self.summary_writer = SummaryWriter(log_dir=log_dir)
            except Exception:
                self.summary_writer = False
        return self.summary_writer or None

    def _batch_iter(self, loader):
        for batch in RepeatingLoader(loader):
            yield self.prepare_data(batch)

    def train(self, resume_from_checkpoint: Optional[str] = None):
        a = self.args
        engine = self.init_engine()
        resume = resume_from_checkpoint or a.resume_from_checkpoint
        if resume:
            it = self.load_checkpoint(resume)
            self.params.resume(it)
            engine.global_steps = it
        if a.lora_config:
            self._inject_lora()
        data_iter = self._batch_iter(self.train_dataloader)
        loss = None
        last_eval_epoch = -1
        while not self.params.should_break():
            loss = engine.train_batch(data_iter)
            self.params.step()
            if self.params.should_log():
                w = self._writer()
                if w is not None:
                    w.add_scalar("Train/loss", float(loss), self.params.global_steps)
                    w.add_scalar("Train/learning_rate", engine.get_lr(), self.params.global_steps)
            if self.params.should_save():
                self.save_checkpoint()
            spe = self.params.num_steps_per_epoch
            if a.eval_strategy == "steps" and a.eval_steps and self.params.global_steps % a.eval_steps == 0:
                self.evaluation()
            elif a.eval_strategy == "epoch" and spe and self.params.global_steps % spe == 0:
                epoch = self.params.global_steps // spe
                if epoch != last_eval_epoch:
                    self.evaluation()
                    last_eval_epoch = epoch
        return loss

    def evaluation(self, max_batches: Optional[int] = None):
        if self.eval_dataset is None:
            return None
        engine = self.init_engine()
        if self.eval_dataloader is None:
            bs = self.args.per_device_eval_batch_size
            static = getattr(self.pipe_model, "static_batch_size", None)
            if static and bs != static:
                log_dist("the traced graph has the micro-batch size %d built in: evaluating with it instead of %d"
                         % (static, bs), ranks=[0])
                bs = static
            self.eval_dataloader = self._make_dataloader(self.eval_dataset, bs, False)
        it = self._batch_iter(self.eval_dataloader)
        n_steps = max(1, len(self.eval_dataloader) // engine.micro_batches)
        if max_batches:
            n_steps = min(n_steps, max_batches)
        elif self.args.eval_steps and self.args.eval_strategy != "steps":
            # the reference's meaning of ``--eval_steps``: how many evaluation steps one evaluation takes
            # (Merak/utils/parameters.py:72-74); with ``eval_strategy=steps`` it is the interval between evaluations
            n_steps = min(n_steps, int(self.args.eval_steps))
        total = 0.0
        metrics = AccMetric()
        for _ in range(n_steps):
            out = engine.eval_batch(it)
            if self.args.return_logits:
                # (loss, logits, labels); the lists are filled on the last pipeline stage only
                out, logits, labels = out
                if self.compute_metrics is not None and logits:
                    self._update_metrics(metrics, logits, labels)
            total += float(out)
        loss = total / n_steps
        self.eval_metrics = self._gather_metrics(metrics) if self.compute_metrics is not None else {}
        w = self._writer()
        if w is not None:
            w.add_scalar("Eval/loss", loss, self.params.global_steps)
            for name, value in self.eval_metrics.items():
                w.add_scalar("Eval/%s" % name, value, self.params.global_steps)
        extra = "".join(", %s: %.4f" % kv for kv in sorted(self.eval_metrics.items()))
        log_dist("eval loss: %.4f%s" % (loss, extra), ranks=[0])
        if dist.is_initialized():
            dist.barrier()
        return loss

    def _update_metrics(self, metrics: "AccMetric", logits, labels):
        """Feeds one evaluation step's last-stage outputs to ``compute_metrics`` (the reference's
        examples/lora/run_vit.py:243-268 does this in a trainer subclass)."""
        from types import SimpleNamespace

        def first(x):
            while isinstance(x, (tuple, list, dict)):
                x = (x["labels"] if "labels" in x else next(iter(x.values()))) if isinstance(x, dict) else x[0]
            return x
        preds = torch.cat([first(t).float().cpu() for t in logits])
        refs = torch.cat([first(t).cpu() for t in labels])
        for name, value in self.compute_metrics(SimpleNamespace(predictions=preds, label_ids=refs)).items():
            metrics.update(name, float(value), int(refs.shape[0]))

    def _gather_metrics(self, metrics: "AccMetric") -> Dict[str, float]:
        """Sample-weighted means over the data-parallel group of what the last pipeline stage measured,
        handed to every rank (rank 0 writes the log)."""
        local = {k: (m.total, m.count) for k, m in metrics.metrics.items()}
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return {k: t / max(1, c) for k, (t, c) in local.items()}
        gathered = [None] * dist.get_world_size()
        dist.all_gather_object(gathered, local)
        sums: Dict[str, list] = {}
        for part in gathered:
            for k, (t, c) in part.items():
                acc = sums.setdefault(k, [0.0, 0])
                acc[0] += t
                acc[1] += c
        return {k: t / max(1, c) for k, (t, c) in sums.items()}

    # ------------------------------------------------------------------------------------------
    def save_checkpoint(self, best_model: bool = False, loss: Optional[float] = None):
        from .checkpoint import CheckpointSaver, rotate_checkpoints
        engine = self.init_engine()
        saver = getattr(self, "_saver", None) or CheckpointSaver(self.args)
        self._saver = saver
        saver.save_checkpoint(self.params.global_steps, engine.module, engine.optimizer, engine.lr_scheduler,
                              engine=engine, best_model=best_model, loss=loss)
        rotate_checkpoints(self.args, saver.root_dir)

    def load_checkpoint(self, path: str) -> int:
        from .checkpoint import CheckpointLoader
        engine = self.init_engine()
        return CheckpointLoader(self.args).load_checkpoint(engine.module, engine.optimizer, engine.lr_scheduler,
                                                           path, engine=engine)

    def _inject_lora(self):
        from .lora import inject_lora
        cfg = self.args.get_lora_config()
        inject_lora(self.engine, cfg, self.args.adapter_name)


class _OptimizerTarget(list):
    """What ``create_optimizer`` receives: the list of this stage's parameters to optimise (each once, tied
    copies removed), which also answers ``named_parameters()`` / ``parameters()`` / ``named_modules()`` /
    ``modules()`` like the pipeline module the reference passes, restricted to those parameters."""

    def __init__(self, params, module: nn.Module):
        super().__init__(params)
        self._module = module

    def named_parameters(self, *args, **kwargs):
        keep = {id(p) for p in self}
        seen = set()
        for name, p in self._module.named_parameters(*args, **kwargs):
            if id(p) in keep and id(p) not in seen:
                seen.add(id(p))
                yield name, p

    def parameters(self, *args, **kwargs):
        return iter(self)

    def named_modules(self, *args, **kwargs):
        return self._module.named_modules(*args, **kwargs)

    def modules(self):
        return self._module.modules()


class _WholeModel(nn.Module):
    """An untraced model as a single pipeline shard (``trace_method='none'``)."""

    def __init__(self, model: nn.Module, input_names):
        super().__init__()
        self.model = model
        self.external_inputs = list(input_names)
        self.input_names, self.output_names = [], ["output"]

    def forward(self, *inputs):
        out = self.model(**dict(zip(self.external_inputs, inputs)))
        return out[0] if isinstance(out, (tuple, list)) and not isinstance(out, torch.Tensor) and len(out) == 1 else out
