"""``PipelineEngine``: executes a pipeline schedule instruction by instruction for one stage.

Responsibilities (Merak/core/merak_engine.py:1047-1487 and its Communication / NetCalculation
helper engines): micro-batch loading, stage forward / backward (incl. early recompute), activation
and gradient p2p with a one-time metadata handshake, tied-weight and data-parallel gradient
reduction, optimizer step with clipping / loss scaling, loss aggregation over dp and pp.

B200-specific choices:
* parameters live in one flat buffer with an fp32 gradient buffer the wgrad GEMMs accumulate into
  (``ops.optim.FlatBuffers``); DP reduction and the fused AdamW work on those flat buffers, ZeRO-1
  is "each dp rank owns a contiguous slice of them";
* p2p transfers run on a side stream ordered by events (no device-wide synchronisation);
* nothing in the step reads a device value on the host except the loss that is logged.
"""
from __future__ import annotations

import os

import math
from typing import Callable, Dict, Iterator, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops.optim import FlatBuffers, FusedAdamW
from ..amp.loss_scaler import DynamicLossScaler
from ..ops.rng import dropout_state
from ..parallel import mpu, p2p
from ..printer import SynchronizedWallClockTimer, log_dist, see_memory_usage, set_timer_log_rank
from ..recompute import RNGManager, checkpoint, pre_checkpoint, run_pending_recomputes
from . import schedules as S
from .module import PipelineModule


def _as_dict(batch, names: Sequence[str]) -> Dict[str, torch.Tensor]:
    if isinstance(batch, dict):
        return dict(batch)
    if isinstance(batch, torch.Tensor):
        batch = (batch,)
    return {n: t for n, t in zip(names, batch)}


class PipelineEngine:

    def __init__(self, model: PipelineModule, args, optimizer=None, lr_scheduler=None, loss_fn: Optional[Callable] = None,
                 tuning_params=None, optimizer_factory: Optional[Callable] = None,
                 lr_scheduler_factory: Optional[Callable] = None):
        self.module = model
        self.args = args
        self.loss_fn = loss_fn or model.loss_fn
        self.device = args.device
        self.stage_id = mpu.get_pipe_parallel_rank()
        self.num_stages = mpu.get_pipe_parallel_world_size()
        self.is_first = self.stage_id == 0
        self.is_last = self.stage_id == self.num_stages - 1
        self.dp_size = mpu.get_data_parallel_world_size()
        self.dp_rank = mpu.get_data_parallel_rank()
        self.micro_batches = args.gradient_accumulation_steps
        self.micro_batch_size = args.per_device_train_batch_size
        self.global_steps = 0
        self.timers = SynchronizedWallClockTimer()
        self.rng_manager = RNGManager()
        self.wall_clock_breakdown = bool(args.wall_clock_breakdown)
        # NVTX ranges around every pipeline instruction and every train_batch (for timeline profilers)
        self._nvtx = bool(getattr(args, "nvtx_ranges", False) or os.environ.get("MERAK_NVTX") == "1") and \
            self.device.type == "cuda"
        grid = mpu.get_grid()
        if grid is not None:
            topo = grid.topology
            set_timer_log_rank([topo.get_rank(pipe=s, data=0, sequence=0, model=0) for s in range(self.num_stages)])

        # names of everything a micro-batch carries, in tuple order
        self.input_names = list(args.input_names or sorted(model.input_to_shard, key=lambda n: model.input_to_shard[n]))
        self.batch_names = self.input_names + ["labels"]
        self.stage_inputs = model.input_to_stage_dic.get(self.stage_id, [])

        model.configure_distributed_model(self.device)
        model.tie_modules()
        self._configure_precision()
        self._configure_optimizer(optimizer, lr_scheduler, optimizer_factory, lr_scheduler_factory, tuning_params)
        self._setup_dp_overlap()

        if args.train_schedule == "last_no_recompute_1f1b" and self.is_last:
            model._force_no_recompute = True
            model.act_ckpt_interval = 0
        if args.train_schedule == "full_critical_path_1f1b":
            if self.is_last:
                model._force_no_recompute = True
                model.act_ckpt_interval = 0

        self._meta_sent = {"act": False, "grad": False}
        self._recv_act_meta = None
        self._recv_grad_meta = None
        self._reset_buffers(2)
        self.total_loss = None
        self.agg_loss = None
        self._warned_unused = False
        n_params = sum(p.numel() for p in model.parameters())
        log_dist("stage %d/%d: %d shards [%d,%d), %.2fM parameters" % (
            self.stage_id, self.num_stages, len(model.local_layers), model.local_start, model.local_stop,
            n_params / 1e6), ranks=[-1] if self.dp_rank == 0 and mpu.get_model_parallel_rank() == 0 else [])

    # ------------------------------------------------------------------------------------------
    # set-up
    # ------------------------------------------------------------------------------------------
    def _configure_precision(self):
        from ..amp import MixedPrecisionConfig
        self.amp = MixedPrecisionConfig(self.args)
        self.loss_scaler = self.amp.make_loss_scaler()

    def _unique_params(self) -> List[nn.Parameter]:
        seen, out = set(), []
        for p in self.module.parameters():
            if id(p) not in seen and p.requires_grad:
                seen.add(id(p))
                out.append(p)
        return out

    def _configure_optimizer(self, optimizer, lr_scheduler, optimizer_factory, lr_scheduler_factory, tuning_params):
        a = self.args
        params = tuning_params if tuning_params is not None else self._unique_params()
        self.flat: Optional[FlatBuffers] = None
        self.zero = a.zero_stage == 1 and self.dp_size > 1
        if optimizer is None and optimizer_factory is None:
            # framework optimizer: flat buffers + fused AdamW (+ ZeRO-1 shard)
            no_decay = set()
            for m in self.module.modules():
                if isinstance(m, nn.LayerNorm) or type(m).__name__.endswith("Norm"):
                    no_decay.update(id(p) for p in m.parameters(recurse=False))
            for p in params:
                p._no_weight_decay = id(p) in no_decay or p.dim() <= 1
            # Expert-parallel parameters differ between the ranks of the expert-parallel group: they get
            # their own flat buffers and optimizer, reduced only over the replicas of the same experts.
            self.flat_expert, self.optimizer_expert = None, None
            expert_params = [p for p in params if getattr(p, "expert_parallel", False)]
            if expert_params and mpu.get_expert_parallel_world_size() > 1:
                if mpu.get_expert_parallel_world_size() != self.dp_size:
                    raise NotImplementedError("expert parallel degree must equal the data parallel degree (or 1)")
                params = [p for p in params if not getattr(p, "expert_parallel", False)]
                self.flat_expert = FlatBuffers(expert_params, grad_dtype=torch.float32, pad_to=64)
                self.optimizer_expert = FusedAdamW(self.flat_expert, lr=a.learning_rate,
                                                   betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                                                   weight_decay=a.weight_decay, max_grad_norm=a.max_grad_norm)
            pad = 64 * self.dp_size
            # Fused data-parallel step over peer-mapped flat buffers (bf16 training on one node);
            # it shards the optimizer state exactly as ZeRO-1 does, so it also sets ``self.zero``.
            self.fused_dp = None
            if self.dp_size > 1 and self.device.type == "cuda" and params[0].dtype == torch.bfloat16:
                from ..parallel.dp_fused import FusedDataParallel
                self.fused_dp = FusedDataParallel.create(mpu.get_data_parallel_group(), self.device, a)
            self.flat = FlatBuffers(params, grad_dtype=torch.float32, pad_to=pad,
                                    allocator=self.fused_dp.allocator if self.fused_dp is not None else None)
            if self.fused_dp is not None:
                self.zero = True
                self.fused_dp.bind(self.flat, exclude_from_norm=self._norm_excluded_params())
            shard = None
            if self.zero:
                per = self.flat.numel // self.dp_size
                shard = (self.dp_rank * per, (self.dp_rank + 1) * per)
            self.optimizer = FusedAdamW(self.flat, lr=a.learning_rate, betas=(a.adam_beta1, a.adam_beta2),
                                        eps=a.adam_epsilon, weight_decay=a.weight_decay, shard=shard,
                                        max_grad_norm=a.max_grad_norm)
        else:
            inner = optimizer if optimizer is not None else optimizer_factory(params)
            self.flat_expert, self.optimizer_expert, self.fused_dp = None, None, None
            low_precision = params[0].dtype in (torch.bfloat16, torch.float16)
            if (self.zero or low_precision) and isinstance(inner, torch.optim.Optimizer):
                # a user optimizer gets fp32 master weights (bf16 / fp16 parameters) and, with
                # zero_stage 1, optimizer-state sharding on the same flat buffers the fused path uses
                # (Merak/core/zero/stage1.py:42-75, Merak/core/amp/fp16_optimizer.py:36-358)
                from ..zero.stage1 import ShardedMasterOptimizer
                self.optimizer = ShardedMasterOptimizer(
                    inner, dp_rank=self.dp_rank, dp_size=self.dp_size, shard=self.zero,
                    max_grad_norm=a.max_grad_norm, allow_untested=bool(a.zero_allow_untested_optimizer))
                self.flat = self.optimizer.flat
            else:
                self.optimizer = inner
                self.zero = False
        if getattr(self, "optimizer_expert", None) is not None:
            self.optimizer_expert.param_groups = self.optimizer.param_groups     # one learning-rate schedule
        self.lr_scheduler = lr_scheduler
        if self.lr_scheduler is None and lr_scheduler_factory is not None:
            # torch schedulers insist on a torch.optim.Optimizer: give them the wrapped one (the
            # parameter-group dicts, hence the learning rates, are shared)
            self.lr_scheduler = lr_scheduler_factory(getattr(self.optimizer, "optimizer", self.optimizer))

    def _norm_excluded_params(self) -> List[nn.Parameter]:
        """Parameters whose gradient this rank must not count in the global gradient norm: replicas of
        non-tensor-parallel parameters on tensor-parallel ranks other than 0, and tied weights on every
        stage but their first owner."""
        out = []
        tp_dup = mpu.get_model_parallel_world_size() > 1 and mpu.get_model_parallel_rank() != 0
        if tp_dup:
            out += [p for p in self._unique_params() if not getattr(p, "model_parallel", False)]
        for spec in getattr(self.module, "tied_local", {}).values():
            if self.stage_id != spec["stages"][0]:
                out.append(spec["param"])
        return out

    # ------------------------------------------------------------------------------------------
    # buffers
    # ------------------------------------------------------------------------------------------
    def _reset_buffers(self, n: int):
        self.num_buffers = n
        self.buf_inputs: List[Optional[Tuple[torch.Tensor, ...]]] = [None] * n      # carried from prev stage
        self.buf_externals: List[Dict[str, torch.Tensor]] = [dict() for _ in range(n)]
        self.buf_labels: List[Optional[torch.Tensor]] = [None] * n
        self.buf_outputs: List[Optional[Tuple[torch.Tensor, ...]]] = [None] * n
        self.buf_out_grads: List[Optional[List[torch.Tensor]]] = [None] * n
        self.buf_in_grads: List[Optional[List[torch.Tensor]]] = [None] * n
        self.buf_loss: List[Optional[torch.Tensor]] = [None] * n

    # ------------------------------------------------------------------------------------------
    # public API
    # ------------------------------------------------------------------------------------------
    def train(self):
        self.module.train()
        return self

    def eval(self):
        self.module.eval()
        return self

    def train_batch(self, data_iter: Iterator):
        """One optimizer step over ``gradient_accumulation_steps`` micro-batches.  Returns the loss
        averaged over micro-batches and data-parallel ranks (a device tensor on every rank)."""
        self.module.train()
        self.data_iter = data_iter
        self.total_loss = None
        self._grads_reduced = False
        self._bwd_done = 0
        if getattr(self, "_ov", None) is not None and not self._graph_capable():
            self._ov["used"] = False
        if getattr(self.args, "failure_detection_timeout", 0) and dist.is_initialized() and dist.get_world_size() > 1:
            if getattr(self, "_failure_detector", None) is None:
                from ..utils.failure import FailureDetector
                self._failure_detector = FailureDetector(timeout_s=float(self.args.failure_detection_timeout))
            self._failure_detector.step_barrier(self.global_steps)      # raises RankFailureError
            if self.device.type == "cuda":
                from ..utils.failure import check_device_status
                check_device_status()                                   # raises DeviceWaitTimeout
        if self.device.type == "cuda" and self.global_steps % 16 == 0:
            # a bounded device-side wait that ran out (peer flag, mbarrier) leaves a bit in the status
            # word; the results since then are invalid, so stop instead of training on
            from ..utils.failure import check_device_status
            check_device_status()
        if self.wall_clock_breakdown:
            self.timers("train_batch").start()
        if self._nvtx:
            torch.cuda.nvtx.range_push("train_batch %d" % self.global_steps)
        if self._graph_capable():
            self._train_batch_graphed()
        else:
            sched = S.make_schedule(self.args.train_schedule, self.micro_batches, self.num_stages, self.stage_id)
            if sched.num_pipe_buffers() != self.num_buffers:
                self._reset_buffers(sched.num_pipe_buffers())
            self._exec_schedule(sched)
        self.agg_loss = self._aggregate_total_loss()
        if self._nvtx:
            torch.cuda.nvtx.range_pop()
        if self.wall_clock_breakdown:
            self.timers("train_batch").stop()
        self.global_steps += 1
        dropout_state().advance_step()
        if self.args.logging_steps and self.global_steps % self.args.logging_steps == 0:
            self._log_step()
        return self.agg_loss

    def eval_batch(self, data_iter: Iterator, compute_loss: bool = True, reduce_output: Optional[str] = "avg",
                   num_micro_batches: Optional[int] = None, batch_fn: Optional[Callable] = None):
        """Forward-only pass over ``num_micro_batches`` micro-batches.  Returns the averaged loss; the
        list of last-stage outputs with ``compute_loss=False``; and with ``args.return_logits`` the triple
        ``(loss, logits, labels)`` whose lists hold one entry per micro-batch on the last stage and are
        empty elsewhere (reference: Merak/core/merak_engine.py:1271-1360)."""
        self.module.eval()
        self.data_iter = data_iter if batch_fn is None else (batch_fn(b) for b in data_iter)
        n = num_micro_batches or self.micro_batches
        self.total_loss = None
        self._eval_outputs: List[torch.Tensor] = []
        self._eval_labels: List = []
        self._compute_loss = compute_loss
        sched = S.InferenceSchedule(n, self.num_stages, self.stage_id)
        if sched.num_pipe_buffers() != self.num_buffers:
            self._reset_buffers(sched.num_pipe_buffers())
        # receive shapes may differ from training (e.g. generation): redo the handshake
        saved = (self._meta_sent, self._recv_act_meta)
        self._meta_sent, self._recv_act_meta = {"act": False, "grad": False}, None
        mb_saved = self.micro_batches
        self.micro_batches = n
        with torch.no_grad():
            self._exec_schedule(sched, training=False)
        self.micro_batches = mb_saved
        self._meta_sent, self._recv_act_meta = saved
        self._compute_loss = True
        if not compute_loss:
            return self._eval_outputs
        loss = self.total_loss if reduce_output is None else self._aggregate_total_loss(n)
        if self.args.return_logits:
            return loss, self._eval_outputs, self._eval_labels
        return loss

    # ------------------------------------------------------------------------------------------
    # CUDA-graph path (single pipeline stage): forward + backward of a micro-batch is captured once
    # and replayed, so the several hundred kernel launches of a step cost one graph launch
    # ------------------------------------------------------------------------------------------
    def _graph_capable(self) -> bool:
        return (bool(getattr(self.args, "cuda_graph", False)) and self.device.type == "cuda" and self.num_stages == 1
                and self.flat is not None and self.loss_scaler is None and not getattr(self, "_graph_failed", False)
                and getattr(self, "flat_expert", None) is None and not hasattr(self.module, "_has_moe"))

    def _graph_step_body(self, overlap: bool = False):
        ov = getattr(self, "_ov", None)
        overlap = overlap and ov is not None and self.micro_batches == 1
        if overlap:
            self._dp_overlap_begin()
            ov["armed"] = True
        out = self.module((), self._g_ext)
        loss = self.loss_fn(out, self._g_labels)
        loss = loss[0] if isinstance(loss, (tuple, list)) else loss
        (loss * (1.0 / self.micro_batches)).backward()
        if overlap:
            ov["armed"] = False
            self._dp_overlap_join()
        self._collect_main_grads()
        return loss.detach()

    def _graph_build(self, batch: Dict[str, torch.Tensor]):
        from ..ops import _lib
        self._g_ext = {k: torch.empty_like(batch[k], device=self.device) for k in self.stage_inputs if k in batch}
        label_keys = [k for k in batch if k not in self.input_names]
        lab = batch[label_keys[0]] if label_keys else None
        self._g_label_key = label_keys[0] if label_keys else None
        self._g_labels = torch.empty_like(lab, device=self.device) if lab is not None else None
        self._graph_copy_in(batch)
        self.module.current_buffer = 0
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):                      # eager warm-up: lazy initialisations happen here
                dropout_state().set_call_id(0)
                self._graph_step_body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.flat.zero_grad()
        dropout_state().set_call_id(0)
        graph = torch.cuda.CUDAGraph()
        before = _lib.launch_count()
        try:
            with torch.cuda.graph(graph):
                self._g_loss = self._graph_step_body(overlap=True)
        except Exception as exc:        # capture is an optimisation: fall back to eager execution
            log_dist("CUDA graph capture failed (%s); running eagerly" % str(exc).splitlines()[0], ranks=[-1])
            self._graph_failed = True
            self._graph = None
            torch.cuda.synchronize()
            self.flat.zero_grad()
            return False
        self._graph = graph
        self._graph_launches = _lib.launch_count() - before
        self.flat.zero_grad()
        return True

    def _graph_copy_in(self, batch: Dict[str, torch.Tensor]):
        for k, dst in self._g_ext.items():
            dst.copy_(batch[k], non_blocking=True)
        if self._g_labels is not None:
            self._g_labels.copy_(batch[self._g_label_key], non_blocking=True)

    def _train_batch_graphed(self):
        for mb in range(self.micro_batches):
            batch = _as_dict(next(self.data_iter), self.batch_names)
            if getattr(self, "_graph", None) is None:
                if not self._graph_build(batch):
                    # eager fallback for this and later steps
                    sched = S.make_schedule(self.args.train_schedule, self.micro_batches, 1, 0)
                    self._reset_buffers(sched.num_pipe_buffers())
                    import itertools
                    self.data_iter = itertools.chain([batch], self.data_iter)
                    self._exec_schedule(sched)
                    return
            self._graph_copy_in(batch)
            if mb > 0:
                dropout_state().advance_micro()     # the replay bakes its call ids in: move the offset
            self._graph.replay()
            self.graph_replay_launches = getattr(self, "graph_replay_launches", 0) + self._graph_launches
            det = self._g_loss.float().clone()
            self.total_loss = det if self.total_loss is None else self.total_loss + det
        self._training_pass = True
        self._exec_reduce_tied_grads()
        self._exec_reduce_grads()
        self._exec_optimizer_step()

    # ------------------------------------------------------------------------------------------
    # schedule execution
    # ------------------------------------------------------------------------------------------
    def _exec_schedule(self, sched, training: bool = True):
        self._training_pass = training
        table = {
            S.LoadMicroBatch: self._exec_load_micro_batch, S.ForwardPass: self._exec_forward_pass,
            S.BackwardPass: self._exec_backward_pass, S.SendActivation: self._exec_send_activations,
            S.RecvActivation: self._exec_recv_activations, S.SendGrad: self._exec_send_grads,
            S.RecvGrad: self._exec_recv_grads, S.SendActivationRecvGrad: self._exec_send_activations_recv_grads,
            S.SendGradRecvActivation: self._exec_send_grads_recv_activations,
            S.PreCheckpointForwardPass: self._exec_precheckpoint_forward_pass,
            S.RecomputeRecvGrad: self._exec_recompute_recv_grads,
            S.RestoreRecomputeStatus: self._exec_restore_recompute_status,
            S.ReduceTiedGrads: self._exec_reduce_tied_grads, S.ReduceGrads: self._exec_reduce_grads,
            S.OptimizerStep: self._exec_optimizer_step,
        }
        nvtx = self._nvtx
        for step_cmds in sched.steps():
            for cmd in step_cmds:
                fn = table[type(cmd)]
                if nvtx:                 # one range per pipeline instruction, named like the instruction
                    torch.cuda.nvtx.range_push("%s(%s)" % (type(cmd).__name__, cmd.kwargs.get("buffer_id", "")))
                try:
                    if "buffer_id" in cmd.kwargs:
                        fn(cmd.buffer_id)
                    else:
                        fn()
                finally:
                    if nvtx:
                        torch.cuda.nvtx.range_pop()

    # -- data ------------------------------------------------------------------------------------
    def _exec_load_micro_batch(self, buf: int):
        if self.wall_clock_breakdown:
            self.timers("batch_input").start()
        batch = _as_dict(next(self.data_iter), self.batch_names)
        moved = {}
        for k, v in batch.items():
            if isinstance(v, torch.Tensor):
                moved[k] = v.to(self.device, non_blocking=True)
        self.buf_externals[buf] = {k: moved[k] for k in self.stage_inputs if k in moved}
        if self.is_last:
            labels = {k: v for k, v in moved.items() if k not in self.input_names}
            self.buf_labels[buf] = labels.get("labels", next(iter(labels.values())) if labels else None)
            if len(labels) > 1:
                self.buf_labels[buf] = labels
        if self.wall_clock_breakdown:
            self.timers("batch_input").stop()

    def _load_middle_stage_inputs(self, buf: int):
        """Stages that are neither first nor last but read a model input themselves."""
        if self.stage_inputs and not self.is_first and not self.is_last:
            batch = _as_dict(next(self.data_iter), self.batch_names)
            self.buf_externals[buf] = {k: batch[k].to(self.device, non_blocking=True) for k in self.stage_inputs
                                       if k in batch}

    # -- compute ---------------------------------------------------------------------------------
    def _exec_forward_pass(self, buf: int):
        if self.wall_clock_breakdown:
            self.timers("forward").start()
        carried = self.buf_inputs[buf] if not self.is_first else ()
        carried = tuple(carried or ())
        self.module.current_buffer = buf
        out = self.module(carried, self.buf_externals[buf])
        self._collect_aux_loss(buf)
        if self.is_last:
            if not getattr(self, "_compute_loss", True) or (not self._training_pass and self.args.return_logits):
                self._eval_outputs.append(out.detach() if isinstance(out, torch.Tensor) else out)
                if getattr(self, "_compute_loss", True):
                    self._eval_labels.append(self.buf_labels[buf])
                if not getattr(self, "_compute_loss", True):
                    if self.wall_clock_breakdown:
                        self.timers("forward").stop()
                    return
            loss = self.loss_fn(out, self.buf_labels[buf]) if self.loss_fn is not None else out
            if isinstance(loss, (tuple, list)):
                loss = loss[0]
            self.buf_loss[buf] = loss
            det = loss.detach().float()
            self.total_loss = det if self.total_loss is None else self.total_loss + det
        else:
            self.buf_outputs[buf] = out if isinstance(out, tuple) else (out,)
        if self.wall_clock_breakdown:
            self.timers("forward").stop()

    def _collect_aux_loss(self, buf: int):
        """Auxiliary losses that layers of this stage left in ``module.aux_loss`` during the forward
        pass (router load balancing) are kept per pipeline buffer and join that buffer's backward."""
        mods = getattr(self, "_aux_modules", None)
        if mods is None:
            mods = self._aux_modules = [m for m in self.module.modules() if hasattr(m, "aux_loss_alpha")]
            self.buf_aux = {}
        total = None
        for m in mods:
            a = getattr(m, "aux_loss", None)
            if a is not None:
                total = a if total is None else total + a
                m.aux_loss = None
        if total is not None and self._training_pass:
            self.buf_aux[buf] = total

    def _exec_precheckpoint_forward_pass(self, buf: int):
        """Forward under ``pre_checkpoint``: every recompute segment registers a record that
        ``RecomputeRecvGrad`` can replay before the backward pass."""
        self.module.pending_records[buf] = []
        self.module.set_recompute(func=pre_checkpoint, interval=max(1, self.module.act_ckpt_interval or 1))
        self.rng_manager.store_fwd_rng_state(buf, self.device.type)
        self._exec_forward_pass(buf)

    def _exec_restore_recompute_status(self):
        self.module.restore_recompute()

    def _exec_recompute_recv_grads(self, buf: int):
        """Post the receive of the output gradient, replay the forward of the pre-checkpointed
        segments of this buffer while it is in flight, then wait."""
        work = self._post_recv_grads(buf)
        if self.wall_clock_breakdown:
            self.timers("recompute").start()
        recs = self.module.pending_records.pop(buf, [])
        if recs:
            run_pending_recomputes(recs)
        if self.wall_clock_breakdown:
            self.timers("recompute").stop()
        if work is not None:
            work.wait()

    def _exec_backward_pass(self, buf: int):
        if self.wall_clock_breakdown:
            self.timers("backward").start()
        self._bwd_done = getattr(self, "_bwd_done", 0) + 1
        ov = getattr(self, "_ov", None)
        overlap = ov is not None and self._training_pass and self._bwd_done == self.micro_batches
        if overlap:                 # the last micro-batch: gradients become final as this pass walks back
            self._dp_overlap_begin()
            ov["armed"] = True
        if self.is_last:
            loss = self.buf_loss[buf]
            scale = 1.0 / self.micro_batches
            if self.loss_scaler is not None:
                scale *= self.loss_scaler.cur_scale
            aux = self.buf_aux.pop(buf, None)
            if aux is not None:
                loss = loss + aux.to(loss.dtype)
            (loss * scale).backward()
            self.buf_loss[buf] = None
        else:
            outs = self.buf_outputs[buf]
            grads = self.buf_out_grads[buf]
            pairs = [(o, g) for o, g in zip(outs, grads or []) if isinstance(o, torch.Tensor) and o.requires_grad]
            aux = self.buf_aux.pop(buf, None)
            if aux is not None and aux.requires_grad:
                scale = (1.0 / self.micro_batches) * (self.loss_scaler.cur_scale if self.loss_scaler is not None else 1.0)
                pairs.append((aux, torch.full_like(aux, scale)))
            if pairs:
                if getattr(self, "buf_out_meta", {}).pop(buf, None) is not None:
                    # freed outputs no longer match their gradients' shapes: call the engine directly
                    from torch.autograd import Variable
                    Variable._execution_engine.run_backward(
                        tensors=tuple(o for o, _ in pairs), grad_tensors=tuple(g for _, g in pairs), keep_graph=False,
                        create_graph=False, inputs=tuple(), allow_unreachable=True, accumulate_grad=True)
                else:
                    torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
            self.buf_outputs[buf] = None
            self.buf_out_grads[buf] = None
        if not self.is_first:
            ins = self.buf_inputs[buf] or ()
            self.buf_in_grads[buf] = [None if not isinstance(t, torch.Tensor) else t.grad if t.grad is not None else
                                      (torch.zeros_like(t) if t.is_floating_point() else None) for t in ins]
            self.buf_inputs[buf] = None
        if overlap:
            ov["armed"] = False
        self._collect_main_grads()
        self.module.pending_records.pop(buf, None)
        if self.wall_clock_breakdown:
            self.timers("backward").stop()

    def _collect_main_grads(self):
        """Gradients autograd produced as ``p.grad`` (PyTorch-path ops) move into the flat buffer."""
        if self.flat is None:
            return
        extra = self.flat_expert.params if getattr(self, "flat_expert", None) is not None else []
        for p in list(self.flat.params) + list(extra):
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None

    # -- p2p ---------------------------------------------------------------------------------------
    def _alloc_from_meta(self, meta, requires_grad_ok: bool):
        bufs = []
        for dtype, rg, shape in meta:
            t = torch.empty(shape, dtype=dtype, device=self.device)
            if requires_grad_ok and rg == 1 and t.is_floating_point():
                t.requires_grad_(True)
            bufs.append(t)
        return bufs

    def _exec_send_activations(self, buf: int):
        if self.is_last:
            return
        outs = self._wire_outputs(buf)
        if self.wall_clock_breakdown:
            self.timers("pipe_send_output").start()
        p2p.send_forward(outs)
        if self.wall_clock_breakdown:
            self.timers("pipe_send_output").stop()
        self._free_sent_outputs(buf)

    def _free_sent_outputs(self, buf: int):
        """``deallocate_pipeline_outputs``: after the activation has been sent this stage only needs the
        outputs' ``grad_fn``; their storage is released (Merak/core/pipeline/utils.py:113-150)."""
        if not getattr(self.args, "deallocate_pipeline_outputs", False):
            return
        from .utils import deallocate_output_tensor
        outs = self.buf_outputs[buf] or ()
        if not hasattr(self, "buf_out_meta"):
            self.buf_out_meta = {}
        self.buf_out_meta[buf] = [(tuple(o.shape), o.dtype) if isinstance(o, torch.Tensor) else None for o in outs]
        for o in outs:
            if isinstance(o, torch.Tensor) and o.requires_grad and o._base is None and o.numel() > 1:
                deallocate_output_tensor(o)

    def _grad_buffers_like(self, buf: int):
        """Receive buffers for the gradients of this buffer's floating-point outputs (shapes from
        before the outputs were freed, when they were)."""
        outs = self.buf_outputs[buf]
        meta = getattr(self, "buf_out_meta", {}).get(buf)
        res = []
        for i, o in enumerate(outs):
            if isinstance(o, torch.Tensor) and o.is_floating_point():
                shape, dtype = meta[i] if meta is not None else (tuple(o.shape), o.dtype)
                res.append(torch.empty(shape, dtype=dtype, device=o.device))
        return res

    def _wire_outputs(self, buf: int):
        """This buffer's stage outputs as the tensors that go to the next stage (Python numbers and devices that
        a graph cut left among them travel as tagged 0-dim tensors); sends their description once."""
        outs, kinds = p2p.to_wire([o.detach() if isinstance(o, torch.Tensor) else o for o in self.buf_outputs[buf]],
                                  self.device)
        self._ensure_act_meta_sent(outs, kinds)
        return outs

    def _ensure_act_meta_sent(self, outs, kinds=None):
        if not self._meta_sent["act"]:
            p2p.send_meta(outs, mpu.get_pipeline_model_parallel_next_rank(), self.device, kinds)
            self._meta_sent["act"] = True

    def _ensure_act_meta_recv(self):
        if self._recv_act_meta is None:
            self._recv_act_meta = p2p.recv_meta(mpu.get_pipeline_model_parallel_prev_rank(), self.device)

    def _exec_recv_activations(self, buf: int):
        if self.is_first:
            return
        self._load_middle_stage_inputs(buf)
        self._ensure_act_meta_recv()
        bufs = self._alloc_from_meta(self._recv_act_meta, self._training_pass)
        if self.wall_clock_breakdown:
            self.timers("pipe_recv_input").start()
        p2p.recv_forward(bufs)
        if self.wall_clock_breakdown:
            self.timers("pipe_recv_input").stop()
        self.buf_inputs[buf] = self._unwire_inputs(bufs)

    def _unwire_inputs(self, bufs):
        if all(kind < 10 for _, kind, _ in self._recv_act_meta):
            return tuple(bufs)
        return tuple(p2p.from_wire(bufs, self._recv_act_meta, self.device))

    def _grad_meta(self, buf: int):
        return [(o.dtype, False, tuple(o.shape)) for o in self.buf_outputs[buf] if isinstance(o, torch.Tensor)]

    def _exec_send_grads(self, buf: int):
        if self.is_first:
            return
        grads = [g for g in (self.buf_in_grads[buf] or []) if g is not None]
        if self.wall_clock_breakdown:
            self.timers("pipe_send_grad").start()
        p2p.send_backward(grads)
        if self.wall_clock_breakdown:
            self.timers("pipe_send_grad").stop()
        self.buf_in_grads[buf] = None

    def _post_recv_grads(self, buf: int):
        if self.is_last:
            return None
        outs = self.buf_outputs[buf]
        bufs = self._grad_buffers_like(buf)
        work = p2p.recv_backward(bufs, wait=False)
        it = iter(bufs)
        self.buf_out_grads[buf] = [next(it) if (isinstance(o, torch.Tensor) and o.is_floating_point()) else None
                                   for o in outs]
        return work

    def _exec_recv_grads(self, buf: int):
        if self.wall_clock_breakdown:
            self.timers("pipe_recv_grad").start()
        work = self._post_recv_grads(buf)
        if work is not None:
            work.wait()
        if self.wall_clock_breakdown:
            self.timers("pipe_recv_grad").stop()

    def _exec_send_activations_recv_grads(self, bufs):
        send_buf, recv_buf = bufs
        if self.is_last:
            return
        outs = self._wire_outputs(send_buf)
        routs = self.buf_outputs[recv_buf]
        gb = self._grad_buffers_like(recv_buf)
        if self.wall_clock_breakdown:
            self.timers("pipe_send_output_recv_grad").start()
        p2p.send_forward_recv_backward(outs, gb)
        if self.wall_clock_breakdown:
            self.timers("pipe_send_output_recv_grad").stop()
        self._free_sent_outputs(send_buf)
        it = iter(gb)
        self.buf_out_grads[recv_buf] = [next(it) if (isinstance(o, torch.Tensor) and o.is_floating_point()) else None
                                        for o in routs]

    def _exec_send_grads_recv_activations(self, bufs):
        send_buf, recv_buf = bufs
        if self.is_first:
            return
        self._load_middle_stage_inputs(recv_buf)
        self._ensure_act_meta_recv()
        grads = [g for g in (self.buf_in_grads[send_buf] or []) if g is not None]
        rb = self._alloc_from_meta(self._recv_act_meta, self._training_pass)
        if self.wall_clock_breakdown:
            self.timers("pipe_send_grad_recv_input").start()
        p2p.send_backward_recv_forward(grads, rb)
        if self.wall_clock_breakdown:
            self.timers("pipe_send_grad_recv_input").stop()
        self.buf_in_grads[send_buf] = None
        self.buf_inputs[recv_buf] = self._unwire_inputs(rb)

    # -- reductions --------------------------------------------------------------------------------
    def _exec_reduce_tied_grads(self):
        if self.wall_clock_breakdown:
            self.timers("backward_tied_allreduce").start()
        self.module.allreduce_tied_weight_gradients()
        self._reduce_sequence_parallel_grads()
        self._reduce_ulysses_grads()
        if self.wall_clock_breakdown:
            self.timers("backward_tied_allreduce").stop()

    def _reduce_sequence_parallel_grads(self):
        """Norm parameters inside a Megatron sequence-parallel region see only their rank's tokens."""
        if mpu.get_model_parallel_world_size() == 1:
            return
        group = mpu.get_model_parallel_group()
        for p in self.module.parameters():
            if getattr(p, "sequence_parallel", False):
                g = getattr(p, "main_grad", None)
                g = g if g is not None else p.grad
                if g is not None:
                    dist.all_reduce(g, group=group)

    def _reduce_ulysses_grads(self):
        """Under Ulysses sequence parallelism every rank of the sequence group saw a different slice
        of the tokens: parameter gradients are summed over that group."""
        n = mpu.get_sequence_parallel_world_size()
        if n == 1:
            return
        group = mpu.get_sequence_parallel_group()
        if self.flat is not None:
            dist.all_reduce(self.flat.grad, group=group)
            for p in self.flat.params:
                if getattr(p, "ulysses_replicated", False):
                    p.main_grad.div_(n)
        else:
            for p in self._unique_params():
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=group)
                    if getattr(p, "ulysses_replicated", False):
                        p.grad.div_(n)

    def _exec_reduce_grads(self):
        if self.wall_clock_breakdown:
            self.timers("backward_allreduce").start()
        self.allreduce_gradients()
        if self.wall_clock_breakdown:
            self.timers("backward_allreduce").stop()

    def allreduce_gradients(self, bucket_elems: Optional[int] = None):
        """DP gradient reduction: all-reduce (or, under ZeRO-1, reduce-scatter to the owning rank) of
        the flat fp32 gradient buffer in buckets; ``1/dp`` is folded into the optimizer's gradient
        scale instead of a separate pass (Merak/core/merak_engine.py:552-621)."""
        if self.dp_size == 1 or self._grads_reduced:
            return
        group = mpu.get_data_parallel_group()
        if self.flat is not None:
            if getattr(self, "fused_dp", None) is not None:
                ov = getattr(self, "_ov", None)
                if ov is not None and ov["used"]:
                    # what the backward pass did not send itself (the first layers) goes now
                    self._dp_overlap_join()
                    if ov["starts"][ov["next"]] > 0:
                        self.fused_dp.push_region(0, ov["starts"][ov["next"]])
                    self.fused_dp.reduce_scatter(staged=True)
                    ov["armed"] = False
                else:
                    self.fused_dp.reduce_scatter()
                self._grads_reduced = True
                return
            g = self.flat.grad
            pre = self._dp_pre_scale()
            if pre != 1.0:
                g.mul_(pre)
            if self.zero:
                self._reduce_scatter_inplace(g, g.numel() // self.dp_size, group)
            else:
                bucket = int(bucket_elems or self.args.zero_reduce_bucket_size or 5e8)
                for lo in range(0, g.numel(), bucket):
                    dist.all_reduce(g[lo:lo + bucket], group=group)
        else:
            grads = [p.grad for p in self._unique_params() if p.grad is not None]
            bucket, size = [], 0
            limit = int(bucket_elems or 5e8)
            for gr in grads + [None]:
                if gr is None or size + gr.numel() > limit:
                    if bucket:
                        flat = torch.cat([b.reshape(-1) for b in bucket])
                        flat.div_(self.dp_size)
                        dist.all_reduce(flat, group=group)
                        off = 0
                        for b in bucket:
                            b.copy_(flat[off:off + b.numel()].view_as(b))
                            off += b.numel()
                    bucket, size = [], 0
                if gr is not None:
                    bucket.append(gr)
                    size += gr.numel()
        self._grads_reduced = True

    def _dp_pre_scale(self) -> float:
        """Factor applied to the gradients before the data-parallel collective
        (``prescale_gradients`` / ``gradient_predivide_factor``, Merak/core/zero/stage1.py:614-668):
        prescaling divides by the group size up front, a predivide factor ``f`` divides by ``f`` up
        front and leaves ``f / dp`` for afterwards.  The fused kernels reduce in fp32 and fold
        ``1 / dp`` into the optimizer's gradient scale, so they ignore both."""
        if self.dp_size == 1 or getattr(self, "fused_dp", None) is not None or self.flat is None:
            return 1.0
        if getattr(self.args, "prescale_gradients", False):
            return 1.0 / self.dp_size
        f = float(getattr(self.args, "gradient_predivide_factor", 1.0) or 1.0)
        return 1.0 / f

    def _dp_post_scale(self) -> float:
        return 1.0 / (self.dp_size * self._dp_pre_scale()) if self.dp_size > 1 else 1.0

    def _zero_allgather(self):
        """Parameter all-gather of the unfused ZeRO-1 step in buckets of
        ``zero_allgather_bucket_size`` elements per rank (Merak/core/zero/stage1.py:734-757)."""
        group = mpu.get_data_parallel_group()
        per = self.optimizer.end - self.optimizer.start
        bucket = max(1, min(per, int(getattr(self.args, "zero_allgather_bucket_size", per) or per)))
        model = self.flat.model
        if bucket >= per:
            dist.all_gather_into_tensor(model, model[self.optimizer.start:self.optimizer.end].clone(), group=group)
            return
        tmp = torch.empty(self.dp_size * bucket, dtype=model.dtype, device=model.device)
        for lo in range(0, per, bucket):
            b = min(bucket, per - lo)
            src = model[self.optimizer.start + lo:self.optimizer.start + lo + b].clone()
            dist.all_gather_into_tensor(tmp[:self.dp_size * b], src, group=group)
            for k in range(self.dp_size):
                model[k * per + lo:k * per + lo + b].copy_(tmp[k * b:(k + 1) * b])

    # -- data-parallel reduction overlapped with the backward pass -----------------------------------
    def _setup_dp_overlap(self):
        """The backward pass finalises the flat gradient buffer from its end (last layer) towards
        its start.  Each local layer's input is watched (a tensor hook): when its gradient arrives,
        every later layer's parameter gradients are complete and their piece of the buffer is
        copied, on a side stream, into the staging buffers of the ranks that own it (copy engines
        over NVLink: no SM is taken from the backward pass).  After the backward pass the rest is
        sent and the reduce-scatter kernel sums local memory only.  The reference reduces everything after the last
        micro-batch (Merak/core/pipeline/schedule.py:246-250)."""
        self._ov = None
        if getattr(self, "fused_dp", None) is None or not getattr(self.args, "overlap_dp_reduce", True):
            return
        expert_parallel = mpu.get_expert_parallel_world_size() > 1 and \
            any(getattr(p, "expert_parallel", False) for p in self.module.parameters())
        if expert_parallel or mpu.get_model_parallel_world_size() > 1 or mpu.get_sequence_parallel_world_size() > 1 \
                or self.num_stages > 1:
            # The backward pass of an expert-parallel layer runs all-to-all kernels that wait for their peers.
            # With the gradient pushes of this overlap issued between them, the 27-layer DeepSeek-V2-Lite shape
            # on 4 GPUs stopped making progress (every rank in a bounded wait); without them it runs.  Until
            # that interaction is understood, the overlap is used where it was measured: pure data
            # parallelism, whose backward pass waits for no peer.  Tensor-, sequence- and pipeline-parallel
            # backward passes also contain kernels or collectives that wait for peers, so they reduce after
            # the backward pass.  (The same on every rank: the test reads the model and the topology only.)
            return
        layers = self.module.local_layers
        offset_of = {id(p): o for p, o in zip(self.flat.params, self.flat.offsets)}
        seen, firsts, owned = set(), [], []
        for layer in layers:
            mine = [p for p in layer.parameters() if id(p) in offset_of and id(p) not in seen]
            seen.update(id(p) for p in layer.parameters())
            firsts.append(min(offset_of[id(p)] for p in mine) if mine else None)
            owned.append(mine)
        starts, nxt = [0] * (len(layers) + 1), self.flat.numel
        starts[len(layers)] = self.flat.numel
        for i in reversed(range(len(layers))):
            if firsts[i] is not None:
                if firsts[i] > nxt:
                    return                  # parameters are not laid out in layer order: keep the serial path
                nxt = firsts[i]
            starts[i] = nxt
        self.fused_dp.enable_staging()
        self._ov = {"starts": starts, "owned": owned, "next": len(layers), "armed": False, "used": False,
                    "side": torch.cuda.Stream(device=self.device),
                    "min_elems": int(getattr(self.args, "dp_overlap_bucket_elems", 8 << 20))}
        self.module.layer_input_hook = self._watch_layer_input

    def _watch_layer_input(self, layer_idx: int, carried):
        for t in carried:
            if isinstance(t, torch.Tensor) and t.requires_grad:
                t.register_hook(lambda g, i=layer_idx: self._dp_overlap_flush(i + 1))
                return

    def _dp_overlap_begin(self):
        ov = self._ov
        ov["next"], ov["used"] = len(self.module.local_layers), True

    def _dp_overlap_flush(self, upto: int, force: bool = False):
        """Layers ``upto ..`` have all their gradients: send the not yet sent part of them."""
        ov = self._ov
        if ov is None or not ov["armed"] or upto >= ov["next"]:
            return None
        lo, hi = ov["starts"][upto], ov["starts"][ov["next"]]
        if hi - lo < ov["min_elems"] and not force:
            return None                     # too small to be worth its copies: wait for more layers
        for i in range(upto, ov["next"]):
            for p in ov["owned"][i]:
                if p.grad is not None:      # a gradient autograd produced itself joins the flat buffer first
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                    p.grad = None
        ov["next"] = upto
        if hi <= lo:
            return None
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)
        ov["side"].wait_event(ev)
        with torch.cuda.stream(ov["side"]):
            self.fused_dp.push_region(lo, hi)
        return None

    def _dp_overlap_join(self):
        """The side stream's pieces are done before anything later on the current stream."""
        if self._ov is not None and self._ov["used"]:
            torch.cuda.current_stream().wait_stream(self._ov["side"])

    def _reduce_scatter_inplace(self, g: torch.Tensor, per: int, group):
        out = torch.empty(per, dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g, group=group)
        g[self.dp_rank * per:(self.dp_rank + 1) * per].copy_(out)

    # -- optimizer ---------------------------------------------------------------------------------
    def _global_grad_sumsq(self) -> torch.Tensor:
        """Squared gradient norm over the whole model: tensor-parallel duplicates counted once, then
        summed over the tensor- and pipeline-parallel groups (and dp under ZeRO)."""
        opt = self.optimizer
        ss = opt.grad_sumsq().clone()
        tp = mpu.get_model_parallel_world_size()
        lo, hi = (opt.start, opt.end) if self.zero else (0, self.flat.numel)
        offset_of = {id(p): o for p, o in zip(self.flat.params, self.flat.offsets)}

        def owned_sumsq(p):
            # ``ss`` covers [lo, hi) of the flat gradient buffer only (the reduce-scattered shard
            # under ZeRO-1): subtract the part of ``p`` inside it, never the unreduced remainder
            o = offset_of.get(id(p))
            if o is None:
                return None
            s, e = max(o, lo), min(o + p.numel(), hi)
            if s >= e:
                return None
            return self.flat.grad[s:e].float().pow(2).sum()

        if tp > 1 and mpu.get_model_parallel_rank() != 0:
            # replicated (non model-parallel) parameters are counted by tp rank 0 only
            for p in self.flat.params:
                if not getattr(p, "model_parallel", False):
                    v = owned_sumsq(p)
                    if v is not None:
                        ss[0] = ss[0] - v
        # a weight shared between stages (tied embeddings) is counted by its first owner only
        for spec in self.module.tied_local.values():
            already_excluded = tp > 1 and mpu.get_model_parallel_rank() != 0 and \
                not getattr(spec["param"], "model_parallel", False)
            if self.stage_id != spec["stages"][0] and not already_excluded:
                v = owned_sumsq(spec["param"])
                if v is not None:
                    ss[0] = ss[0] - v
        if self.zero:
            dist.all_reduce(ss, group=mpu.get_data_parallel_group())
        if tp > 1:
            dist.all_reduce(ss, group=mpu.get_model_parallel_group())
        if self.num_stages > 1:
            dist.all_reduce(ss, group=mpu.get_pipe_parallel_group())
        return ss

    def _exec_optimizer_step(self):
        if self.wall_clock_breakdown:
            self.timers("step").start()
        a = self.args
        grad_scale = self._dp_post_scale()
        if self.loss_scaler is not None:
            grad_scale /= self.loss_scaler.cur_scale
        if self.flat is not None:
            expert_ss = None
            if getattr(self, "optimizer_expert", None) is not None:
                # squared norm of the expert gradients of the whole expert-parallel group
                expert_ss = self.optimizer_expert.grad_sumsq().clone()
                dist.all_reduce(expert_ss, group=mpu.get_expert_parallel_group())
                if self.num_stages > 1:
                    dist.all_reduce(expert_ss, group=mpu.get_pipe_parallel_group())
            if getattr(self, "fused_dp", None) is not None:
                sumsq = None
                if mpu.get_model_parallel_world_size() > 1 or self.num_stages > 1 or expert_ss is not None:
                    sumsq = self.fused_dp.gathered_sumsq()
                    if mpu.get_model_parallel_world_size() > 1:
                        dist.all_reduce(sumsq, group=mpu.get_model_parallel_group())
                    if self.num_stages > 1:
                        dist.all_reduce(sumsq, group=mpu.get_pipe_parallel_group())
                    if expert_ss is not None:
                        sumsq = sumsq + expert_ss
                self.fused_dp.adamw_allgather(self.optimizer, grad_scale, sumsq)
            else:
                distributed_norm = (mpu.get_model_parallel_world_size() > 1 or self.num_stages > 1 or self.zero
                                    or expert_ss is not None)
                sumsq = self._global_grad_sumsq() if distributed_norm else None
                if expert_ss is not None:
                    sumsq = sumsq + expert_ss
                self.optimizer.step(grad_scale=grad_scale, sumsq=sumsq)
                if self.zero:
                    self._zero_allgather()
            if getattr(self, "optimizer_expert", None) is not None:
                self.optimizer_expert.step(grad_scale=grad_scale, sumsq=sumsq)
                self.flat_expert.zero_grad()
            if self.loss_scaler is not None:
                self.loss_scaler.update_scale(bool(self.optimizer.skipped().item()))
            self.flat.zero_grad()
        else:
            params = self._unique_params()
            if grad_scale != 1.0 and self.dp_size == 1:
                for p in params:
                    if p.grad is not None:
                        p.grad.mul_(grad_scale)
            if a.max_grad_norm and a.max_grad_norm > 0:
                torch.nn.utils.clip_grad_norm_(params, a.max_grad_norm)
            self.optimizer.step()
            self.optimizer.zero_grad(set_to_none=True)
        if self.lr_scheduler is not None:
            self.lr_scheduler.step()
        if self.wall_clock_breakdown:
            self.timers("step").stop()

    # -- loss --------------------------------------------------------------------------------------
    def _aggregate_total_loss(self, n_micro: Optional[int] = None) -> torch.Tensor:
        n = n_micro or self.micro_batches
        if self.is_last and self.total_loss is not None:
            loss = (self.total_loss / n).reshape(1).to(self.device)
            if self.dp_size > 1:
                dist.all_reduce(loss, group=mpu.get_data_parallel_group())
                loss /= self.dp_size
        else:
            loss = torch.zeros(1, dtype=torch.float32, device=self.device)
        if self.num_stages > 1:
            src = mpu.get_grid().stage_to_global(self.num_stages - 1)
            dist.broadcast(loss, src, group=mpu.get_pipe_parallel_group())
        return loss.squeeze(0)

    def _log_step(self):
        lr = self.get_lr()
        elapsed = self.timers("train_batch").elapsed(reset=True) / 1000.0 if self.wall_clock_breakdown else float("nan")
        steps = self.args.logging_steps
        iter_time = elapsed / steps if steps else float("nan")
        tput = self.micro_batch_size * self.micro_batches * self.dp_size / iter_time if iter_time and iter_time > 0 else 0.0
        log_dist("steps: %d loss: %.4f iter time (s): %.3f total samples/sec: %.3f learning rate: %.3e" % (
            self.global_steps, float(self.agg_loss), iter_time, tput, lr),
            ranks=[-1] if (self.is_last and self.dp_rank == 0 and mpu.get_model_parallel_rank() == 0) else [])
        if self.wall_clock_breakdown:
            self.timers.log(["batch_input", "forward", "backward", "recompute", "backward_allreduce",
                             "backward_tied_allreduce", "step", "pipe_send_output", "pipe_send_grad",
                             "pipe_recv_input", "pipe_recv_grad", "pipe_send_grad_recv_input",
                             "pipe_send_output_recv_grad"], normalizer=max(1, steps))
        see_memory_usage("after step %d" % self.global_steps, force=False)

    def get_lr(self) -> float:
        groups = getattr(self.optimizer, "param_groups", None)
        return groups[0]["lr"] if groups else float("nan")

    def set_lr(self, lr: float):
        for g in self.optimizer.param_groups:
            g["lr"] = lr
