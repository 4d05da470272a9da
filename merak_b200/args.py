"""``MerakArguments``: the single configuration object of the framework.

Field-for-field the extra arguments of the reference's dataclass
(Merak/merak_args/args.py:37-676) on top of the Hugging-Face-``TrainingArguments``-style basics
the trainer consumes (batch size, accumulation, optimizer hyper-parameters, schedule, logging,
saving, precision).  It is a plain dataclass: importing it does not import ``transformers``.
``HfArgumentParser``-style command lines are parsed by :func:`parse_args`.

Module-level ``get_args()`` returns the arguments registered by the trainer
(``manual_set_args``), which is how deep components read configuration, as in the reference.
"""
from __future__ import annotations

import argparse
import dataclasses
import os
from dataclasses import dataclass, field, fields
from typing import Any, List, Optional

import torch


@dataclass
class MerakArguments:
    # ---- basics shared with HF TrainingArguments ----------------------------------------------
    output_dir: str = field(default="./output", metadata={"help": "Where checkpoints and logs go."})
    do_train: bool = True
    do_eval: bool = False
    per_device_train_batch_size: int = field(default=8, metadata={"help": "Micro-batch size per rank."})
    per_device_eval_batch_size: int = 8
    gradient_accumulation_steps: int = field(default=1, metadata={"help": "Micro-batches per optimizer step."})
    learning_rate: float = 5e-5
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    num_train_epochs: float = 3.0
    max_steps: int = -1
    lr_scheduler_type: str = "linear"
    warmup_ratio: float = 0.0
    warmup_steps: int = 0
    logging_steps: int = 500
    save_steps: int = 500
    eval_steps: Optional[int] = None
    eval_strategy: str = field(default="no", metadata={
        "help": "When to evaluate during training: no | steps (every eval_steps) | epoch.  do_eval=true alone means epoch."})
    evaluation_strategy: Optional[str] = field(default=None, metadata={"help": "Older spelling of eval_strategy."})
    seed: int = 42
    fp16: bool = False
    bf16: bool = False
    adafactor: bool = False
    dataloader_num_workers: int = 0
    dataloader_drop_last: bool = True
    resume_from_checkpoint: Optional[str] = None
    logging_dir: Optional[str] = None
    report_to: str = "tensorboard"
    local_rank: int = -1
    no_cuda: bool = False
    remove_unused_columns: bool = False

    # ---- pipeline / graph sharding --------------------------------------------------------------
    train_schedule: str = field(default="1f1b", metadata={
        "help": "1f1b | ds_default | pre_recompute_1f1b | last_no_recompute_1f1b | full_critical_path_1f1b "
                "(alias shifted_critical_path)"})
    partition_method: str = field(default="uniform_floor", metadata={
        "help": "uniform | uniform_floor | parameters | custom | autopipe"})
    split_method: str = field(default="nearest_min_deps", metadata={
        "help": "farthest_min_deps | nearest_min_deps | layer_split"})
    custom_split_points: Optional[List[str]] = None
    trace_method: str = field(default="fx", metadata={"help": "fx | dynamo | none"})
    trace_model: str = ""
    init_method_std: float = 0.02
    activation_checkpointing: bool = True
    checkpoint_num_layers: int = 1
    input_names: Optional[List[str]] = None
    num_layers: Optional[int] = None
    seq_length: Optional[int] = None
    hidden_size: Optional[int] = None
    num_heads: Optional[int] = None
    wall_clock_breakdown: bool = True
    shard_count: Optional[int] = None
    prescale_gradients: bool = False
    gradient_predivide_factor: float = 1.0
    cache_sharding: bool = False
    cache_name: Optional[str] = None
    return_logits: bool = False

    # ---- ZeRO / checkpointing ------------------------------------------------------------------
    zero_allow_untested_optimizer: bool = False
    zero_stage: Optional[int] = None
    zero_allgather_bucket_size: int = 500000000
    zero_reduce_bucket_size: int = 500000000
    save: bool = False
    finetune: bool = False
    no_save_rng: bool = False
    no_save_optim: bool = False
    no_load_optim: bool = False
    no_load_rng: bool = False
    split_inputs: bool = field(default=False, metadata={
        "help": "accepted for command-line compatibility; nothing reads it (the same holds for the reference, "
                "Merak/merak_args/args.py:344)"})
    save_total_limit: int = -1

    # ---- tensor / sequence parallel -------------------------------------------------------------
    parallel_vocab: bool = False
    sequence_parallel: bool = False
    sequence_dim: int = 1
    megatron_sequence_parallel: bool = field(default=False, metadata={
        "help": "Reduce-scatter / all-gather along the sequence inside the tensor-parallel group."})
    dealloc_pipeoutput: bool = False
    activation_checkpoint_ratio: Optional[List[str]] = None
    tp_overlapping_level: int = field(default=0, metadata={"help": "0..3: sub-pipelined tensor parallelism"})
    comm_mode: str = field(default="fused", metadata={
        "help": "fused: sm_100a kernels fused with their collectives over peer memory; "
                "nccl: plain torch.distributed collectives (baseline / oracle)"})
    deallocate_pipeline_outputs: bool = field(default=False, metadata={
        "help": "free a stage's output activations once they have been sent to the next stage"})
    failure_detection_timeout: float = field(default=0.0, metadata={
        "help": "> 0: heartbeat every rank through the process-group store and raise RankFailureError at the "
                "next step boundary when a peer has been silent for this many seconds"})

    # ---- mixed precision ------------------------------------------------------------------------
    half_precision_backend: str = "cuda_amp"
    loss_scale: float = 0.0
    initial_scale_power: int = 32
    loss_scale_window: int = 1000
    hysteresis: int = 2
    min_loss_scale: float = 1.0

    # ---- partition / tie / generation / LoRA -----------------------------------------------------
    custom_partition: Optional[List[int]] = None
    no_tie_modules: bool = False
    out_seq_length: int = 1024
    temperature: float = 0.9
    top_k: int = 0
    top_p: float = 0.9
    lora_config: Optional[str] = None
    adapter_name: str = "default"

    # ---- B200 runtime ---------------------------------------------------------------------------
    cuda_graph: bool = field(default=False, metadata={"help": "Capture each stage's micro-batch step in a CUDA graph."})
    nvtx_ranges: bool = field(default=False, metadata={
        "help": "emit an NVTX range per pipeline instruction and per train_batch (also MERAK_NVTX=1)"})
    overlap_dp_reduce: bool = field(default=True, metadata={"help": "Reduce DP gradients during the last backward."})
    dp_overlap_bucket_elems: int = field(default=8 << 20, metadata={
        "help": "smallest piece of the gradient buffer (elements) worth its own overlapped reduction launch"})

    # filled by the trainer
    params_dtype: Any = field(default=None, repr=False)
    use_cpu_initialization: bool = field(default=False, repr=False)

    def __post_init__(self):
        if self.train_schedule == "shifted_critical_path":
            self.train_schedule = "full_critical_path_1f1b"
        if not self.activation_checkpointing:
            self.checkpoint_num_layers = 0
        if self.dealloc_pipeoutput:        # the reference's name for the same switch (args.py:372)
            self.deallocate_pipeline_outputs = True
        if self.zero_stage not in (None, 0, 1):
            raise ValueError("zero_stage supports only 1 (optimizer-state sharding)")
        if self.tp_overlapping_level not in (0, 1, 2, 3):
            raise ValueError("tp_overlapping_level must be in 0..3")
        if self.half_precision_backend not in ("cuda_amp", "apex", "cpu_amp", "auto"):
            raise ValueError("half_precision_backend must be cuda_amp, apex or cpu_amp")
        if self.fp16 and self.bf16:
            raise ValueError("choose one of fp16 / bf16")
        if self.evaluation_strategy is not None:
            self.eval_strategy = self.evaluation_strategy
        self.eval_strategy = str(getattr(self.eval_strategy, "value", self.eval_strategy)).lower()
        if self.eval_strategy not in ("no", "steps", "epoch"):
            raise ValueError("eval_strategy must be no, steps or epoch")
        if self.eval_strategy == "no" and self.do_eval:
            self.eval_strategy = "epoch"
        self.do_eval = self.eval_strategy != "no"
        if self.eval_strategy == "steps" and not self.eval_steps:
            self.eval_steps = self.logging_steps          # as in Hugging Face's TrainingArguments
        if isinstance(self.activation_checkpoint_ratio, (str, float, int)):
            self.activation_checkpoint_ratio = [str(self.activation_checkpoint_ratio)]
        self._setup_devices()

    # -- device / rank helpers (Merak/merak_args/args.py:517-579) -----------------------------------
    def _setup_devices(self):
        if self.local_rank == -1:
            for key in ("LOCAL_RANK", "SLURM_LOCALID"):
                if key in os.environ:
                    self.local_rank = int(os.environ[key])
                    break
        self.use_cpu = self.no_cuda or not torch.cuda.is_available()

    @property
    def device(self) -> torch.device:
        if self.use_cpu:
            return torch.device("cpu")
        return torch.device("cuda", max(self.local_rank, 0))

    @property
    def train_batch_size(self) -> int:
        return self.per_device_train_batch_size

    @property
    def eval_batch_size(self) -> int:
        return self.per_device_eval_batch_size

    @property
    def compute_dtype(self) -> torch.dtype:
        if self.bf16:
            return torch.bfloat16
        if self.fp16:
            return torch.float16
        return torch.float32

    def get_lora_config(self):
        if not self.lora_config:
            return None
        from .lora.config import LoraConfig
        return LoraConfig.from_json_file(self.lora_config)

    def get_warmup_steps(self, num_training_steps: int) -> int:
        return self.warmup_steps if self.warmup_steps > 0 else int(num_training_steps * self.warmup_ratio)

    def main_process_first(self, local: bool = True, desc: str = "work"):
        """Context manager: rank 0 runs the body first, the others after a barrier."""
        import contextlib
        import torch.distributed as dist

        @contextlib.contextmanager
        def ctx():
            is_main = (self.local_rank in (-1, 0)) if local else (not dist.is_initialized() or dist.get_rank() == 0)
            if dist.is_initialized() and not is_main:
                dist.barrier()
            try:
                yield
            finally:
                if dist.is_initialized() and is_main:
                    dist.barrier()
        return ctx()

    def to_dict(self):
        d = dataclasses.asdict(self)
        d["params_dtype"] = str(d["params_dtype"])
        return d


_GLOBAL_ARGS: Optional[MerakArguments] = None


def manual_set_args(args: MerakArguments):
    """Registers ``args`` globally and derives ``params_dtype`` (bf16 is mapped, unlike the
    reference which only knows fp16/fp32 - Merak/merak_args/args.py:581-589)."""
    global _GLOBAL_ARGS
    args.params_dtype = args.compute_dtype
    args.use_cpu_initialization = True
    _GLOBAL_ARGS = args
    return args


def get_args() -> MerakArguments:
    if _GLOBAL_ARGS is None:
        raise RuntimeError("arguments are not initialised; construct a MerakTrainer or call manual_set_args")
    return _GLOBAL_ARGS


def has_args() -> bool:
    return _GLOBAL_ARGS is not None


_CONFIG_ALIASES = {
    "num_layers": ["num_hidden_layers", "n_layer", "num_layers", "encoder_layers", "n_layers"],
    "num_heads": ["num_attention_heads", "n_head", "num_heads", "encoder_attention_heads", "n_heads"],
    "hidden_size": ["hidden_size", "n_embd", "d_model", "dim"],
    "seq_length": ["max_position_embeddings", "n_positions", "max_seq_len", "max_source_positions"],
}


def mergeargs(training_args: MerakArguments, model_config) -> MerakArguments:
    """Fills model-derived fields from a (HF-style) model config
    (Merak/merak_args/args.py:598-676): layer count, heads, hidden size, sequence length and the
    default ``shard_count = 2*num_layers + 4``."""
    def lookup(cfg, names):
        for n in names:
            v = getattr(cfg, n, None)
            if isinstance(v, int) and not isinstance(v, bool):
                return v
            if isinstance(v, dict) and v and all(isinstance(x, int) for x in v.values()):
                return sum(v.values())      # LXMERT: {"vision": 5, "cross_encoder": 5, "language": 9}
        return None

    cfgs = [model_config]
    for sub in ("text_config", "vision_config", "encoder", "decoder"):
        c = getattr(model_config, sub, None)
        if c is not None and not isinstance(c, (int, str)):
            cfgs.append(c)
    for key, names in _CONFIG_ALIASES.items():
        if getattr(training_args, key) is None:
            vals = [lookup(c, names) for c in cfgs]
            vals = [v for v in vals if v is not None]
            if vals:
                setattr(training_args, key, sum(vals) if key == "num_layers" and len(vals) > 1 else vals[0])
    depths = getattr(model_config, "depths", None)
    if training_args.num_layers is None and depths is not None:
        training_args.num_layers = int(sum(depths))
    if training_args.num_layers is None:
        # three-stream configurations (LXMERT: language, cross-modality and region layers)
        streams = [getattr(model_config, k, None) for k in ("l_layers", "x_layers", "r_layers")]
        if all(isinstance(v, int) for v in streams):
            training_args.num_layers = sum(streams)
    if training_args.shard_count is None and training_args.num_layers is not None:
        training_args.shard_count = 2 * training_args.num_layers + 4
    return training_args


def print_args(args: MerakArguments, printer=print):
    printer("------------------------ MerakArguments ------------------------")
    for f in sorted(fields(args), key=lambda f: f.name):
        printer("  %s %s %s" % (f.name, "." * max(1, 40 - len(f.name)), getattr(args, f.name)))
    printer("-----------------------------------------------------------------")


def _str2bool(v):
    if isinstance(v, bool):
        return v
    if v.lower() in ("yes", "true", "t", "y", "1"):
        return True
    if v.lower() in ("no", "false", "f", "n", "0"):
        return False
    raise argparse.ArgumentTypeError("boolean value expected, got %r" % v)


def build_parser(cls=MerakArguments) -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    for f in fields(cls):
        if not f.repr or f.name in ("params_dtype", "use_cpu_initialization"):
            continue
        help_ = f.metadata.get("help", "")
        tp = f.type if not isinstance(f.type, str) else f.type
        tname = str(tp)
        default = f.default if f.default is not dataclasses.MISSING else None
        if "bool" in tname:
            parser.add_argument("--" + f.name, type=_str2bool, nargs="?", const=True, default=default, help=help_)
        elif "List[str]" in tname:
            parser.add_argument("--" + f.name, type=str, nargs="+", default=default, help=help_)
        elif "List[int]" in tname:
            parser.add_argument("--" + f.name, type=int, nargs="+", default=default, help=help_)
        elif "int" in tname:
            parser.add_argument("--" + f.name, type=int, default=default, help=help_)
        elif "float" in tname:
            parser.add_argument("--" + f.name, type=float, default=default, help=help_)
        else:
            parser.add_argument("--" + f.name, type=str, default=default, help=help_)
    return parser


def parse_args(argv=None, cls=MerakArguments, allow_extra: bool = False):
    """Command line -> ``MerakArguments`` (same flag names as the dataclass fields)."""
    parser = build_parser(cls)
    if allow_extra:
        ns, extra = parser.parse_known_args(argv)
        return cls(**vars(ns)), extra
    return cls(**vars(parser.parse_args(argv)))
