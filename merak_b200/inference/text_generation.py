"""Autoregressive text generation on top of the pipeline engine
(Merak/inference/text_generation_inference.py:35-400).

Every new token runs the current sequence through all pipeline stages with ``eval_batch`` (the
reference does the same: there is no KV cache across pipeline stages); the last stage gathers the
vocabulary shards when the head is vocab-parallel, filters the logits (temperature, top-k,
top-p), samples, and broadcasts the token and the "done" flag to every rank.  Filtering and
sampling stay on the device; the only host read per token is the done flag.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..parallel import mpu


def top_k_top_p_filter(logits: torch.Tensor, top_k: int = 0, top_p: float = 0.0,
                       filter_value: float = -float("inf")) -> torch.Tensor:
    """Keeps the ``top_k`` highest logits and/or the smallest set whose probability mass exceeds
    ``top_p``; everything else becomes ``filter_value``.  ``logits`` is ``[batch, vocab]``."""
    logits = logits.clone()
    if top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.shape[-1]))[0][..., -1, None]
        logits[logits < kth] = filter_value
    if top_p > 0.0:
        sorted_logits, sorted_idx = torch.sort(logits, descending=True, dim=-1)
        cum = torch.cumsum(F.softmax(sorted_logits, dim=-1), dim=-1)
        remove = cum > top_p
        remove[..., 1:] = remove[..., :-1].clone()
        remove[..., 0] = False
        mask = torch.zeros_like(remove).scatter(-1, sorted_idx, remove)
        logits[mask] = filter_value
    return logits


def sample_next_token(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0,
                      greedy: bool = False, generator: Optional[torch.Generator] = None,
                      uniforms: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Next token per row of ``logits`` ``[batch, vocab]``.  On CUDA with ``1 <= top_k <= 1024`` the whole
    chain (temperature, top-k, top-p, softmax, draw) is one kernel launch (``csrc/sampling.cu``); other
    settings and CPU tensors take the PyTorch formulation.  ``uniforms`` (one number in [0, 1) per row)
    fixes the draw."""
    if greedy or temperature <= 0:
        return logits.argmax(-1)
    if logits.is_cuda and 1 <= top_k <= 1024 and logits.dtype in (torch.float32, torch.bfloat16) and logits.dim() == 2:
        from ..ops import _lib
        x = logits if logits.stride(1) == 1 else logits.contiguous()
        if uniforms is None:
            uniforms = torch.rand(x.shape[0], device=x.device, generator=generator)
        out = torch.empty(x.shape[0], dtype=torch.long, device=x.device)
        _lib.check(_lib.kernels().mrk_sample_topk_topp(
            x.data_ptr(), int(x.dtype == torch.bfloat16), x.shape[0], x.shape[1], x.stride(0), int(top_k), float(top_p),
            float(temperature), 0, uniforms.float().contiguous().data_ptr(), 0, 0, out.data_ptr(), None,
            _lib.stream_ptr()), "mrk_sample_topk_topp")
        return out
    logits = top_k_top_p_filter(logits.float() / temperature, top_k, top_p)
    probs = F.softmax(logits, dim=-1)
    if uniforms is not None:             # inverse CDF over the descending order, like the kernel
        sp, si = torch.sort(probs, descending=True, dim=-1, stable=True)
        pick = (torch.cumsum(sp, -1) <= uniforms[:, None].to(sp.dtype)).sum(-1).clamp(max=probs.shape[-1] - 1)
        return si.gather(-1, pick[:, None]).squeeze(-1)
    return torch.multinomial(probs, 1, generator=generator).squeeze(-1)


class text_generation_pipeline:
    """``text_generation_pipeline(engine_or_trainer, args, tokenizer)``; ``generate(prompts)`` returns
    token ids (and text when a tokenizer is given); ``generate_samples_interactive()`` is a REPL."""

    def __init__(self, model, args, tokenizer=None, eos_token_id: Optional[int] = None):
        from ..trainer import MerakTrainer
        self.engine = model.init_engine() if isinstance(model, MerakTrainer) else model
        self.args = args
        self.tokenizer = tokenizer
        self.eos = eos_token_id if eos_token_id is not None else getattr(tokenizer, "eos_token_id", None)
        self.device = self.engine.device

    def _last_rank(self) -> int:
        """The rank every other rank takes the new token from: the last global rank, which sits on
        the last pipeline stage (the pipeline axis is the outermost one), as in the reference
        (Merak/inference/text_generation_inference.py:238-270).  Every rank must name the same one."""
        return dist.get_world_size() - 1 if dist.is_initialized() else 0

    @torch.no_grad()
    def generate(self, prompts, max_new_tokens: Optional[int] = None, greedy: bool = False, seed: Optional[int] = None):
        a = self.args
        if self.tokenizer is not None and isinstance(prompts[0], str):
            ids = [self.tokenizer.encode(p) for p in prompts]
        else:
            ids = [list(p) for p in prompts]
        assert len({len(x) for x in ids}) == 1, "prompts of one call must have equal length"
        tokens = torch.tensor(ids, dtype=torch.long, device=self.device)
        max_len = min(a.out_seq_length, getattr(a, "seq_length", None) or a.out_seq_length)
        budget = max_new_tokens if max_new_tokens is not None else max_len - tokens.shape[1]
        gen = None
        if seed is not None:
            gen = torch.Generator(device=self.device)
            gen.manual_seed(seed)
        done = torch.zeros(tokens.shape[0], dtype=torch.bool, device=self.device)
        last = self._last_rank()
        engine = self.engine
        name = engine.input_names[0]
        for _ in range(max(0, budget)):
            outs = engine.eval_batch(iter([{name: tokens}]), compute_loss=False, num_micro_batches=1)
            nxt = torch.zeros(tokens.shape[0], dtype=torch.long, device=self.device)
            if engine.is_last:
                logits = outs[0]
                logits = logits[0] if isinstance(logits, (tuple, list)) else logits
                step_logits = logits[:, -1, :]
                tp = mpu.get_model_parallel_world_size()
                if tp > 1 and getattr(a, "parallel_vocab", False):
                    parts = [torch.empty_like(step_logits) for _ in range(tp)]
                    dist.all_gather(parts, step_logits.contiguous(), group=mpu.get_model_parallel_group())
                    step_logits = torch.cat(parts, -1)
                nxt = sample_next_token(step_logits, a.temperature, getattr(a, "top_k", 0), getattr(a, "top_p", 0.0),
                                        greedy, gen)
            if dist.is_initialized() and dist.get_world_size() > 1:
                dist.broadcast(nxt, last)
            if self.eos is not None:
                nxt = torch.where(done, torch.full_like(nxt, self.eos), nxt)
                done = done | (nxt == self.eos)
            tokens = torch.cat([tokens, nxt[:, None]], dim=1)
            if self.eos is not None and bool(done.all()):
                break
        out_ids = tokens.tolist()
        if self.tokenizer is not None:
            return out_ids, [self.tokenizer.decode(x) for x in out_ids]
        return out_ids

    def generate_samples_interactive(self, print_frequency: int = 24):   # pragma: no cover - needs a terminal
        rank0 = not dist.is_initialized() or dist.get_rank() == 0
        while True:
            text = [""]
            if rank0:
                try:
                    text = [input("\nContext prompt (stop to exit) >>> ")]
                except EOFError:
                    text = ["stop"]
            if dist.is_initialized() and dist.get_world_size() > 1:
                dist.broadcast_object_list(text, 0)
            if text[0].strip() == "stop":
                return
            ids, decoded = self.generate([text[0]])
            if rank0:
                print("\nMerak:", decoded[0], flush=True)
