"""Step bookkeeping, samplers and loaders used by the trainer
(Merak/utils/parameters.py:31-136, Merak/utils/trainer_utils.py:24-115)."""
from __future__ import annotations

import math
from typing import Iterator, List, Optional

import torch


class BaseParams:
    """Batch-size and step arithmetic: ``total_batch_size = mbs * gas * dp``."""

    def __init__(self, args, dp_size: int):
        self.args = args
        self.mbs = args.per_device_train_batch_size
        self.gas = args.gradient_accumulation_steps
        self.dp = dp_size
        self.total_batch_size = self.mbs * self.gas * self.dp
        self.global_steps = 0
        self.epoch = 0
        self.step_in_epoch = 0
        self.max_steps = args.max_steps
        self.num_steps_per_epoch = None
        self.num_train_epochs = int(math.ceil(args.num_train_epochs))

    def train(self, num_micro_batches_per_epoch: Optional[int]):
        """``num_micro_batches_per_epoch``: length of this rank's micro-batch loader."""
        if num_micro_batches_per_epoch is not None:
            self.num_steps_per_epoch = max(1, num_micro_batches_per_epoch // self.gas)
        if self.max_steps and self.max_steps > 0:
            if self.num_steps_per_epoch:
                self.num_train_epochs = int(math.ceil(self.max_steps / self.num_steps_per_epoch))
        elif self.num_steps_per_epoch:
            self.max_steps = int(self.num_steps_per_epoch * self.args.num_train_epochs)
        return self.max_steps

    def resume(self, iteration: int):
        self.global_steps = iteration
        if self.num_steps_per_epoch:
            self.epoch = iteration // self.num_steps_per_epoch
            self.step_in_epoch = iteration % self.num_steps_per_epoch

    def step(self):
        self.global_steps += 1
        self.step_in_epoch += 1

    def should_break(self) -> bool:
        return bool(self.max_steps and self.max_steps > 0 and self.global_steps >= self.max_steps)

    def should_log(self) -> bool:
        return bool(self.args.logging_steps) and self.global_steps % self.args.logging_steps == 0

    def should_save(self) -> bool:
        return bool(self.args.save and self.args.save_steps) and self.global_steps % self.args.save_steps == 0


class MegatronPretrainingRandomSampler:
    """Data-parallel sharded random sampler: every epoch draws one permutation (seeded by the epoch)
    of the bucket of samples this dp rank owns and yields micro-batches of indices."""

    def __init__(self, total_samples: int, consumed_samples: int, micro_batch_size: int, data_parallel_rank: int,
                 data_parallel_size: int, seed: int = 0):
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.micro_batch_size = micro_batch_size
        self.rank, self.size = data_parallel_rank, data_parallel_size
        self.global_mb = micro_batch_size * data_parallel_size
        self.last_batch_size = total_samples % self.global_mb
        self.seed = seed
        assert total_samples > 0 and micro_batch_size > 0 and 0 <= data_parallel_rank < data_parallel_size

    def __len__(self):
        return (self.total_samples - self.last_batch_size) // self.global_mb

    def __iter__(self) -> Iterator[List[int]]:
        active = self.total_samples - self.last_batch_size
        epoch = self.consumed_samples // active
        within = self.consumed_samples % active
        bucket = active // self.size
        offset = within // self.size
        start = self.rank * bucket
        g = torch.Generator()
        g.manual_seed(self.seed + epoch)
        perm = torch.randperm(bucket, generator=g).tolist()
        idx = [start + x for x in perm[offset:]]
        batch = []
        for i in idx:
            batch.append(i)
            if len(batch) == self.micro_batch_size:
                self.consumed_samples += self.global_mb
                yield batch
                batch = []


class RepeatingLoader:
    """Restarts the wrapped loader when it is exhausted."""

    def __init__(self, loader):
        self.loader = loader
        self.it = iter(loader)

    def __iter__(self):
        return self

    def __len__(self):
        return len(self.loader)

    def __next__(self):
        try:
            return next(self.it)
        except StopIteration:
            self.it = iter(self.loader)
            return next(self.it)


class WorkerInitObj:
    def __init__(self, seed: int):
        self.seed = seed

    def __call__(self, worker_id: int):
        import random

        import numpy as np
        np.random.seed(self.seed + worker_id)
        random.seed(self.seed + worker_id)
