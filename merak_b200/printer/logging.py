"""Logger, rank-filtered logging and running metrics (Merak/core/printer/logging.py:20-116)."""
from __future__ import annotations

import logging
import sys
from typing import Iterable, Optional

import torch.distributed as dist


class LoggerFactory:
    @staticmethod
    def create_logger(name: str = "Merak", level=logging.INFO) -> logging.Logger:
        lg = logging.getLogger(name)
        if not lg.handlers:
            lg.setLevel(level)
            lg.propagate = False
            h = logging.StreamHandler(stream=sys.stdout)
            h.setFormatter(logging.Formatter("[%(asctime)s] [%(levelname)s] [%(filename)s:%(lineno)d] %(message)s"))
            lg.addHandler(h)
        return lg


logger = LoggerFactory.create_logger()


def log_dist(message: str, ranks: Optional[Iterable[int]] = None, level=logging.INFO):
    """Logs on the listed global ranks only (``None`` or ``[-1]``: every rank)."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    ranks = list(ranks) if ranks is not None else [-1]
    if not ranks:
        return
    if -1 in ranks or rank in ranks:
        logger.log(level, "[Rank %d] %s" % (rank, message))


class Metric:
    def __init__(self, name: str):
        self.name = name
        self.reset()

    def reset(self):
        self.total, self.count = 0.0, 0

    def update(self, value: float, n: int = 1):
        self.total += float(value) * n
        self.count += n

    @property
    def avg(self) -> float:
        return self.total / max(1, self.count)


class AccMetric:
    """Running means of several named metrics (used for evaluation accuracy)."""

    def __init__(self):
        self.metrics = {}

    def update(self, name: str, value: float, n: int = 1):
        self.metrics.setdefault(name, Metric(name)).update(value, n)

    def avg(self, name: str) -> float:
        return self.metrics[name].avg

    def reset(self):
        for m in self.metrics.values():
            m.reset()

    def summary(self) -> dict:
        return {k: m.avg for k, m in self.metrics.items()}
