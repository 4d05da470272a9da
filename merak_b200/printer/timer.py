"""Named timers for the per-instruction breakdown the engine logs
(Merak/core/printer/timer.py:21-123).

On CUDA each timer brackets its region with CUDA *events* on the current stream, so timing never
inserts a device-wide synchronisation into the step (the reference synchronises the device at
every start/stop); elapsed times are resolved when they are logged.  On CPU it is wall clock.
"""
from __future__ import annotations

import time
from typing import Dict, Iterable, List, Optional

import torch

from .logging import log_dist

_LOG_RANKS: List[int] = [0]


def set_timer_log_rank(ranks: Iterable[int]):
    _LOG_RANKS[:] = list(ranks)


class _Timer:
    def __init__(self, name: str):
        self.name = name
        self.started = False
        self.elapsed_ms = 0.0
        self._pairs = []
        self._t0 = 0.0
        self._ev0 = None
        self.count = 0

    def start(self):
        if self.started:
            return
        self.started = True
        if torch.cuda.is_available():
            self._ev0 = torch.cuda.Event(enable_timing=True)
            self._ev0.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self):
        if not self.started:
            return
        self.started = False
        self.count += 1
        if torch.cuda.is_available():
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            self._pairs.append((self._ev0, ev1))
        else:
            self.elapsed_ms += (time.perf_counter() - self._t0) * 1000.0

    def elapsed(self, reset: bool = True) -> float:
        """Milliseconds accumulated since the last reset."""
        if self._pairs:
            self._pairs[-1][1].synchronize()
            for a, b in self._pairs:
                self.elapsed_ms += a.elapsed_time(b)
            self._pairs = []
        v = self.elapsed_ms
        if reset:
            self.elapsed_ms, self.count = 0.0, 0
        return v


class SynchronizedWallClockTimer:
    def __init__(self):
        self.timers: Dict[str, _Timer] = {}

    def __call__(self, name: str) -> _Timer:
        if name not in self.timers:
            self.timers[name] = _Timer(name)
        return self.timers[name]

    def has(self, name: str) -> bool:
        return name in self.timers

    def log(self, names: Iterable[str], normalizer: float = 1.0, reset: bool = True, ranks: Optional[List[int]] = None):
        parts = []
        for n in names:
            if n in self.timers:
                parts.append("%s: %.2f" % (n, self.timers[n].elapsed(reset) / normalizer))
        if parts:
            log_dist("time (ms) | " + " | ".join(parts), ranks=ranks if ranks is not None else _LOG_RANKS)


class ThroughputTimer:
    """Samples/second over a window of steps."""

    def __init__(self, batch_size: int, start_step: int = 2):
        self.batch_size, self.start_step = batch_size, start_step
        self.steps, self.total_s, self._t0 = 0, 0.0, None

    def start(self):
        self._t0 = time.perf_counter()

    def stop(self):
        if self._t0 is None:
            return
        self.steps += 1
        if self.steps > self.start_step:
            self.total_s += time.perf_counter() - self._t0
        self._t0 = None

    def avg_samples_per_sec(self) -> float:
        n = self.steps - self.start_step
        return self.batch_size * n / self.total_s if n > 0 and self.total_s > 0 else 0.0
