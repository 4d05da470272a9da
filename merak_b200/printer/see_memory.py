"""Device / host memory report (Merak/core/printer/see_memory.py:54-101)."""
from __future__ import annotations

import torch

from .logging import log_dist


def see_memory_usage(message: str, force: bool = False, ram: bool = False, ranks=(0,)):
    if not force:
        return
    parts = [message]
    if torch.cuda.is_available():
        gb = 1024 ** 3
        parts.append("MA %.2f GB | Max_MA %.2f GB | CA %.2f GB | Max_CA %.2f GB" % (
            torch.cuda.memory_allocated() / gb, torch.cuda.max_memory_allocated() / gb,
            torch.cuda.memory_reserved() / gb, torch.cuda.max_memory_reserved() / gb))
        torch.cuda.reset_peak_memory_stats()
    if ram:
        try:
            import psutil
            vm = psutil.virtual_memory()
            parts.append("CPU used %.2f GB (%.1f%%)" % ((vm.total - vm.available) / 1024 ** 3, vm.percent))
        except Exception:
            pass
    log_dist(" | ".join(parts), ranks=list(ranks))
