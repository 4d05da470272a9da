"""Host-side rank-failure detection.

The reference has no failure handling beyond ``sys.exit(1)`` on checkpoint errors (Merak/core/
checkpoint/checkpoint.py:478-480); its recovery story is restart + ``--resume_from_checkpoint``.
This module adds the detection half so that a job whose worker died stops with a typed error
instead of hanging in the next collective:

* every rank runs a heartbeat thread that bumps a counter in the process group's key-value store;
* :meth:`FailureDetector.step_barrier` is called between optimizer steps, before anything is
  launched: it publishes this rank's step and waits until every peer has published the same step.
  A peer whose heartbeat counter has not moved for ``timeout_s`` (or a store that stopped answering:
  rank 0 hosts it) raises :class:`RankFailureError` naming the ranks;
* device-side waits are bounded on their own (status word, see ``ops._lib.status``);
  :func:`check_device_status` turns a non-zero word into :class:`DeviceWaitTimeout`.

Ranks leave only between steps with nothing in flight, so survivors never sit in a collective with a
dead peer.  Recovery is a relaunch that resumes from the last checkpoint.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional

import torch.distributed as dist


class RankFailureError(RuntimeError):
    def __init__(self, ranks: List[int], detail: str = ""):
        self.ranks = list(ranks)
        super().__init__("rank(s) %s stopped responding%s" % (self.ranks, (": " + detail) if detail else ""))


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait (mbarrier or peer flag) ran out; the step's result is invalid."""


def check_device_status(clear: bool = True):
    from ..ops import _lib
    word = _lib.status(clear=clear)
    if word:
        names = [n for bit, n in ((1, "mbarrier wait"), (2, "peer-flag wait"), (4, "bad kernel argument")) if word & bit]
        raise DeviceWaitTimeout("device status word 0x%x (%s)" % (word, ", ".join(names) or "unknown"))


class FailureDetector:
    def __init__(self, store=None, rank: Optional[int] = None, world_size: Optional[int] = None,
                 interval_s: float = 0.5, timeout_s: float = 10.0, prefix: str = "merak_fd"):
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world_size is None else world_size
        self.interval, self.timeout, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._beats = 0
        self._seen: Dict[int, tuple] = {}          # peer -> (last counter value, local time it changed)
        self._thread = threading.Thread(target=self._run, name="merak-heartbeat", daemon=True)
        self._beat()
        self._thread.start()

    # -- heartbeat -------------------------------------------------------------------------------
    def _key(self, kind: str, rank: int) -> str:
        return "%s/%s/%d" % (self.prefix, kind, rank)

    def _beat(self):
        self._beats += 1
        self.store.set(self._key("hb", self.rank), str(self._beats))

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                self._beat()
            except Exception:
                return          # the store is gone: step_barrier reports it

    def stop(self):
        self._stop.set()

    # -- observation -----------------------------------------------------------------------------
    def _read(self, kind: str, rank: int) -> Optional[int]:
        key = self._key(kind, rank)
        if not self.store.check([key]):
            return None
        return int(self.store.get(key).decode())

    def stale_peers(self) -> List[int]:
        """Peers whose heartbeat counter has not changed for ``timeout_s`` of local time."""
        now, dead = time.monotonic(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read("hb", r)
            last = self._seen.get(r)
            if last is None or last[0] != v:
                self._seen[r] = (v, now)
            elif now - last[1] > self.timeout:
                dead.append(r)
        return dead

    def step_barrier(self, step: int, poll_s: float = 0.05):
        """Publishes ``step`` and returns once every peer has published it too; raises
        :class:`RankFailureError` if one of them stops beating first."""
        try:
            self.store.set(self._key("step", self.rank), str(step))
            while True:
                behind = []
                for r in range(self.world):
                    if r != self.rank:
                        seen = self._read("step", r)
                        if seen is None or seen < step:
                            behind.append(r)
                if not behind:
                    return
                dead = [r for r in self.stale_peers() if r in behind]
                if dead:
                    if self.rank == 0:
                        # rank 0 hosts the store: keep it up long enough for the other survivors to
                        # reach the same verdict before this process unwinds
                        time.sleep(self.timeout)
                    raise RankFailureError(dead, "no heartbeat for %.1f s before step %d" % (self.timeout, step))
                time.sleep(poll_s)
        except RankFailureError:
            raise
        except Exception as exc:          # the store lives on rank 0
            if self.rank != 0:
                raise RankFailureError([0], "key-value store unreachable (%s)" % type(exc).__name__) from exc
            raise
