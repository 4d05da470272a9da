"""Two or more gloo ranks step in lockstep through FailureDetector.step_barrier; the rank named by
--die_rank leaves (os._exit) after --die_after steps, between steps.  Survivors write what they saw."""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from merak_b200.utils.failure import FailureDetector, RankFailureError


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--die_rank", type=int, default=-1)
    ap.add_argument("--die_after", type=int, default=2)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--out", required=True)
    o = ap.parse_args()
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    fd = FailureDetector(interval_s=0.1, timeout_s=1.5)
    result = {"rank": rank, "completed": 0, "error": None}
    t0 = time.monotonic()
    try:
        for step in range(o.steps):
            fd.step_barrier(step)
            x = torch.ones(4) * (rank + 1)
            dist.all_reduce(x)                     # the step's collective: every rank is known to be alive
            result["completed"] = step + 1
            if rank == o.die_rank and step + 1 == o.die_after:
                os._exit(17)                       # leaves between steps, nothing in flight
    except RankFailureError as exc:
        result["error"] = {"type": type(exc).__name__, "ranks": exc.ranks, "after_s": time.monotonic() - t0}
    with open("%s.%d" % (o.out, rank), "w") as f:
        json.dump(result, f)
    fd.stop()
    os._exit(0)      # do not wait for a peer that is gone


if __name__ == "__main__":
    main()
