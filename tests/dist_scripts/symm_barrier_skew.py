"""Two ranks map each other's control blocks; rank 1 arrives late at every barrier.  Each barrier
must complete without a timeout, and a reduce-scatter right after it must see the peer's data."""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from merak_b200.ops import _lib
from merak_b200.parallel.symm import SymmGroup


def main():
    out = sys.argv[1]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, n = dist.get_rank(), dist.get_world_size()
    sg = SymmGroup.create(dist.group.WORLD, dev)
    assert sg is not None, "peer mapping unavailable"
    numel = 64 * n * 1024
    gbuf = sg.alloc(numel * 4, torch.float32)
    g = gbuf.tensor[:numel]
    lib = _lib.kernels()
    ok = True
    for it in range(4):
        g.fill_(float(rank + 1 + it))
        torch.cuda.synchronize()
        if rank == 1:
            time.sleep(0.4)                     # deliberately late
        per = numel // n
        _lib.check(lib.mrk_dp_reduce_scatter(gbuf.table, sg.ctrl.table, n, rank, rank * per, per, None, it + 1, 1, 5000,
                                             _lib.stream_ptr()), "rs")
        sg.barrier(which=9, budget_ms=5000)    # nobody refills its buffer while a peer still reads it
        torch.cuda.synchronize()
        want = float(sum(r + 1 + it for r in range(n)))
        ok = ok and bool((g[rank * per:(rank + 1) * per] == want).all())
    status = _lib.status()
    res = torch.tensor([1 if (ok and status == 0) else 0], device=dev)
    dist.all_reduce(res, op=dist.ReduceOp.MIN)
    if rank == 0:
        with open(out, "w") as f:
            json.dump({"ok": int(res.item()), "status": status}, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
