"""``init(pp, tp, dp, sp=1)``: bring up ``torch.distributed`` and the parallel grid.

Positional order is the reference's real one, ``init(pp, tp, dp, sp=1, backend='nccl')``
(Merak/initialize.py:36); keyword use (``init(dp=2, tp=2, pp=2)``) is accepted too.  Unlike the
reference, ``backend`` is honoured (``'gloo'`` runs the whole framework on CPU for tests), a
backend is chosen automatically when CUDA is absent, and an expert-parallel degree ``ep`` (a
divisor of ``dp``) can be given.
"""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist

from .parallel import mpu
from .parallel.topology import ParallelGrid, PipeDataSequenceModelParallelTopology


def init(pp: int = 1, tp: int = 1, dp: int = 1, sp: int = 1, backend: Optional[str] = None, ep: int = 1,
         timeout_s: Optional[float] = None):
    """Creates the process groups of a ``pp x dp x sp x tp`` grid (tp innermost) and registers them."""
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    world = pp * tp * dp * sp
    if not dist.is_initialized():
        if "RANK" not in os.environ:
            if world != 1:
                raise RuntimeError("init(pp=%d,tp=%d,dp=%d,sp=%d) needs %d processes; launch with torchrun"
                                   % (pp, tp, dp, sp, world))
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29512")
            os.environ.setdefault("LOCAL_RANK", "0")
            os.environ["RANK"] = "0"
            os.environ["WORLD_SIZE"] = "1"
        kwargs = {}
        if timeout_s is not None:
            kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
        if backend == "nccl":
            local = int(os.environ.get("LOCAL_RANK", os.environ.get("SLURM_LOCALID", "0")))
            torch.cuda.set_device(local)
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, **kwargs)
    if dist.get_world_size() != world:
        raise ValueError("pp*tp*dp*sp = %d but the job has %d ranks" % (world, dist.get_world_size()))
    topo = PipeDataSequenceModelParallelTopology(num_pp=pp, num_dp=dp, num_sp=sp, num_mp=tp)
    grid = ParallelGrid(topo, ep=ep)
    mpu.set_grid(grid, topo)
    return grid


def get_topo():
    return mpu.get_topo()


def get_grid():
    return mpu.get_grid()


def print_rank_0(*args, **kwargs):
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(*args, **kwargs, flush=True)


def destroy():
    mpu.destroy_model_parallel()
    if dist.is_initialized():
        dist.destroy_process_group()
