"""merak_b200: automated 3D-parallel (data / tensor / pipeline, plus sequence and expert) training
for B200, with the public API of Merak: ``init``, ``MerakArguments``, ``MerakTrainer``."""
from .args import MerakArguments, get_args, manual_set_args, mergeargs, parse_args
from .initialize import get_grid, get_topo, init, print_rank_0
from .utils.device_to_meta import init_empty_weights

__version__ = "0.1.0"


def __getattr__(name):
    if name == "MerakTrainer":
        from .trainer import MerakTrainer
        return MerakTrainer
    if name == "mpu":
        from .parallel import mpu
        return mpu
    raise AttributeError(name)


__all__ = ["MerakTrainer", "init", "get_grid", "get_args", "get_topo", "MerakArguments", "print_rank_0",
           "init_empty_weights", "mpu"]
