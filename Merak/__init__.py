"""Import alias: ``import Merak`` gives the ``merak_b200`` public API under the reference's name."""
from merak_b200 import *  # noqa: F401,F403
from merak_b200 import MerakArguments, get_args, get_grid, get_topo, init, init_empty_weights, print_rank_0


def __getattr__(name):
    import merak_b200
    return getattr(merak_b200, name)
