"""Shared helpers of the example scripts: repository import path, parallel degrees from the
environment (``PP``, ``TP``, ``DP``, ``SP``, ``EP``; default: everything in data parallel) and a
``--model_size`` switch so every script also runs on a laptop CPU."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def degrees():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pp, tp = int(os.environ.get("PP", "1")), int(os.environ.get("TP", "1"))
    sp, ep = int(os.environ.get("SP", "1")), int(os.environ.get("EP", "1"))
    dp = int(os.environ.get("DP", str(max(1, world // (pp * tp * sp)))))
    return dict(pp=pp, tp=tp, dp=dp, sp=sp, ep=ep)


def parse(extra=None):
    """MerakArguments from the command line plus the example's own options (``extra``: name -> default)."""
    import argparse

    from merak_b200.args import MerakArguments, build_parser
    parser = build_parser(MerakArguments)
    fields = {f for f in MerakArguments.__dataclass_fields__}
    for k, v in (extra or {}).items():
        if k in fields:           # an example-specific default for a framework argument
            parser.set_defaults(**{k: v})
        else:
            parser.add_argument("--" + k, type=type(v) if v is not None else str, default=v)
    ns = parser.parse_args()
    own = {k: getattr(ns, k) for k in (extra or {})}
    args = MerakArguments(**{k: v for k, v in vars(ns).items() if k in fields})
    return args, argparse.Namespace(**own)
