"""``import Merak``: the ``merak_b200`` API under the reference's package name AND module paths, so
that scripts written against the reference import unchanged:

    import Merak
    from Merak import MerakArguments, MerakTrainer, init_empty_weights, print_rank_0
    from Merak.utils.datasets import DynamicGenDataset
    from Merak.core import mpu
    from Merak.core.printer import AccMetric, logger
    from Merak.core.tensor_parallel.mp_attrs import set_tp_layer_lists
    from Merak.inference import text_generation_pipeline

No code lives here.  A meta-path finder resolves every ``Merak.<path>`` import through the table below:
an entry with ONE source module is that module itself (one object under two names, so state such as
the process grid is shared); an entry with several sources is a package-like namespace holding the
public names of all of them, the way the reference's ``__init__`` files re-export their sub-modules
(e.g. Merak/core/mpu/__init__.py:1-43).  A path below a single-source package that the table does not
list is translated by prefix (``Merak.core.printer.timer`` -> ``merak_b200.printer.timer``).
"""
import importlib
import importlib.abc
import importlib.machinery
import sys
import types

from merak_b200 import *  # noqa: F401,F403
from merak_b200 import MerakArguments, get_args, get_grid, get_topo, init, init_empty_weights, print_rank_0

_P = "merak_b200."
# reference module path (below ``Merak.``) -> source modules (below ``merak_b200.``)
_TABLE = {
    "initialize": ["initialize"],
    "merak_trainer": ["trainer"],
    "merak_args": ["args"],
    "merak_args.args": ["args"],
    "utils": ["utils.device_to_meta", "utils.trainer_utils"],
    "utils.datasets": ["utils.datasets"],
    "utils.device_to_meta": ["utils.device_to_meta"],
    "utils.trainer_utils": ["utils.trainer_utils"],
    "utils.parameters": ["utils.trainer_utils"],                 # BaseParams
    "inference": ["inference"],
    "inference.text_generation_inference": ["inference.text_generation"],
    "core": ["pipeline.engine", "pipeline.module"],              # PipelineEngine, PipelineModule (+ sub-packages)
    "core.merak_engine": ["pipeline.engine"],
    "core.mpu": ["parallel.mpu", "parallel.layers", "parallel.mappings", "parallel.utils", "parallel.cross_entropy"],
    "core.mpu.initialize": ["parallel.mpu"],
    "core.mpu.layers": ["parallel.layers"],
    "core.mpu.mappings": ["parallel.mappings"],
    "core.mpu.utils": ["parallel.utils"],
    "core.mpu.cross_entropy": ["parallel.cross_entropy"],
    "core.mpu.topology": ["parallel.topology"],
    "core.mpu.p2p_communication": ["parallel.p2p"],
    "core.printer": ["printer"],
    "core.recompute": ["recompute"],
    "core.checkpoint": ["checkpoint"],
    "core.pipeline": ["pipeline.module", "pipeline.schedules", "pipeline.partition"],
    "core.pipeline.module": ["pipeline.module"],
    "core.pipeline.schedule": ["pipeline.schedules"],
    "core.pipeline.exec_schedule": ["pipeline.schedules"],
    "core.pipeline.layers_partition": ["pipeline.partition"],
    "core.pipeline.module_utils": ["pipeline.partition"],
    "core.pipeline.profiler": ["pipeline.profiler"],
    "core.pipeline.utils": ["pipeline.utils"],
    "core.fx": ["fx.convert", "fx.shard"],
    "core.fx.convert": ["fx.convert"],
    "core.fx.tracer": ["fx.tracer", "fx.export_trace"],
    "core.fx.graph_shard": ["fx.shard", "fx.split"],
    "core.tensor_parallel": ["parallel.tp_transform", "parallel.tp_overlap"],
    "core.tensor_parallel.mp_attrs": ["parallel.tp_transform"],
    "core.tensor_parallel.mp_layers": ["parallel.tp_transform"],
    "core.tensor_parallel.mp_mapping": ["parallel.tp_transform"],
    "core.tensor_parallel.model_parallel": ["parallel.tp_transform"],
    "core.tensor_parallel.transformer_blocks": ["parallel.tp_overlap"],
    "core.zero": ["zero"],
    "core.amp": ["amp"],
    "core.amp.amp_engine": ["amp"],
    "core.amp.fp16_optimizer": ["amp"],
    "core.finetuning": [],
    "core.finetuning.lora": ["lora"],
    "core.sequence_parallel": ["parallel.ulysses"],
    "core.sequence_parallel.operation": ["parallel.ulysses"],
    "core.sequence_parallel.modeling": [],
    "core.sequence_parallel.modeling.llama": ["parallel.ulysses"],
}
# names the reference spells differently: alias module -> {reference name: (source module, attribute)}
_RENAMED = {
    "core.mpu": {"LayerNorm": ("ops.modules", "LayerNorm")},
    "core.mpu.layers": {"LayerNorm": ("ops.modules", "LayerNorm")},
    "core.finetuning.lora": {"_find_and_replace": ("lora.utils", "find_and_replace")},
    "core.fx.tracer": {"tf_symbolic_trace": ("fx.tracer", "trace_model"), "LayerProxyTracer": ("fx.tracer", "MerakTracer")},
    "core.recompute": {"model_parallel_cuda_manual_seed": ("recompute.checkpointing", "model_parallel_manual_seed")},
}
# sub-packages that are attributes of an alias package (``from Merak.core import mpu``)
_CHILDREN = {"core": ["mpu", "recompute", "printer"]}


def _resolve(rel: str):
    """Source module names for the reference path ``rel``; None when nothing corresponds."""
    if rel in _TABLE:
        return _TABLE[rel]
    head = rel
    while "." in head:                                   # longest listed prefix that is one real package
        head = head.rsplit(".", 1)[0]
        if head in _TABLE and len(_TABLE[head]) == 1 and head not in _RENAMED:
            return [_TABLE[head][0] + rel[len(head):]]
    return None


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith("Merak."):
            return None
        rel = fullname[len("Merak."):]
        sources = _resolve(rel)
        if sources is None:
            raise ModuleNotFoundError("No module named %r (merak_b200 has no counterpart of this reference module)"
                                      % fullname, name=fullname)
        return importlib.machinery.ModuleSpec(fullname, self, is_package=True)

    def create_module(self, spec):
        rel = spec.name[len("Merak."):]
        sources = _resolve(rel)
        try:
            mods = [importlib.import_module(_P + s) for s in sources]
        except ModuleNotFoundError as exc:
            raise ModuleNotFoundError("No module named %r" % spec.name, name=spec.name) from exc
        has_children = any(k.startswith(rel + ".") for k in _TABLE)
        if len(mods) == 1 and rel not in _RENAMED and rel not in _CHILDREN and \
                (hasattr(mods[0], "__path__") or not has_children):
            return mods[0]                                # the module itself under a second name
        ns = types.ModuleType(spec.name, "Names of %s under the reference's module path." % ", ".join(m.__name__ for m in mods))
        ns.__path__ = []                                  # a package: its children come through this finder
        for m in mods:
            for k in getattr(m, "__all__", None) or [k for k in vars(m) if not k.startswith("_")]:
                ns.__dict__.setdefault(k, getattr(m, k))
        for name, (src, attr) in _RENAMED.get(rel, {}).items():
            setattr(ns, name, getattr(importlib.import_module(_P + src), attr))
        return ns

    def exec_module(self, module):
        rel = getattr(module.__spec__, "name", "")[len("Merak."):] if module.__name__.startswith("Merak.") else None
        for child in _CHILDREN.get(rel or "", []):
            setattr(module, child, importlib.import_module("Merak.%s.%s" % (rel, child)))


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())


def __getattr__(name):
    import merak_b200
    if name in ("core", "utils", "inference", "merak_args", "merak_trainer", "initialize"):
        return importlib.import_module("Merak." + name)
    return getattr(merak_b200, name)
