"""Names that the reference implementation imports from ``transformers`` 4.x and that
``transformers`` 5.x no longer has, registered from outside the reference's own tree so that
the unmodified package under ``baseline/_ref`` imports.

* ``transformers.file_utils.cached_property`` / ``torch_only_method``
  (Merak/merak_args/args.py:29-32)
* ``transformers.utils.fx`` with ``HFTracer``, ``symbolic_trace``, ``_SUPPORTED_MODELS`` and
  ``_generate_supported_model_class_names`` (Merak/core/fx/convert.py:26,
  Merak/core/fx/tracer/_symbolic_trace.py:25, Merak/core/tensor_parallel/mp_mapping.py:18,
  Merak/core/tensor_parallel/utils.py:27).  The stub declares no supported Hugging Face model,
  so every model takes the reference's plain ``torch.fx`` path (Merak/core/fx/convert.py:72-85).
* ``transformers.modeling_utils.Conv1D`` (Merak/core/tensor_parallel/mp_attrs.py:22).

Nothing here touches the reference's code; it only fills ``sys.modules``.
"""
from __future__ import annotations

import functools
import sys
import types


def install() -> None:
    import torch.fx
    import transformers
    import transformers.file_utils as file_utils
    import transformers.modeling_utils as modeling_utils
    import transformers.utils as tf_utils
    from transformers.pytorch_utils import Conv1D

    if not hasattr(file_utils, "cached_property"):
        file_utils.cached_property = functools.cached_property
    if not hasattr(file_utils, "torch_only_method"):
        file_utils.torch_only_method = lambda fn: fn

    if "transformers.utils.fx" not in sys.modules:
        fx = types.ModuleType("transformers.utils.fx")

        class HFTracer(torch.fx.Tracer):
            """Placeholder base class: no Hugging Face model is declared traceable."""

        def symbolic_trace(model, input_names=None, **kwargs):
            raise NotImplementedError("transformers.utils.fx was removed from transformers 5.x")

        fx.HFTracer = HFTracer
        fx.symbolic_trace = symbolic_trace
        fx._SUPPORTED_MODELS = ()
        fx._generate_supported_model_class_names = lambda *a, **k: []
        sys.modules["transformers.utils.fx"] = fx
        tf_utils.fx = fx

    if not hasattr(modeling_utils, "Conv1D"):
        modeling_utils.Conv1D = Conv1D
    if not hasattr(transformers, "Conv1D"):
        transformers.Conv1D = Conv1D
