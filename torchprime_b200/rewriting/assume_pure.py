"""``model.pure_modules``: classes the user declares free of side effects.

In the reference these are wrapped in torch_xla's ``PureModule`` so they are traced once
and their profile scopes also show up in backward (torchprime/torch_xla_models/
model_rewriting/assume_pure.py:1-40).  Eager CUDA execution has no tracing cost to avoid,
so the declaration is used for what remains meaningful: the listed classes get a trace
scope named after the class in both forward and the recomputation inside backward, and
unknown class names are rejected.
"""

from __future__ import annotations

import functools

import torch.nn as nn

from ..utils.profiling import trace_scope
from .rematerialization_utils import get_classes_by_names


def mark_pure_modules(model: nn.Module, config) -> nn.Module:
  names = list(config.model.get("pure_modules", []) or [])
  if not names:
    return model
  classes = get_classes_by_names(model, names)
  for mod in model.modules():
    if isinstance(mod, classes) and not getattr(mod, "_pure_marked", False):
      inner = mod.forward
      label = type(mod).__name__

      @functools.wraps(inner)
      def scoped(*a, _inner=inner, _label=label, **k):
        with trace_scope(_label):
          return _inner(*a, **k)

      mod.forward = scoped
      mod._pure_marked = True
  return model
