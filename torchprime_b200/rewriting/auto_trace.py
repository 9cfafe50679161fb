"""Adds a named trace scope around the forward of selected leaf modules.

Counterpart of the reference's ``auto_trace`` (torchprime/torch_xla_models/model_rewriting/
auto_trace.py:1-35), which wraps every ``nn.Linear`` in ``xp.Trace(<attribute name>)``.
Here the scope is an NVTX range + ``record_function`` region (utils/profiling.py), visible
in the Chrome trace written for the profiling window.
"""

from __future__ import annotations

import functools

import torch.nn as nn

from ..utils.profiling import trace_scope


def auto_trace(model: nn.Module, types: tuple = (nn.Linear,)) -> nn.Module:
  for parent in model.modules():
    for attr, child in parent.named_children():
      if isinstance(child, types) and not getattr(child, "_auto_traced", False):
        _wrap(child, attr)
  return model


def _wrap(mod: nn.Module, label: str):
  inner = mod.forward

  @functools.wraps(inner)
  def traced(*args, **kwargs):
    with trace_scope(label):
      return inner(*args, **kwargs)

  mod.forward = traced
  mod._auto_traced = True
