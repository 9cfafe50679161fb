"""Profiling helpers: the capture-window arithmetic and named trace scopes.

``ensure_profile_end_step`` has the behaviour of the reference's
torchprime/utils/profiling.py:8-36.  ``trace_scope`` is the analogue of its
``xp.Trace`` / ``@xp.trace_me`` scopes: an NVTX range plus a ``record_function``
region, active only while a capture is running so the steady state pays nothing.
"""

from __future__ import annotations

import logging
from contextlib import contextmanager

import torch

logger = logging.getLogger(__name__)
_TRACE_ON = False


def set_tracing(on: bool):
  global _TRACE_ON
  _TRACE_ON = bool(on)


def tracing_enabled() -> bool:
  return _TRACE_ON


@contextmanager
def trace_scope(name: str):
  if not _TRACE_ON:
    yield
    return
  nvtx = torch.cuda.is_available()
  if nvtx:
    torch.cuda.nvtx.range_push(name)
  try:
    with torch.profiler.record_function(name):
      yield
  finally:
    if nvtx:
      torch.cuda.nvtx.range_pop()


def ensure_profile_end_step(config, num_profile_steps: int = 20):
  """Clamp the profiling window to the run (config is modified in place and returned).

  Profiling is switched off (both steps -1) when the start is negative or leaves fewer
  than two steps; otherwise the end defaults to ``start + num_profile_steps``, is kept
  five steps clear of ``max_steps`` and is at least ``start + 1``."""
  start = config.get("profile_start_step", -1)
  start = -1 if start is None else start
  window = config.get("num_profile_steps", None) or num_profile_steps
  last = config.task.max_steps
  if start < 0 or start >= last - 1:
    config.profile_start_step = -1
    config.profile_end_step = -1
    return config
  stop = config.get("profile_end_step", None)
  if stop is None:
    stop = start + window
  config.profile_end_step = max(min(stop, last - 5), start + 1)
  return config
