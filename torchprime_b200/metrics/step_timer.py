"""Device-side step timing.

The reference derives the step time from the device profile: the median of the
start-to-start deltas of consecutive executions of the step program on device 0, the
mean when there are fewer than three intervals
(torchprime/metrics/step_duration.py:122-192).  The CUDA analogue records one event at
the start of every step on the compute stream; consecutive event pairs give the same
start-to-start deltas, measured by the GPU.  The reported value is the max over ranks of
each rank's statistic.
"""

from __future__ import annotations

import statistics
import time

import torch


class StepTimer:
  def __init__(self, use_cuda: bool | None = None):
    self.use_cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
    self._marks = []   # (step, event or host time)

  def mark(self, step: int):
    """Call at the start of every step (and once after the last one)."""
    if self.use_cuda:
      ev = torch.cuda.Event(enable_timing=True)
      ev.record(torch.cuda.current_stream())
      self._marks.append((step, ev))
    else:
      self._marks.append((step, time.perf_counter()))

  def deltas(self, first_step: int = 0, last_step: int | None = None) -> list[float]:
    """Seconds between consecutive marks whose step lies in [first_step, last_step]."""
    if self.use_cuda:
      torch.cuda.synchronize()
    out = []
    for (s0, a), (s1, b) in zip(self._marks[:-1], self._marks[1:]):
      if s0 < first_step or (last_step is not None and s1 > last_step):
        continue
      out.append(a.elapsed_time(b) / 1e3 if self.use_cuda else b - a)
    return out

  @staticmethod
  def summarize(deltas: list[float]) -> float | None:
    """Median of the intervals; the mean when there are fewer than three."""
    if not deltas:
      return None
    return statistics.median(deltas) if len(deltas) >= 3 else sum(deltas) / len(deltas)

  def step_duration(self, first_step: int = 0, last_step: int | None = None, reduce_max: bool = True) -> float | None:
    from ..dist import runtime as rt
    val = self.summarize(self.deltas(first_step, last_step))
    if val is None:
      return None
    return rt.all_reduce_max_float(val) if reduce_max else val
