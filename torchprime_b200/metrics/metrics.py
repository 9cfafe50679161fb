"""Run-level metrics record written to ``train_metrics.json``.

Field names and JSON encoding (durations as seconds) match the reference's ``Metrics`` /
``MetricsLogger`` (torchprime/metrics/metrics.py:11-86) so downstream tooling that reads
``outputs/train_metrics.json`` keeps working.
"""

from __future__ import annotations

import dataclasses
import json
import time
from dataclasses import dataclass
from datetime import timedelta
from pathlib import Path

_DURATION_FIELDS = ("train_runtime", "step_execution_time")


@dataclass(frozen=True, eq=True)
class Metrics:
  train_runtime: timedelta
  """Wall time of the whole run, start-up included."""
  step_execution_time: timedelta | None
  """Median device time of one training step (max over ranks)."""
  mfu: float | None
  tokens_per_second: float | None
  num_steps: int | None

  def __str__(self):
    return "".join(f"{k:20} = {v if v is not None else 'N/A'}\n" for k, v in dataclasses.asdict(self).items())

  def to_dict(self) -> dict:
    d = dataclasses.asdict(self)
    for k in _DURATION_FIELDS:
      if d[k] is not None:
        d[k] = d[k].total_seconds()
    return d

  def to_json(self) -> str:
    return json.dumps(self.to_dict())

  @staticmethod
  def from_json(text: str) -> "Metrics":
    d = json.loads(text)
    for k in _DURATION_FIELDS:
      if d.get(k) is not None:
        d[k] = timedelta(seconds=d[k])
    return Metrics(**d)

  def save(self, path: Path):
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(self.to_json())

  @staticmethod
  def load(path: Path) -> "Metrics":
    return Metrics.from_json(Path(path).read_text())


class MetricsLogger:
  """Collects the pieces of :class:`Metrics`; the wall clock starts at construction."""

  def __init__(self):
    self.start_time = time.time()
    self.train_runtime = None
    self.step_execution_time = None
    self.mfu = None
    self.tokens_per_second = None
    self.num_steps = None

  def log_step_execution_time(self, seconds: float):
    self.step_execution_time = seconds

  def log_mfu(self, mfu: float):
    self.mfu = mfu

  def log_tokens_per_second(self, tps: float):
    self.tokens_per_second = tps

  def log_num_steps(self, n: int):
    self.num_steps = n

  def finalize(self) -> Metrics:
    elapsed = timedelta(seconds=time.time() - self.start_time)
    self.train_runtime = elapsed
    step = timedelta(seconds=self.step_execution_time) if self.step_execution_time else None
    return Metrics(train_runtime=elapsed, step_execution_time=step, mfu=self.mfu,
                   tokens_per_second=self.tokens_per_second, num_steps=self.num_steps)
