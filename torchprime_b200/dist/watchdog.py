"""Host-side failure detection: a per-rank step deadline and a heartbeat over the store.

The reference has no liveness machinery beyond xpk restarts (launcher/cli.py:388-391).
Here a daemon thread watches the training loop: if a step does not finish within the
deadline it dumps where the rank is stuck and either raises in the main thread on the
next ``end_step`` or (``abort=True``) exits the process so the launcher can tear the job
down.  Device-side waits are already bounded (kernels report into a status block, see
csrc/common.cuh), so a stuck rank is always a host-visible condition.
"""

from __future__ import annotations

import faulthandler
import logging
import os
import sys
import threading
import time

logger = logging.getLogger(__name__)


class StepDeadlineExceeded(RuntimeError):
  pass


class StepWatchdog:
  def __init__(self, deadline_s: float, abort: bool = False, poll_s: float | None = None, on_timeout=None):
    self.deadline_s = float(deadline_s)
    self.abort = abort
    self.poll_s = poll_s if poll_s is not None else min(1.0, self.deadline_s / 4)
    self.on_timeout = on_timeout
    self._lock = threading.Lock()
    self._step = None
    self._t0 = None
    self._tripped = None
    self._stop = threading.Event()
    self._thread = threading.Thread(target=self._run, name="step-watchdog", daemon=True)
    self._thread.start()

  def begin_step(self, step: int):
    with self._lock:
      self._step, self._t0 = step, time.monotonic()

  def end_step(self, step: int):
    with self._lock:
      self._step, self._t0 = None, None
      tripped = self._tripped
    if tripped is not None:
      raise StepDeadlineExceeded(f"step {tripped[0]} exceeded the {self.deadline_s:.1f} s deadline "
                                 f"(ran {tripped[1]:.1f} s)")

  def tripped(self):
    return self._tripped

  def stop(self):
    self._stop.set()
    self._thread.join(timeout=2 * self.poll_s + 1)

  def _run(self):
    while not self._stop.wait(self.poll_s):
      with self._lock:
        step, t0 = self._step, self._t0
      if step is None or self._tripped is not None:
        continue
      ran = time.monotonic() - t0
      if ran > self.deadline_s:
        self._tripped = (step, ran)
        logger.error("watchdog: step %d has been running for %.1f s (deadline %.1f s)", step, ran, self.deadline_s)
        try:
          faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
        except Exception:  # noqa: BLE001
          pass
        if self.on_timeout is not None:
          self.on_timeout(step, ran)
        if self.abort:
          os._exit(3)


class Heartbeat:
  """Ranks publish a counter in the rendezvous store; anyone can ask who went silent."""

  def __init__(self, store, rank: int, world_size: int, prefix: str = "hb"):
    self.store, self.rank, self.world_size, self.prefix = store, rank, world_size, prefix
    self._seen = {}

  def beat(self, step: int):
    self.store.set(f"{self.prefix}/{self.rank}", f"{step}:{time.time()}")

  def stale_ranks(self, max_age_s: float) -> list[int]:
    now = time.time()
    stale = []
    for r in range(self.world_size):
      try:
        if not self.store.check([f"{self.prefix}/{r}"]):
          stale.append(r)
          continue
        _step, ts = self.store.get(f"{self.prefix}/{r}").decode().split(":")
        if now - float(ts) > max_age_s:
          stale.append(r)
      except Exception:  # noqa: BLE001 - an unreachable store counts as "unknown", not dead
        stale.append(r)
    return stale
