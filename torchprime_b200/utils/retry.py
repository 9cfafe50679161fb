"""Retry with jittered back-off for flaky I/O (tokenizer / dataset / hub fetches).
Same contract as the reference's torchprime/utils/retry.py:10-26."""

from __future__ import annotations

import logging
import random
import time
from typing import Callable, TypeVar

T = TypeVar("T")
logger = logging.getLogger(__name__)


def retry(fn: Callable[[], T], retry_count: int = 3, retry_delay: float = 10) -> T:
  """Call ``fn`` up to ``retry_count`` times, sleeping ``delay * (1 + U[0,1))`` between
  attempts, and re-raise the last exception."""
  attempt = 0
  while True:
    attempt += 1
    try:
      return fn()
    except Exception as exc:  # noqa: BLE001 - the caller decides what is fatal
      if attempt >= retry_count:
        logger.error("giving up after %d attempts: %s", retry_count, exc)
        raise
      pause = retry_delay * (1.0 + random.random())
      logger.warning("attempt %d/%d failed (%s); retrying in %.1f s", attempt, retry_count, exc, pause)
      time.sleep(pause)
