"""Range-checked debug mode for the kernels whose addresses come from data.

The kernels that index memory with values read from a tensor (token ids, targets, positions, the
MoE plan's row maps, the exchange descriptors) trust those values on the normal path: checking them
costs a pass over the index tensor and a host read.  With ``TPB_DEBUG_BOUNDS=1`` every such wrapper
validates its index tensors on the device first and raises ``IndexError`` naming the op, the
argument, how many entries are out of range and the first of them, before the kernel is launched:
an out-of-range index becomes a Python exception instead of a memory fault.  The check reads one
scalar back per call, so the mode is for debugging runs and for the test suite, not for timing.

Tile arithmetic (shapes, strides, tails) is covered by the shape sweeps of the numerics tests; this
mode covers the other class of out-of-bounds access, the one that depends on the data.
"""

from __future__ import annotations

import os

import torch


def bounds_enabled() -> bool:
  return os.environ.get("TPB_DEBUG_BOUNDS", "0") == "1"


def check_index(op: str, name: str, t, lo: int, hi: int, also_allowed: int | None = None) -> None:
  """Raise IndexError unless every entry of the integer tensor ``t`` is in [lo, hi) (or equals
  ``also_allowed``, e.g. an ignore index or a "skip" marker).  A no-op unless the mode is on, and
  while a CUDA graph is being captured (no host read is possible then)."""
  if not bounds_enabled() or t is None or t.numel() == 0:
    return
  if t.is_cuda and torch.cuda.is_current_stream_capturing():
    return
  bad = (t < lo) | (t >= hi)
  if also_allowed is not None:
    bad &= t != also_allowed
  n_bad = int(bad.sum().item())
  if n_bad:
    first = int(torch.nonzero(bad.reshape(-1))[0].item())
    raise IndexError(f"{op}: {n_bad} of {t.numel()} entries of `{name}` are outside [{lo}, {hi}); "
                     f"first at flat position {first}: {int(t.reshape(-1)[first].item())}")


def check_monotone(op: str, name: str, t, lo: int, hi: int) -> None:
  """Raise IndexError unless ``t`` is non-decreasing with every entry in [lo, hi]."""
  if not bounds_enabled() or t is None or t.numel() == 0:
    return
  if t.is_cuda and torch.cuda.is_current_stream_capturing():
    return
  check_index(op, name, t, lo, hi + 1)
  if t.numel() > 1 and bool((t[1:] < t[:-1]).any().item()):
    raise IndexError(f"{op}: `{name}` is not non-decreasing")


def check_exchange_descriptors(op: str, desc, n_blocks: int, n_rows: int, world: int, max_rows: int) -> None:
  """Validate the block descriptors of the expert-exchange push kernel: ``desc`` is int64
  ``start[n_blocks + 1] | dst_rank[n_blocks] (-1: skip) | dst_row0[n_blocks]``.  Block starts must be
  non-decreasing inside the ``n_rows`` send rows, destination ranks inside the group, and every
  block that is sent must fit the ``max_rows`` of the receive buffer."""
  if not bounds_enabled():
    return
  if desc.is_cuda and torch.cuda.is_current_stream_capturing():
    return
  if desc.numel() != 3 * n_blocks + 1:
    raise IndexError(f"{op}: descriptor tensor has {desc.numel()} entries, {3 * n_blocks + 1} expected")
  start, dst_rank, dst_row0 = desc[: n_blocks + 1], desc[n_blocks + 1: 2 * n_blocks + 1], desc[2 * n_blocks + 1:]
  check_monotone(op, "start", start, 0, n_rows)
  check_index(op, "dst_rank", dst_rank, 0, world, also_allowed=-1)
  live = (dst_rank >= 0) & (dst_rank < world)
  check_index(op, "dst_row0", dst_row0[live], 0, max_rows + 1)
  check_index(op, "dst_row0 + block rows", (dst_row0 + (start[1:] - start[:-1]))[live], 0, max_rows + 1)
