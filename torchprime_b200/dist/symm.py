"""Symmetric (peer-mapped) device memory over NVLink for the fused compute+collective kernels.

Allocation, handle exchange and mapping use ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations exported to every rank of the group); what this module adds is the small amount of
bookkeeping the kernels need: the table of peer base pointers, epoch-numbered flag arrays and a
device-side barrier between phases that touch peer memory.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist


class SymmetricBuffer:
  """A tensor that exists at the same size on every rank of ``group`` and is mapped into all of them."""

  def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group=None):
    import torch.distributed._symmetric_memory as symm_mem
    self.group = group if group is not None else dist.group.WORLD
    self.local = symm_mem.empty(numel, dtype=dtype, device=device)
    self.handle = symm_mem.rendezvous(self.local, group=self.group)
    self.world = self.handle.world_size
    self.rank = self.handle.rank
    self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
    elem = self.local.element_size()
    self._elem = elem

  def ptr_table(self, offset_elems: int = 0):
    """ctypes array of every rank's base pointer (+ offset), for the C entry points."""
    arr = (ctypes.c_void_p * self.world)()
    for i, p in enumerate(self.ptrs):
      arr[i] = p + offset_elems * self._elem
    return arr

  def barrier(self):
    """Device-side barrier over the group (ordered on the current stream)."""
    self.handle.barrier()


def is_supported(device: torch.device) -> bool:
  if device.type != "cuda" or not dist.is_initialized():
    return False
  try:
    import torch.distributed._symmetric_memory  # noqa: F401
    return True
  except Exception:  # noqa: BLE001
    return False
