"""Symmetric (peer-mapped) device memory over NVLink for the fused compute+collective kernels.

A :class:`SymmetricBuffer` is a tensor that exists with the same size on every rank of a group and
is mapped into every rank's address space; kernels receive the table of base pointers and read,
write or ``red.add`` into their peers' copies directly.

Two backends:

* ``native`` (default) - the C++ runtime of this package (``csrc/symm_runtime.cu``): the segment is a
  ``cudaMalloc`` allocation exported as an inter-process handle, the 64-byte handles are exchanged
  over the host process group, peers are mapped with lazy peer access, and the barrier is a
  bounded device-side barrier on a signal pad in front of each segment (a wait that runs out
  reports into the status block instead of hanging).
* ``torch`` - ``torch.distributed._symmetric_memory`` (CUDA VMM allocations).  Used when
  ``TPB_SYMM_BACKEND=torch`` or when the native path cannot export or map a segment on this
  machine; every rank takes the same decision.  ``TPB_SYMM_STRICT=1`` turns the fallback into an
  error.
"""

from __future__ import annotations

import ctypes
import logging
import os

import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)


class _DeviceMemoryView:
  """Lets torch alias a raw device range through the CUDA array interface."""

  def __init__(self, ptr: int, nbytes: int):
    self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _native_lib():
  from ..ops import _lib
  L = _lib.lib()
  if not hasattr(L, "tpb_symm_alloc"):
    return None
  P, I, LL, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint
  L.tpb_symm_alloc.argtypes = [LL, ctypes.POINTER(P), ctypes.c_char_p]
  L.tpb_symm_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(P)]
  L.tpb_symm_release.argtypes = [P]
  L.tpb_symm_copy.argtypes = [P, P, LL, P]
  L.tpb_symm_live_segments.argtypes = []
  L.tpb_symm_barrier.argtypes = [ctypes.POINTER(P), I, I, U, P]
  for f in (L.tpb_symm_alloc, L.tpb_symm_open, L.tpb_symm_release, L.tpb_symm_copy, L.tpb_symm_live_segments,
            L.tpb_symm_barrier):
    f.restype = I
  return L


class SymmetricBuffer:
  """A tensor that exists at the same size on every rank of ``group`` and is mapped into all of them."""

  def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group=None, backend: str | None = None):
    self.group = group if group is not None else dist.group.WORLD
    self.world = dist.get_world_size(self.group)
    self.rank = dist.get_rank(self.group)
    self._elem = torch.empty(0, dtype=dtype).element_size()
    self._epoch = 0
    self._closed = False
    self.multicast_ptr = 0            # NVSwitch multicast address of the buffers (torch backend only), else 0
    backend = backend or os.environ.get("TPB_SYMM_BACKEND", "native")
    assert backend in ("native", "torch"), backend
    self.backend = None
    if backend == "native":
      why = self._init_native(numel, dtype, torch.device(device))
      if why is not None:
        if os.environ.get("TPB_SYMM_STRICT", "0") == "1":
          raise RuntimeError(f"native symmetric memory unavailable: {why}")
        logger.warning("native symmetric memory unavailable (%s); using torch symmetric memory", why)
    if self.backend is None:
      self._init_torch(numel, dtype, device)

  # ---------------------------------------------------------------- native runtime
  def _init_native(self, numel, dtype, device):
    """Returns None on success, else the reason (identical on every rank)."""
    L = _native_lib()
    nbytes = numel * self._elem
    payload = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(64)
    rc = -1 if L is None else L.tpb_symm_alloc(nbytes, ctypes.byref(payload), handle)
    mine = (rc, handle.raw)
    everyone = [None] * self.world
    dist.all_gather_object(everyone, mine, group=self.group)
    if any(r != 0 for r, _ in everyone):
      if rc == 0:
        L.tpb_symm_release(payload)
      return f"allocation/export failed with codes {[r for r, _ in everyone]}"
    ptrs, opened, bad = [0] * self.world, [], 0
    for r, (_, h) in enumerate(everyone):
      if r == self.rank:
        ptrs[r] = payload.value
        continue
      p = ctypes.c_void_p()
      rc = L.tpb_symm_open(h, ctypes.byref(p))
      if rc != 0:
        bad = rc
        break
      ptrs[r] = p.value
      opened.append(p)
    verdicts = [None] * self.world
    dist.all_gather_object(verdicts, bad, group=self.group)
    if any(v != 0 for v in verdicts):
      for p in opened:
        L.tpb_symm_release(p)
      dist.barrier(group=self.group)              # peers unmapped before any owner frees
      L.tpb_symm_release(payload)
      return f"mapping a peer segment failed with codes {verdicts}"
    self._L = L
    self._view = _DeviceMemoryView(payload.value, max(nbytes, 1))
    self.local = torch.as_tensor(self._view, device=device)[:nbytes].view(dtype)
    self.ptrs = ptrs
    self._table = (ctypes.c_void_p * self.world)(*ptrs)
    self.backend = "native"
    return None

  # ---------------------------------------------------------------- torch symmetric memory
  def _init_torch(self, numel, dtype, device):
    import torch.distributed._symmetric_memory as symm_mem
    self.local = symm_mem.empty(numel, dtype=dtype, device=device)
    self.handle = symm_mem.rendezvous(self.local, group=self.group)
    off = int(getattr(self.handle, "offset", 0) or 0)
    self.ptrs = [int(p) + off for p in self.handle.buffer_ptrs]
    assert self.ptrs[self.rank] == self.local.data_ptr(), "symmetric buffer pointer table does not match the tensor"
    mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
    self.multicast_ptr = mc + off if mc else 0
    self.backend = "torch"

  # ---------------------------------------------------------------- common surface
  def ptr_table(self, offset_elems: int = 0):
    """ctypes array of every rank's base pointer (+ offset), for the C entry points."""
    arr = (ctypes.c_void_p * self.world)()
    for i, p in enumerate(self.ptrs):
      arr[i] = p + offset_elems * self._elem
    return arr

  def barrier(self):
    """Device-side barrier over the group (ordered on the current stream)."""
    if self.backend == "torch":
      self.handle.barrier()
      return
    from ..ops import _lib
    self._epoch += 1
    _lib.check(self._L.tpb_symm_barrier(self._table, self.rank, self.world, self._epoch & 0xFFFFFFFF,
                                        _lib.stream_ptr()), "symm_barrier")

  def copy_from_rank(self, out: torch.Tensor, src_rank: int, offset_elems: int = 0):
    """``out`` <- ``out.numel()`` elements of rank ``src_rank``'s copy (copy engine, current stream)."""
    from ..ops import _lib
    L = _native_lib()
    assert L is not None and out.is_contiguous() and out.element_size() == self._elem
    _lib.check(L.tpb_symm_copy(out.data_ptr(), self.ptrs[src_rank] + offset_elems * self._elem,
                               out.numel() * self._elem, _lib.stream_ptr()), "symm_copy")
    return out

  def close(self):
    """Collective: unmap the peers, meet, then free the own segment (native backend)."""
    if self._closed or self.backend != "native":
      return
    self._closed = True
    torch.cuda.synchronize()
    for r, p in enumerate(self.ptrs):
      if r != self.rank:
        self._L.tpb_symm_release(ctypes.c_void_p(p))
    dist.barrier(group=self.group)
    self.local = None
    self._L.tpb_symm_release(ctypes.c_void_p(self.ptrs[self.rank]))


def live_native_segments() -> int:
  L = _native_lib()
  return 0 if L is None else L.tpb_symm_live_segments()


def is_supported(device: torch.device) -> bool:
  if device.type != "cuda" or not dist.is_initialized():
    return False
  if _native_lib() is not None:
    return True
  try:
    import torch.distributed._symmetric_memory  # noqa: F401
    return True
  except Exception:  # noqa: BLE001
    return False
