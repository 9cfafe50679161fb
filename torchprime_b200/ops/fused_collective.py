"""GEMMs fused with their collective over NVLink peer memory.

``ag_gemm``: ``y = x @ W^T`` where the flat buffer that contains ``W`` is sharded over the ranks of a
group (FSDP parameter shards, or a row-sharded activation/weight for tensor parallelism).  A few
copier CTAs of the same kernel move the shards while the other CTAs compute: by default every rank
PUSHES its shard into the peers' gathered buffers with plain 16-byte stores (posted writes over
NVLink) and raises per-chunk flags in the peers' memory; ``push=False`` makes every rank pull the
remote shards instead (bulk copies from peer memory through shared memory, no multicast).  The
GEMM CTAs load their B tiles locally as soon as the chunks they need have landed.  The rank's own
shard is put in place by a device-to-device copy on the same stream before the kernel starts.
Where the gathered buffers are bound to an NVSwitch multicast object (``multicast=True``, or by
default when the platform offers it), the push is one ``multimem.st`` per 16 bytes that the switch
replicates into every rank's buffer, so each rank sends its shard once instead of once per peer.
After the call the whole buffer is gathered, so the other weights of the same FSDP unit are ready
too.

``gemm_rs``: ``dW = dY^T X`` (or any GEMM) whose epilogue adds ``alpha * tile`` directly into the
owning rank's bf16 gradient shard with 16-byte ``red.add`` over P2P, replacing the separate
reduce-scatter.  Shards must be zero and all ranks synchronised before the first contribution.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import torch

from . import _lib
from ._lib import check, lib, ptr, stream_ptr

P, I, LL, FL, U = c_void_p, c_int, c_longlong, c_float, c_uint
_lib.register_signature("tpb_ag_gemm_bf16", [P, P, I, I, I, LL, LL, I, P, LL, P, LL, P, I, LL, P, LL, P, U, I, I, P, P, P, P])
_lib.register_signature("tpb_gemm_rs_bf16", [P, P, I, I, I, LL, LL, LL, I, I, FL, P, I, LL, LL, I, P])

CHUNK_ELEMS = 16384


def num_flags(world: int, shard_elems: int) -> int:
  return world * ((shard_elems + CHUNK_ELEMS - 1) // CHUNK_ELEMS)


class AllGatherGemm:
  """State for repeated fused all-gather + GEMM calls on one sharded flat buffer."""

  def __init__(self, shard_buffer, shard_elems: int, copiers: int = 32, push: bool = True,
               multicast: bool | None = None):
    """``push``: every rank sends its shard to the peers (posted stores over NVLink) instead of
    fetching theirs.  The gathered buffer and the flags then live in symmetric memory owned by this
    object (``self.gathered``), and the ranks must be synchronised between two calls (nobody may
    still be reading the previous gather when the next one starts to arrive).  ``multicast``: push
    through the NVSwitch multicast mapping of the gathered buffers (None: with more than two ranks,
    when available; ``TPB_AG_MULTICAST=0/1`` overrides)."""
    self.sb = shard_buffer                     # dist.symm.SymmetricBuffer holding this rank's shard
    self.world = shard_buffer.world
    self.shard_elems = shard_elems
    self.copiers = copiers
    self.push = push
    dev = shard_buffer.local.device
    self.epoch = 0
    if push:
      from ..dist.symm import SymmetricBuffer
      import os
      if multicast is None:
        # measured: equal to per-peer stores on 8 GPUs with half the copier CTAs, slower on 2
        multicast = os.environ.get("TPB_AG_MULTICAST", "1" if self.world > 2 else "0") != "0"
      self.gathered_sb, self.multicast_ptr = None, 0
      if multicast:
        # multicast objects come with torch's symmetric allocations (CUDA VMM + cuMulticast); without
        # multicast support the same buffer is used with per-peer stores
        self.gathered_sb = SymmetricBuffer(shard_elems * self.world, torch.bfloat16, dev, group=shard_buffer.group,
                                           backend="torch")
        self.multicast_ptr = self.gathered_sb.multicast_ptr
      if self.gathered_sb is None:
        self.gathered_sb = SymmetricBuffer(shard_elems * self.world, torch.bfloat16, dev, group=shard_buffer.group)
      self.flags_sb = SymmetricBuffer(num_flags(self.world, shard_elems), torch.int32, dev, group=shard_buffer.group)
      self.flags_sb.local.zero_()
      self.gathered = self.gathered_sb.local
      self.flags = self.flags_sb.local
      self.flags_sb.barrier()
    else:
      self.gathered = None
      self.flags = torch.zeros(num_flags(self.world, shard_elems), dtype=torch.int32, device=dev)

  def __call__(self, x2d, gathered, b_offset: int, n: int, k: int, shard_offset: int = 0, out=None,
               epi=_lib.EPI_BF16, aux=None, c2=None):
    """out = x2d @ B^T with B = gathered[b_offset : b_offset + n*k].view(n, k); gathers every rank's
    ``shard_elems`` elements (starting ``shard_offset`` elements into its symmetric buffer)."""
    m = x2d.shape[0]
    self.epoch += 1
    if self.push:
      gathered = self.gathered
    if out is None:
      out = torch.empty(m, n // 2 if epi == _lib.EPI_SWIGLU else n, dtype=torch.bfloat16, device=x2d.device)
    table = self.sb.ptr_table(shard_offset)
    rank = self.sb.rank
    gathered[rank * self.shard_elems:(rank + 1) * self.shard_elems].copy_(
        self.sb.local[shard_offset:shard_offset + self.shard_elems])
    rc = lib().tpb_ag_gemm_bf16(ptr(x2d), ptr(out), m, n, k, x2d.stride(0), out.stride(0), epi, ptr(aux),
                                aux.stride(0) if aux is not None else 0, ptr(c2), c2.stride(0) if c2 is not None else 0,
                                table, self.world, self.shard_elems, ptr(gathered), b_offset, ptr(self.flags),
                                self.epoch, self.copiers, rank,
                                self.gathered_sb.ptr_table() if self.push else None,
                                self.flags_sb.ptr_table() if self.push else None,
                                (self.multicast_ptr or None) if self.push else None, stream_ptr())
    check(rc, f"ag_gemm M={m} N={n} K={k} world={self.world}")
    return out


def gemm_rs(a, b, *, a_mn, b_mn, m, n, ldc, grad_shards, shard_elems: int, c_offset: int, alpha: float,
            shard_offset: int = 0):
  """Adds ``alpha * (A @ B^T)`` ([m, n], row pitch ``ldc`` inside the flat sharded buffer at
  ``c_offset``) into the owners' shards.  ``grad_shards`` is the SymmetricBuffer of gradient shards."""
  k = a.shape[0] if a_mn else a.shape[1]
  table = grad_shards.ptr_table(shard_offset)
  rc = lib().tpb_gemm_rs_bf16(ptr(a), ptr(b), m, n, k, a.stride(0), b.stride(0), ldc, int(a_mn), int(b_mn),
                              float(alpha), table, grad_shards.world, shard_elems, c_offset, grad_shards.rank,
                              stream_ptr())
  check(rc, f"gemm_rs M={m} N={n} K={k} world={grad_shards.world}")


class AllReduceGemm:
  """``sum over the ranks of a group of (A_r @ B_r^T) (+ residual)`` with the all-reduce inside the GEMM
  epilogue: the output lives in a symmetric buffer bound to an NVSwitch multicast object, every rank's
  epilogue adds its tile into ALL ranks' copies with one ``multimem.red`` per 16 bytes, and when the
  kernels have finished every rank holds the sum.  This is the row-parallel linear of tensor
  parallelism (and, in the backward pass, the input gradient of the column-parallel one) without a
  separate all-reduce pass.

  Per call: zero the local copy, device barrier (all copies are zero), GEMM, device barrier (all
  contributions have landed), copy the result out of the shared buffer.  The residual, when given,
  is added by rank 0 only.  ``available`` is False where the platform offers no multicast mapping;
  callers then use the NCCL all-reduce."""

  def __init__(self, group, device):
    import torch.distributed as dist
    self.group = group
    self.device = device
    self.world = dist.get_world_size(group)
    self.rank = dist.get_rank(group)
    self._bufs = {}
    self.available = True
    self.calls = 0

  def _buffer(self, m: int, n: int):
    from ..dist.symm import SymmetricBuffer
    key = (m, n)
    if key not in self._bufs:
      sb = SymmetricBuffer(m * n, torch.bfloat16, self.device, group=self.group, backend="torch")
      if not sb.multicast_ptr:
        self.available = False
      self._bufs[key] = sb
    return self._bufs[key]

  def usable(self, m: int, n: int, k: int) -> bool:
    if not self.available or n % 32 or k % 8:
      return False
    self._buffer(m, n)                      # collective on first use of a shape: every rank takes this path
    return self.available

  def gemm_allreduce(self, a2d, b, residual2d=None, b_mn: bool = False):
    """a2d [M, K]; b [N, K] (or [K, N] with ``b_mn``); returns the reduced [M, N] bf16 tensor."""
    m, kdim = a2d.shape
    n = b.shape[1] if b_mn else b.shape[0]
    sb = self._buffer(m, n)
    assert sb.multicast_ptr and a2d.stride(1) == 1 and b.stride(1) == 1
    sb.local.zero_()
    sb.barrier()
    aux = residual2d if (residual2d is not None and self.rank == 0) else None
    rc = lib().tpb_gemm_bf16(ptr(a2d), ptr(b), c_void_p(sb.multicast_ptr), m, n, kdim, a2d.stride(0), b.stride(0), n,
                             0, int(b_mn), _lib.EPI_AR_BF16, 1.0, ptr(aux), aux.stride(0) if aux is not None else 0,
                             None, 0, 0, stream_ptr())
    check(rc, f"gemm_allreduce M={m} N={n} K={kdim} world={self.world}")
    sb.barrier()
    self.calls += 1
    return sb.local.view(m, n).clone()
