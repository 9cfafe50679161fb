"""Peer-memory collectives of the FSDP engine (``engine.fsdp_collectives=peer``).

What the reference gets from the SPMD partitioner plus XLA's latency-hiding scheduler for
``[fsdp, null]`` parameter specs (one all-gather of a layer's weights before use, one reduce-scatter
of its gradients, both overlapped with compute; torchprime/torch_xla_models/configs/model/sharding/
llama-fsdp.yaml:2-13, torchprime/launcher/Dockerfile:69) is done here over NVLink peer mappings
without NCCL kernels, so that no SM is taken from the GEMMs while parameters and gradients move:

* **All-gather.**  The bf16 parameter shards live in symmetric memory.  A unit's gather is one
  copy-engine copy per peer (peer shard -> local gathered buffer, the own shard first, then peers in
  rotated order so that every GPU serves one reader at a time), each followed by a one-thread kernel that
  publishes a flag.  GEMMs that read a weight of a unit whose gather is still in flight wait on the
  flags under their B tile inside the TMA producer (``tpb_gemm_ag_wait_bf16``): the first GEMM of a
  layer starts as soon as the shards that hold its weight have landed.  Everything else that reads the
  unit waits on a stream event.
* **Reduce-scatter.**  Every owner has a staging area of ``fsdp`` slots per unit buffer.  The weight
  gradient GEMMs store their tiles straight into this rank's slot at the owner of each tile row
  (``tpb_gemm_rs_store_bf16``: plain 16-byte stores over NVLink from the epilogue); whatever the GEMMs
  did not produce (norm weights, embedding rows, gradients that arrived through plain autograd) follows
  by copy-engine copies.  A signal tells the owners that this rank's contribution is complete; the
  owner waits for all signals and adds the slots in rank order in fp32 (``tpb_rs_reduce_bf16``),
  scaling by 1/fsdp and writing (or accumulating into) its gradient shard.  The sum therefore has a
  fixed order and is rounded to bf16 once.  The owner then signals the slot free; a rank waits for
  that signal before the next unit that uses the same slot starts to push.

Cross-step hazards are closed by two device barriers per step (``params_will_change`` before the
optimizer overwrites the shards that peers may still be copying, ``params_changed`` after it).
All waits are bounded and report into the status block instead of hanging.
"""

from __future__ import annotations

import ctypes
import logging
import os
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import torch

from ..dist.symm import SymmetricBuffer
from ..ops import _lib
from ..ops._lib import check, lib, ptr

logger = logging.getLogger(__name__)

P, I, LL, FL, U = c_void_p, c_int, c_longlong, c_float, c_uint
_lib.register_signature("tpb_flag_set", [P, U, P])
_lib.register_signature("tpb_peer_signal", [P, I, LL, U, P])
_lib.register_signature("tpb_flag_wait", [P, I, LL, U, I, P])
_lib.register_signature("tpb_rs_reduce_bf16", [P, I, LL, LL, P, I, I, FL, P])
_lib.register_signature("tpb_gemm_rs_store_bf16", [P, P, I, I, I, LL, LL, LL, I, I, FL, P, I, LL, LL, I, P])
_lib.register_signature("tpb_gemm_ag_wait_bf16", [P, P, I, I, I, LL, LL, I, P, LL, P, LL, P, LL, I, LL, LL, P, U, P])
_lib.register_signature("tpb_symm_copy", [P, P, LL, P])
_lib.register_signature("tpb_embedding_fwd_peer", [P, I, LL, LL, P, P, I, I, LL, P])

_SITE_DONE, _SITE_FREE = 91, 92


class GatherContext:
  """The gather that is in flight for the unit whose forward is running: what a GEMM needs in order to
  wait for its weight inside the kernel."""

  def __init__(self, comm, unit):
    self.comm, self.unit = comm, unit
    buf = unit._gather_buf
    self.base = buf.data_ptr()
    self.nbytes = buf.numel() * buf.element_size()
    self.world = comm.world
    self.shard_elems = unit.shard_size
    self.chunk_elems = unit.shard_size
    self.flags = unit._ag_flags
    self.epoch = unit._ag_epoch

  def offset_of(self, w: torch.Tensor):
    """Element offset of ``w`` inside the gathered buffer, or None when it lives elsewhere."""
    p = w.data_ptr()
    if self.base <= p < self.base + self.nbytes:
      return (p - self.base) // 2
    return None

  def wait_all(self):
    """Order the current stream after the whole gather (for readers that cannot wait in-kernel)."""
    self.comm.wait_gather(self.unit)


def gather_shards(dst_ptr: int, src_ptrs, nbytes: int, flags_ptr: int, epoch: int, rank: int, streams):
  """Enqueue the copy-engine all-gather of one buffer: shard p (``nbytes`` bytes at ``src_ptrs[p]``, peer
  memory) lands at ``dst_ptr + p * nbytes``, then flag p becomes ``epoch``.  Own shard first, peers in
  rotated order (every GPU serves one reader at a time); consecutive copies alternate between the given
  streams so that one copy engine already moves the next shard while the flag of the previous one is
  being published.  The caller orders the streams before and joins them after."""
  L = lib()
  world = len(src_ptrs)
  for j in range(world):
    p = (rank + j) % world
    s = streams[j % len(streams)].cuda_stream
    check(L.tpb_symm_copy(dst_ptr + p * nbytes, src_ptrs[p], nbytes, s), "fsdp gather copy")
    check(L.tpb_flag_set(flags_ptr + 4 * p, epoch, s), "fsdp gather flag")


class PeerLookup:
  """Where an embedding table lives while it stays sharded: every rank's shard of its unit's flat buffer
  (peer-mapped) and the table's offset in that buffer."""

  def __init__(self, comm, unit, slot):
    self.table = comm.param_sb.ptr_table(unit.shard_offset)
    self.world, self.shard_elems, self.offset = comm.world, unit.shard_size, slot.offset
    self.vocab, self.dim = int(slot.shape[0]), int(slot.shape[1])

  def lookup(self, flat_ids, out):
    check(lib().tpb_embedding_fwd_peer(self.table, self.world, self.shard_elems, self.offset, ptr(flat_ids), ptr(out),
                                       flat_ids.numel(), self.dim, self.vocab, _lib.stream_ptr()), "embedding_fwd_peer")


class PeerFsdpComm:
  def __init__(self, engine):
    e = self.engine = engine
    self.group, self.world, self.rank = e.fsdp_group, e.fsdp, e.fsdp_rank
    dev = e.device
    # bf16 parameter shards (and the expert-local region behind them) in symmetric memory
    self.param_sb = SymmetricBuffer(max(e.total_shard, 8), torch.bfloat16, dev, group=self.group)
    # staging slots: the two pool slots shared by layer-sized units, one slot per larger unit
    self.slot_off, self.slot_cap = [], []
    off = 0
    if e.pool_size:
      for _ in range(2):
        self.slot_off.append(off)
        self.slot_cap.append(e.pool_size)
        off += e.pool_size
    for u in e.units:
      if u.big:
        u._rs_slot = len(self.slot_off)
        self.slot_off.append(off)
        self.slot_cap.append(u.total)
        off += u.total
      else:
        u._rs_slot = u.index % 2
    self.n_slots = len(self.slot_off)
    self.stage_sb = SymmetricBuffer(max(off, 8), torch.bfloat16, dev, group=self.group)
    self.flags_sb = SymmetricBuffer(2 * self.n_slots * self.world, torch.int32, dev, group=self.group)
    self.flags_sb.local.zero_()
    self._flag_table = self.flags_sb.ptr_table()
    self.slot_use = [0] * self.n_slots
    self.copy_stream = torch.cuda.Stream(device=dev)    # second lane of the gathers (see gather_shards)
    self.inkernel_wait = os.environ.get("TPB_FSDP_INKERNEL_WAIT", "1") != "0"
    self.push_wgrad = os.environ.get("TPB_FSDP_PUSH_WGRAD", "1") != "0"
    self.peer_embedding = os.environ.get("TPB_FSDP_PEER_EMBEDDING", "1") != "0"
    for u in e.units:
      slots = [s for s in u.slots if not s.local]
      u.peer_lookup = None
      if (self.peer_embedding and getattr(u.module, "supports_peer_lookup", False) and len(u.slots) == 1
          and len(slots) == 1 and len(slots[0].shape) == 2 and slots[0].shape[1] % 8 == 0 and slots[0].tp_dim is None):
        u.peer_lookup = PeerLookup(self, u, slots[0])     # this unit is never gathered
    for u in e.units:
      u._ag_flags = torch.zeros(self.world, dtype=torch.int32, device=dev)
      u._ag_epoch = 0
      u._ag_event = None
      u._pushed = []
    torch.cuda.synchronize(dev)
    self.flags_sb.barrier()
    torch.cuda.synchronize(dev)
    logger.info("FSDP collectives over peer memory: %d ranks, %d staging slots (%.2f GB), backend %s",
                self.world, self.n_slots, off * 2 / 1e9, self.param_sb.backend)

  def close(self):
    torch.cuda.synchronize(self.engine.device)
    for sb in (self.flags_sb, self.stage_sb, self.param_sb):
      sb.close()

  # ------------------------------------------------------------------ step-level ordering
  def params_will_change(self):
    """Every rank's copies out of the parameter shards have finished before anybody overwrites them."""
    self.param_sb.barrier()

  def params_changed(self):
    """Every rank's shards hold the new values before anybody copies them."""
    self.param_sb.barrier()

  # ------------------------------------------------------------------ all-gather
  def issue_gather(self, u, buf: torch.Tensor):
    """Enqueue the gather of unit ``u`` into ``buf`` on the communication stream (the caller has
    ordered that stream after the last reader of ``buf``)."""
    e = self.engine
    L = lib()
    n = u.shard_size
    u._ag_epoch += 1
    u._gather_buf = buf
    s = e.comm_stream.cuda_stream
    nbytes = n * 2
    u._ag_small_event = None
    if self.inkernel_wait and getattr(u.module, "fsdp_inkernel_gather", False):
      for owner, a, cnt in self._small_ranges(u):
        src = self.param_sb.ptrs[owner] + 2 * (u.shard_offset + a - owner * n)
        check(L.tpb_symm_copy(buf.data_ptr() + 2 * a, src, 2 * cnt, s), "fsdp gather copy (small)")
      u._ag_small_event = torch.cuda.Event()
      u._ag_small_event.record(e.comm_stream)
    fork = torch.cuda.Event()
    fork.record(e.comm_stream)
    self.copy_stream.wait_event(fork)
    gather_shards(buf.data_ptr(), [p + u.shard_offset * 2 for p in self.param_sb.ptrs], nbytes,
                  u._ag_flags.data_ptr(), u._ag_epoch, self.rank, (e.comm_stream, self.copy_stream))
    join = torch.cuda.Event()
    join.record(self.copy_stream)
    e.comm_stream.wait_event(join)
    ev = torch.cuda.Event()
    ev.record(e.comm_stream)
    u._ag_event = ev

  def _small_ranges(self, u):
    """(owner, offset, length) of everything in the unit that is not a matrix read by a GEMM: these
    few kilobytes are copied ahead of the shards so that their readers need not wait for the rest."""
    if getattr(u, "_small", None) is None:
      out = []
      for s in u.slots:
        if s.local or len(s.shape) == 2:
          continue
        a, b = s.offset, s.offset + s.numel
        while a < b:
          owner = a // u.shard_size
          end = min(b, (owner + 1) * u.shard_size)
          out.append((owner, a, end - a))
          a = end
      u._small = out
    return u._small

  def wait_small(self, u):
    ev = getattr(u, "_ag_small_event", None)
    if ev is not None:
      torch.cuda.current_stream().wait_event(ev)

  def wait_gather(self, u):
    if u._ag_event is not None:
      torch.cuda.current_stream().wait_event(u._ag_event)

  def gather_context(self, u):
    """A context for in-kernel waits, or None when the unit's readers must wait on the stream."""
    if not (self.inkernel_wait and getattr(u.module, "fsdp_inkernel_gather", False)):
      return None
    return GatherContext(self, u)

  # ------------------------------------------------------------------ reduce-scatter
  def begin_unit_backward(self, u):
    """Before the first gradient of ``u`` is pushed: the owners have drained the previous user of
    the unit's staging slot."""
    sid = u._rs_slot
    self.slot_use[sid] += 1
    u._rs_use = self.slot_use[sid]
    u._pushed = []
    if u._rs_use > 1 and self.world > 1:
      free = self.flags_sb.local.data_ptr() + 4 * (self.n_slots + sid) * self.world
      check(lib().tpb_flag_wait(free, self.world, 1, u._rs_use - 1, _SITE_FREE, _lib.stream_ptr()), "fsdp slot wait")

  def _slot_table(self, u):
    """This rank's staging slot for ``u`` inside every owner's memory."""
    off = self.slot_off[u._rs_slot] + self.rank * u.shard_size
    return self.stage_sb.ptr_table(off)

  def try_push_wgrad(self, u, sink: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor) -> bool:
    """dW = dy2^T @ x2 stored into the owners' staging slots instead of ``sink`` (a view into the
    unit's local gradient buffer, whose position gives the flat offset)."""
    if not self.push_wgrad or sink.dtype != torch.bfloat16 or sink.dim() != 2 or not sink.is_contiguous():
      return False
    full = u.grad_full
    c_off = (sink.data_ptr() - full.data_ptr()) // 2
    rows, cols = sink.shape
    if c_off < 0 or c_off + rows * cols > u.total or cols % 8 or c_off % 8 or rows * cols < (1 << 16):
      return False
    for lo, n in u._pushed:
      if lo < c_off + rows * cols and c_off < lo + n:
        raise _lib.KernelError("a weight received a second gradient after its first one was pushed to the owner; "
                               "run this model with engine.fsdp_collectives=nccl")
    k = dy2.shape[0]
    rc = lib().tpb_gemm_rs_store_bf16(ptr(dy2), ptr(x2), rows, cols, k, dy2.stride(0), x2.stride(0), cols, 1, 1, 1.0,
                                      self._slot_table(u), self.world, u.shard_size, c_off, self.rank,
                                      _lib.stream_ptr())
    check(rc, f"gemm_rs_store M={rows} N={cols} K={k} world={self.world}")
    u._pushed.append((c_off, rows * cols))
    return True

  def check_not_pushed(self, u, sink: torch.Tensor):
    """A gradient is about to be ACCUMULATED into the local buffer: its first part must be there too."""
    c_off = (sink.data_ptr() - u.grad_full.data_ptr()) // 2
    for lo, n in u._pushed:
      if lo < c_off + sink.numel() and c_off < lo + n:
        raise _lib.KernelError("a weight received a second gradient after its first one was pushed to the owner; "
                               "run this model with engine.fsdp_collectives=nccl")

  def _leftover(self, u):
    """Flat ranges of the unit that no GEMM pushed, cut at shard boundaries: (owner, offset, length)."""
    out, pos = [], 0
    for lo, n in sorted(u._pushed) + [(u.total, 0)]:
      a, b = pos, lo
      while a < b:
        owner = a // u.shard_size
        end = min(b, (owner + 1) * u.shard_size)
        out.append((owner, a, end - a))
        a = end
      pos = max(pos, lo + n)
    return out

  def reduce_scatter(self, u, out: torch.Tensor, accumulate: bool):
    """Called when the unit's backward has been enqueued on the compute stream."""
    e = self.engine
    L = lib()
    sid = u._rs_slot
    comm = e.comm_stream
    comm.wait_stream(torch.cuda.current_stream())
    s = comm.cuda_stream
    full = u.grad_full
    for owner, a, n in self._leftover(u):
      dst = self.stage_sb.ptrs[owner] + 2 * (self.slot_off[sid] + self.rank * u.shard_size + a - owner * u.shard_size)
      check(L.tpb_symm_copy(dst, full.data_ptr() + 2 * a, 2 * n, s), "fsdp scatter copy")
    check(L.tpb_peer_signal(self._flag_table, self.world, sid * self.world + self.rank, u._rs_use, s), "fsdp done signal")
    done = self.flags_sb.local.data_ptr() + 4 * sid * self.world
    check(L.tpb_flag_wait(done, self.world, 1, u._rs_use, _SITE_DONE, s), "fsdp done wait")
    stage = self.stage_sb.local.data_ptr() + 2 * self.slot_off[sid]
    check(L.tpb_rs_reduce_bf16(stage, self.world, u.shard_size, u.shard_size, out.data_ptr(),
                               int(out.dtype == torch.float32), int(accumulate), 1.0 / self.world, s), "fsdp reduce")
    check(L.tpb_peer_signal(self._flag_table, self.world, (self.n_slots + sid) * self.world + self.rank, u._rs_use, s),
          "fsdp free signal")
    ev = torch.cuda.Event()
    ev.record(comm)
    return ev


def gemm_ag_wait(ctx: GatherContext, x2, b_offset: int, n: int, k: int, out, epi, aux=None, c2=None):
  """out = epilogue(x2 @ W^T) where W = gathered[b_offset : b_offset + n*k] is still being gathered."""
  m = x2.shape[0]
  rc = lib().tpb_gemm_ag_wait_bf16(ptr(x2), ptr(out), m, n, k, x2.stride(0), out.stride(0), epi, ptr(aux),
                                   aux.stride(0) if aux is not None else 0, ptr(c2),
                                   c2.stride(0) if c2 is not None else 0, ctx.base, b_offset, ctx.world,
                                   ctx.shard_elems, ctx.chunk_elems, ctx.flags.data_ptr(), ctx.epoch,
                                   _lib.stream_ptr())
  check(rc, f"gemm_ag_wait M={m} N={n} K={k} world={ctx.world}")
  return out
