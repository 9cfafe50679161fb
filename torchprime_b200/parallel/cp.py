"""Context parallelism: query rows are sharded over the ``context`` axis, K/V are gathered.

Same flavour as the reference (K/V replicated along the sequence, Q sharded:
configs/model/sharding/llama-fsdp-tp-cp.yaml:22-24, utils/kernel_utils.py:287-316), including
the optional load-balanced (zig-zag) layout in which rank r owns chunks r and 2cp-1-r.  Here
each rank gathers the other ranks' K/V over NVLink (backward: the matching reduce-scatter of
dK/dV; on the fused path through per-source staging slots in peer memory and a fixed-order reduction), restores the natural key order for the zig-zag layout and calls the attention kernel
with the absolute positions of its own query rows, so the kernel's block skipping sees the
true causal structure.  Works for forward and backward (the reference's custom wrapper is
forward-only, kernel_utils.py:124-131).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import functional as ops
from ..utils.parallelism_utils import reorder_sequence
from .collectives import all_gather_dim


class _FusedExchangeAttention(torch.autograd.Function):
  """Causal attention whose forward kernel also performs the K/V exchange: copier CTAs push this
  rank's keys and values into every rank's gathered buffers over NVLink while the attention CTAs
  run.  Backward uses the gathered tensors the forward produced and returns dK/dV to their owners
  with a reduce-scatter."""

  @staticmethod
  def forward(ctx, q, k, v, cpa, pos32, scale):
    from ..ops import attention_sm100 as A
    st = cpa._fused_state(q, k)
    st["epoch"] += 1
    st["k_all"].barrier()            # every rank is done reading the buffers of the previous call
    o, lse = A.attn_fwd_cp(q, k, v, st["k_all"], st["v_all"], st["flags"], pos32, zigzag=cpa.load_balanced,
                           epoch=st["epoch"], copiers=cpa.fused_copiers, scale=scale, multicast=cpa.fused_multicast)
    from ..ops import functional as ops
    ops._ATTN_USED["last"] = "sm100 tcgen05 kernel with the K/V exchange inside (context parallel)"
    b, s_local, hkv, d = k.shape
    sk = s_local * cpa.cp
    # the symmetric buffers are reused by the next layer: keep this layer's gathered K/V for backward
    k_all = st["k_all"].local.view(b, sk, hkv, d).clone()
    v_all = st["v_all"].local.view(b, sk, hkv, d).clone()
    ctx.save_for_backward(q, k_all, v_all, o, lse, pos32)
    ctx.cpa, ctx.scale = cpa, scale
    return o

  @staticmethod
  def backward(ctx, do):
    from ..ops import attention_sm100 as A
    q, k_all, v_all, o, lse, pos32 = ctx.saved_tensors
    cpa = ctx.cpa
    dq, dk_all, dv_all = A.attn_bwd(do, q, k_all, v_all, o, lse, causal=True, scale=ctx.scale, q_pos=pos32)
    if cpa.load_balanced:            # back to rank-major (zig-zag) order, as the owners hold it
      dk_all = reorder_sequence(dk_all, cpa.cp, seq_dim=1, to_contiguous=False)
      dv_all = reorder_sequence(dv_all, cpa.cp, seq_dim=1, to_contiguous=False)
    b, sk, hkv, d = dk_all.shape
    s_local = sk // cpa.cp
    if cpa.peer_scatter:
      dk, dv = cpa._peer_reduce_scatter(dk_all, dv_all)
      return dq, dk, dv, None, None, None

    def scatter(g):
      parts = g.view(b, cpa.cp, s_local, hkv, d).transpose(0, 1).contiguous()   # [cp, b, s_local, ...]
      out = torch.empty(b, s_local, hkv, d, dtype=g.dtype, device=g.device)
      dist.reduce_scatter_tensor(out, parts, group=cpa.group)
      return out

    return dq, scatter(dk_all), scatter(dv_all), None, None, None


class ContextParallelAttention:
  def __init__(self, mesh, load_balanced: bool = False, fused_exchange: bool = False, fused_copiers: int = 16,
               fused_multicast: bool | None = None):
    self.group = mesh.group("context")
    self.cp = mesh.size("context")
    self.rank = mesh.index("context")
    self.load_balanced = load_balanced
    self.fused_exchange = fused_exchange      # K/V exchange inside the attention forward kernel
    self.fused_copiers = fused_copiers
    if fused_multicast is None:
      import os
      fused_multicast = os.environ.get("TPB_CP_MULTICAST", "1" if self.cp > 2 else "0") != "0"
    self.fused_multicast = fused_multicast    # push K/V with one multimem store for all ranks where available
    self._pos_cache = {}
    self._fused = {}
    # backward of the fused path: dK/dV go back to their owners through per-source staging slots in peer
    # memory (copy-engine copies, signal, fixed-order fp32 reduction) instead of an NCCL reduce-scatter
    import os as _os
    self.peer_scatter = fused_exchange and _os.environ.get("TPB_CP_PEER_SCATTER", "1") != "0"
    self._scatter = {}

  def _fused_state(self, q, k):
    """Symmetric gathered K/V buffers and flags for this shape (allocated once, on every rank)."""
    from ..dist.symm import SymmetricBuffer
    b, s_local, hkv, d = k.shape
    key = (b, s_local, hkv, d)
    if key not in self._fused:
      n = b * s_local * self.cp * hkv * d
      flags = SymmetricBuffer(b * s_local * self.cp // 128, torch.int32, q.device, group=self.group)
      flags.local.zero_()
      # with multicast the gathered buffers come from torch's symmetric allocator (it binds them
      # to an NVSwitch multicast object where the platform has one)
      backend = "torch" if self.fused_multicast else None
      self._fused[key] = {"k_all": SymmetricBuffer(n, k.dtype, q.device, group=self.group, backend=backend),
                          "v_all": SymmetricBuffer(n, k.dtype, q.device, group=self.group, backend=backend),
                          "flags": flags, "epoch": 0}
      flags.barrier()
    return self._fused[key]

  def _peer_reduce_scatter(self, dk_all, dv_all):
    """dK/dV of all keys ([b, cp * s_local, hkv, d], this rank's contribution, rank-major row order) ->
    the sum over ranks of the rows this rank owns.  Every rank copies the rows of owner p into its own
    slot of p's staging buffer (copy engines over NVLink; the own rows by a local copy), signals, and the
    owner adds the cp slots in rank order in fp32: deterministic, and no SM moves gradient bytes."""
    from ..dist.symm import SymmetricBuffer
    from ..ops._lib import check, lib, stream_ptr
    from . import fsdp_comm  # noqa: F401  (registers the C signatures)
    dk_all, dv_all = dk_all.contiguous(), dv_all.contiguous()
    b, sk, hkv, d = dk_all.shape
    s_local = sk // self.cp
    n = b * s_local * hkv * d                       # elements of one owner's dK (or dV)
    key = (b, s_local, hkv, d)
    st = self._scatter.get(key)
    dev = dk_all.device
    if st is None:
      st = {"stage": SymmetricBuffer(self.cp * 2 * n, dk_all.dtype, dev, group=self.group),
            "flags": SymmetricBuffer(2 * self.cp, torch.int32, dev, group=self.group), "use": 0}
      st["flags"].local.zero_()
      st["table"] = st["flags"].ptr_table()
      st["flags"].barrier()
      self._scatter[key] = st
    L, s = lib(), stream_ptr()
    st["use"] += 1
    use = st["use"]
    flags = st["flags"].local.data_ptr()
    if use > 1:      # every owner has reduced the previous contents of its staging buffer
      check(L.tpb_flag_wait(flags + 4 * self.cp, self.cp, 1, use - 1, 93, s), "cp scatter slot wait")
    row = hkv * d
    for j in range(self.cp):
      p = (self.rank + j) % self.cp
      base = st["stage"].ptrs[p] + 2 * (self.rank * 2 * n)
      for which, g in enumerate((dk_all, dv_all)):
        for bi in range(b):
          src = g.data_ptr() + 2 * ((bi * sk + p * s_local) * row)
          dst = base + 2 * (which * n + bi * s_local * row)
          check(L.tpb_symm_copy(dst, src, 2 * s_local * row, s), "cp scatter copy")
    check(L.tpb_peer_signal(st["table"], self.cp, self.rank, use, s), "cp scatter done signal")
    check(L.tpb_flag_wait(flags, self.cp, 1, use, 94, s), "cp scatter done wait")
    out = torch.empty(2, b, s_local, hkv, d, dtype=dk_all.dtype, device=dev)
    check(L.tpb_rs_reduce_bf16(st["stage"].local.data_ptr(), self.cp, 2 * n, 2 * n, out.data_ptr(), 0, 0, 1.0, s),
          "cp scatter reduce")
    check(L.tpb_peer_signal(st["table"], self.cp, self.cp + self.rank, use, s), "cp scatter free signal")
    return out[0], out[1]

  def _can_fuse(self, q, k, v, segment_ids) -> bool:
    if not (self.fused_exchange and q.is_cuda and segment_ids is None and ops.use_kernels(q, k, v)):
      return False
    s_local = k.shape[1]
    return (q.shape[-1] == 128 and v.shape[-1] == 128 and q.dtype == torch.bfloat16
            and s_local % (256 if self.load_balanced else 128) == 0)

  def query_positions(self, s_local: int, device) -> torch.Tensor:
    """Absolute positions of this rank's rows, [s_local] int64."""
    key = (s_local, str(device))
    if key not in self._pos_cache:
      if self.load_balanced:
        half = s_local // 2
        a = torch.arange(self.rank * half, (self.rank + 1) * half, device=device)
        c = 2 * self.cp - 1 - self.rank
        b = torch.arange(c * half, (c + 1) * half, device=device)
        pos = torch.cat([a, b])
      else:
        pos = torch.arange(self.rank * s_local, (self.rank + 1) * s_local, device=device)
      self._pos_cache[key] = pos
    return self._pos_cache[key]

  def attention(self, q, k, v, segment_ids=None, scale=None):
    b, s_local = q.shape[0], q.shape[1]
    if self._can_fuse(q, k, v, segment_ids):
      pos32 = self.query_positions(s_local, q.device)[None].expand(b, s_local).to(torch.int32).contiguous()
      return _FusedExchangeAttention.apply(q, k, v, self, pos32, scale)
    k_all = all_gather_dim(k.contiguous(), self.group, 1)
    v_all = all_gather_dim(v.contiguous(), self.group, 1)
    kv_seg = None
    if segment_ids is not None:
      kv_seg = all_gather_dim(segment_ids.contiguous(), self.group, 1)
    if self.load_balanced:
      k_all = reorder_sequence(k_all, self.cp, seq_dim=1, to_contiguous=True)
      v_all = reorder_sequence(v_all, self.cp, seq_dim=1, to_contiguous=True)
      if kv_seg is not None:
        kv_seg = reorder_sequence(kv_seg, self.cp, seq_dim=1, to_contiguous=True)
    pos = self.query_positions(s_local, q.device)
    return ops.attention(q, k_all, v_all, causal=True, scale=scale, q_segment_ids=segment_ids,
                         kv_segment_ids=kv_seg, q_positions=pos[None].expand(b, s_local))
