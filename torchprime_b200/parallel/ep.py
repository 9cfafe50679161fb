"""Expert parallelism: every rank of the expert group owns ``E / ep`` experts; tokens travel to the
owner of their expert and back with two all-to-alls around the local grouped MLP.

The reference expresses this with resharding annotations that XLA turns into all-to-alls
(model/llama4/model.py:259-321, model/mixtral/model.py:802-834).  Here the exchange is explicit:
(token, slot) pairs are sorted by destination rank then expert, row counts are exchanged, rows move
with one variable-size all-to-all, the local experts run through the grouped tcgen05 GEMMs
(ops/moe.py), results return with the mirrored all-to-all and are combined with the routing
weights on the source rank.  Gradients flow through the same path (all-to-all is its own adjoint).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import moe as moe_ops
from .collectives import all_to_all_rows


class PushAllToAll:
  """Variable-size all-to-all of bf16 rows done by this framework's own kernel: every rank stores the
  block meant for rank r straight into r's receive buffer over NVLink (plain 16-byte stores, posted
  writes) and raises a flag there; the receiver waits (bounded, on the stream) for all sources.
  Receive buffer, flags and the completion counter live in symmetric memory and are allocated once
  for ``max_rows`` rows.  Differentiable: the backward is the mirrored NCCL all-to-all."""

  def __init__(self, group, max_rows: int, dim: int, device, dtype=torch.bfloat16):
    from ..dist.symm import SymmetricBuffer
    self.group, self.dim, self.max_rows = group, dim, max_rows
    self.recv = SymmetricBuffer(max_rows * dim, dtype, device, group=group)
    self.flags = SymmetricBuffer(8, torch.int32, device, group=group)
    self.flags.local.zero_()
    self.counter = torch.zeros(1, dtype=torch.int32, device=device)
    self.world, self.rank = self.recv.world, self.recv.rank
    self.epoch = 0
    self.flags.barrier()

  def exchange(self, x, count_matrix):
    """``x``: rows sorted by destination rank; ``count_matrix[s][r]``: rows rank s sends to rank r
    (host integers, the same on every rank).  Returns the rows this rank receives, source-major."""
    return _PushAllToAllFn.apply(x, self, count_matrix)


class _PushAllToAllFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, a2a, m):
    import ctypes

    from ..ops import _lib
    from ..ops._lib import check, lib, ptr, stream_ptr
    me, world = a2a.rank, a2a.world
    in_splits = [int(m[me][r]) for r in range(world)]
    out_splits = [int(m[s][me]) for s in range(world)]
    n_recv = sum(out_splits)
    assert n_recv <= a2a.max_rows, f"receive buffer holds {a2a.max_rows} rows, {n_recv} arrive"
    assert x.shape[0] == sum(in_splits) and x.shape[1] == a2a.dim and x.is_contiguous()
    src_start = (ctypes.c_int * (world + 1))(*([0] + [sum(in_splits[:r + 1]) for r in range(world)]))
    dst_row0 = (ctypes.c_longlong * world)(*[sum(int(m[s][r]) for s in range(me)) for r in range(world)])
    a2a.epoch += 1
    a2a.recv.barrier()             # nobody is still reading its receive buffer from the previous exchange
    _lib.register_signature("tpb_a2a_push_rows", [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                  ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                  ctypes.c_uint, ctypes.c_void_p, ctypes.c_void_p])
    _lib.register_signature("tpb_a2a_wait", [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_void_p])
    check(lib().tpb_a2a_push_rows(ptr(x), x.shape[0], a2a.dim, world, me, src_start, dst_row0, a2a.recv.ptr_table(),
                                  a2a.flags.ptr_table(), a2a.epoch, ptr(a2a.counter), stream_ptr()), "a2a_push_rows")
    check(lib().tpb_a2a_wait(ptr(a2a.flags.local), world, a2a.epoch, stream_ptr()), "a2a_wait")
    ctx.group, ctx.in_splits, ctx.out_splits = a2a.group, in_splits, out_splits
    return a2a.recv.local[: n_recv * a2a.dim].view(n_recv, a2a.dim).clone()

  @staticmethod
  def backward(ctx, g):
    out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
    dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.in_splits, input_split_sizes=ctx.out_splits,
                           group=ctx.group)
    return out, None, None


class ExpertParallelMLP:
  def __init__(self, mesh, num_experts: int, fused_exchange: bool = False):
    self.group = mesh.group("expert")
    self.ep = mesh.size("expert")
    self.rank = mesh.index("expert")
    self.num_experts = num_experts
    assert num_experts % self.ep == 0, f"{num_experts} experts not divisible by expert axis {self.ep}"
    self.local_experts = num_experts // self.ep
    self.fused_exchange = fused_exchange     # dispatch / return by PushAllToAll instead of NCCL
    self._push = {}

  def _push_pair(self, t, k, dim, device):
    """Dispatch and return exchangers for ``t`` tokens of ``k`` slots (worst case: every pair of
    every rank lands on one rank)."""
    key = (t, k, dim)
    if key not in self._push:
      self._push[key] = (PushAllToAll(self.group, self.ep * t * k, dim, device),
                         PushAllToAll(self.group, t * k, dim, device))
    return self._push[key]

  def grouped_mlp(self, x, weights, idx, w_gate, w_up, w_down, capacity=None, rows_per_group=None,
                  fused_gate_up=False):
    """Same contract as :func:`ops.moe.grouped_mlp` but ``w_*`` hold only the local experts."""
    t, k = idx.shape
    e, el = self.num_experts, self.local_experts
    flat = idx.reshape(-1).long()
    keep = torch.ones_like(flat, dtype=torch.bool)
    if capacity is not None:
      keep = (moe_ops.build_dispatch_plan(idx, e, capacity, rows_per_group).dest >= 0).reshape(-1)
    key = torch.where(keep, flat, torch.full_like(flat, e))
    order = torch.argsort(key, stable=True)
    counts = torch.bincount(key, minlength=e + 1)[:e]
    n_send = int(counts.sum().item())
    order = order[:n_send]
    send_rows = x[order // k]
    send_expert = (key[order] % el).to(torch.int32)
    per_rank = counts.view(self.ep, el).sum(1)
    in_splits = [int(v) for v in per_rank.tolist()]
    recv_counts = torch.empty_like(per_rank)
    if dist.get_backend(self.group) == "gloo":
      gathered = [torch.empty_like(per_rank) for _ in range(self.ep)]
      dist.all_gather(gathered, per_rank, group=self.group)
      recv_counts = torch.stack(gathered)[:, self.rank].contiguous()
    else:
      dist.all_to_all_single(recv_counts, per_rank, group=self.group)
    out_splits = [int(v) for v in recv_counts.tolist()]
    push = None
    if (self.fused_exchange and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0
        and dist.get_backend(self.group) == "nccl"):
      # the full count matrix lets every rank compute where its block starts in each receive buffer
      cm = [torch.empty_like(per_rank) for _ in range(self.ep)]
      dist.all_gather(cm, per_rank, group=self.group)
      matrix = torch.stack(cm).tolist()
      push = self._push_pair(t, k, x.shape[-1], x.device)
      rows = push[0].exchange(send_rows.contiguous(), matrix)
    else:
      rows = all_to_all_rows(send_rows, in_splits, out_splits, self.group)
    experts = all_to_all_rows(send_expert.view(-1, 1), in_splits, out_splits, self.group).view(-1)
    ones = torch.ones(rows.shape[0], 1, dtype=torch.float32, device=x.device)
    if rows.shape[0] > 0:
      y_rows = moe_ops.grouped_mlp(rows, ones, experts.view(-1, 1).to(torch.int32), w_gate, w_up, w_down,
                                   fused_gate_up=fused_gate_up)
    else:
      y_rows = rows.new_zeros(rows.shape) + 0.0 * (w_gate.sum() + w_down.sum() + (0 if fused_gate_up else w_up.sum()))
    if push is not None:
      back = push[1].exchange(y_rows.contiguous(), [list(col) for col in zip(*matrix)])
    else:
      back = all_to_all_rows(y_rows, out_splits, in_splits, self.group)
    # weighted combine on the source rank
    w_flat = weights.reshape(-1)[order].to(back.dtype)
    out = torch.zeros(t, x.shape[-1], dtype=torch.float32, device=x.device)
    out.index_add_(0, order // k, (back * w_flat[:, None]).float())
    return out.to(x.dtype)
