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

from ..ops import _lib
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

  def exchange_blocks(self, x, desc, n_blocks: int, n_out: int, zero_rows=None):
    """Block form (not differentiable; the expert-parallel MLP function drives it in both passes):
    ``x`` rows are ``n_blocks`` consecutive blocks described by the device tensor ``desc`` (int64:
    ``start[n_blocks+1]``, ``dst_rank[n_blocks]`` (-1: skip), ``dst_row0[n_blocks]``).  Returns a
    copy of the first ``n_out`` rows of this rank's receive buffer with ``zero_rows`` cleared."""
    import ctypes

    from ..ops import _debug, _lib
    from ..ops._lib import check, lib, ptr, stream_ptr
    assert n_out <= self.max_rows, f"receive buffer holds {self.max_rows} rows, {n_out} needed"
    assert x.shape[1] == self.dim and x.is_contiguous() and desc.numel() == 3 * n_blocks + 1
    P, I, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint
    _lib.register_signature("tpb_a2a_push_blocks", [P, I, I, I, I, I, P, P, P, U, P, P])
    _lib.register_signature("tpb_a2a_wait", [P, I, U, P])
    _debug.check_exchange_descriptors("a2a_push_blocks", desc, n_blocks, x.shape[0], self.world, self.max_rows)
    self.epoch += 1
    self.recv.barrier()            # nobody is still reading its receive buffer from the previous exchange
    check(lib().tpb_a2a_push_blocks(ptr(x), x.shape[0], self.dim, n_blocks, self.world, self.rank, ptr(desc),
                                    self.recv.ptr_table(), self.flags.ptr_table(), self.epoch, ptr(self.counter),
                                    stream_ptr()), "a2a_push_blocks")
    check(lib().tpb_a2a_wait(ptr(self.flags.local), self.world, self.epoch, stream_ptr()), "a2a_wait")
    out = self.recv.local[: n_out * self.dim].view(n_out, self.dim).clone()
    if zero_rows is not None:
      out.index_fill_(0, zero_rows, 0)
    return out

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


def _prefix(v):
  out = [0]
  for a in v:
    out.append(out[-1] + int(a))
  return out


class _ExchangePlan:
  """Host-side description of one dispatch / return pair, computed from the count matrix
  ``C[s][e]`` (pairs of rank s routed to global expert e), the same on every rank.

  Send layout (on every rank): its pairs sorted by expert, compact.  Receive layout on the owner:
  expert-major, every expert's segment padded to a multiple of ``row_align`` (128 or 256) rows, inside
  a segment the rows of source 0, 1, ... in order.  So rows arrive grouped for the grouped GEMMs,
  whatever rank they came from, and no expert ids travel."""

  def __init__(self, C, me: int, ep: int, el: int, device):
    import numpy as np
    E = ep * el
    C = np.asarray(C, dtype=np.int64).reshape(ep, E)
    tot = C.sum(axis=0).reshape(ep, el)                              # rows owner r receives for its expert j
    # 256-row segments (CTA-pair GEMM tiles) when experts see about a thousand rows or more; the
    # choice is made from the whole matrix, so every rank pads every owner's layout the same way
    al = 256 if int(tot.sum()) // E >= 1024 else 128
    self.row_align = al
    padded = (tot + al - 1) // al * al
    offpad = np.zeros((ep, el + 1), dtype=np.int64)
    offpad[:, 1:] = np.cumsum(padded, axis=1)
    send_off = np.zeros((ep, E + 1), dtype=np.int64)
    send_off[:, 1:] = np.cumsum(C, axis=1)
    before_me = C[:me].sum(axis=0)                                   # rows of lower ranks inside each segment
    # dispatch: one block per global expert, in send order
    owner = np.arange(E) // el
    row0 = offpad[owner, np.arange(E) % el] + before_me
    dispatch = np.concatenate([send_off[me], owner, row0])
    self.dispatch_blocks = E
    self.n_send = int(send_off[me, -1])
    # return: walk the receive layout; padding rows form blocks that go nowhere (rank -1)
    mine = C[:, me * el:(me + 1) * el]                               # [source, local expert]
    within = np.zeros((el, ep + 1), dtype=np.int64)
    within[:, 1:] = np.cumsum(mine.T, axis=1)
    start = (offpad[me, :el, None] + within).reshape(-1)             # per expert: ep source blocks + the padding block
    rank = np.tile(np.concatenate([np.arange(ep), [-1]]), el)
    src_row0 = np.concatenate([send_off[:, me * el:(me + 1) * el].T, np.zeros((el, 1), dtype=np.int64)], axis=1)
    ret = np.concatenate([start, [offpad[me, el]], rank, src_row0.reshape(-1)])
    self.ret_blocks = el * (ep + 1)
    self.n_pad = int(offpad[me, el])
    pad_lo, pad_hi = offpad[me, :el] + tot[me], offpad[me, 1:]
    zero = np.concatenate([np.arange(a, b) for a, b in zip(pad_lo, pad_hi)]) if self.n_pad else np.zeros(0, np.int64)
    tiles = np.repeat(np.arange(el), (padded[me] // 128))
    # one host-to-device copy for everything
    packed = torch.from_numpy(np.concatenate([dispatch, ret, zero, tiles, offpad[me]]).astype(np.int64))
    if torch.device(device).type == "cuda":
      packed = packed.pin_memory().to(device, non_blocking=True)
    n_d, n_r, n_z, n_t = dispatch.size, ret.size, zero.size, tiles.size
    self.dispatch = packed[:n_d]
    self.ret = packed[n_d:n_d + n_r]
    self.zero_rows = packed[n_d + n_r:n_d + n_r + n_z] if n_z else None
    self.tile_expert = packed[n_d + n_r + n_z:n_d + n_r + n_z + n_t].to(torch.int32)
    self.k_offsets = packed[n_d + n_r + n_z + n_t:].to(torch.int32)
    self.num_rows = self.n_pad


class _EPGroupedMLPFn(torch.autograd.Function):
  """Routed SwiGLU experts across the expert group with this framework's own exchange kernels in both
  passes: sort pairs by expert, push rows to the owners (they land grouped by expert), grouped
  GEMMs, push results back, weighted combine.  One host synchronisation per call (the count matrix)."""

  @staticmethod
  def forward(ctx, x, weights, w_gate, w_up, w_down, epm, idx, fused_gate_up):
    t, k = idx.shape
    dev = x.device
    flat = idx.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=epm.num_experts)
    cm = torch.empty(epm.ep, epm.num_experts, dtype=counts.dtype, device=dev)
    dist.all_gather_into_tensor(cm, counts, group=epm.group)
    plan = _ExchangePlan(cm.tolist(), epm.rank, epm.ep, epm.local_experts, dev)
    src_tok = (order // k).to(torch.int32).contiguous()
    dest_pos = torch.empty(t * k, dtype=torch.int32, device=dev)
    dest_pos[order] = torch.arange(t * k, dtype=torch.int32, device=dev)
    dest_pos = dest_pos.view(t, k)
    a2a_d, a2a_r = epm._push_pair(t, k, x.shape[-1], dev)
    send = moe_ops.gather_rows(x, src_tok)
    xg = a2a_d.exchange_blocks(send, plan.dispatch, plan.dispatch_blocks, plan.n_pad, plan.zero_rows)
    need_grad = any(ctx.needs_input_grad)
    gu = act = None
    if plan.n_pad > 0:
      n2 = w_gate.shape[2] if fused_gate_up else 2 * w_gate.shape[2]
      gu = torch.empty(plan.n_pad, n2, dtype=x.dtype, device=dev) if need_grad else None
      act = moe_ops.grouped_gemm_rows(xg, w_gate, plan, b_mn=True, b2=None if fused_gate_up else w_up,
                                      epi=_lib.EPI_SWIGLU, c2=gu, n_total=n2)
      rows = moe_ops.grouped_gemm_rows(act, w_down, plan, b_mn=True)
    else:
      rows = xg
    back = a2a_r.exchange_blocks(rows, plan.ret, plan.ret_blocks, t * k)
    y = moe_ops.combine_rows(back, dest_pos, weights)
    ctx.epm, ctx.plan, ctx.fused, ctx.tk = epm, plan, fused_gate_up, (t, k)
    if need_grad:
      ctx.save_for_backward(weights, w_gate, w_up, w_down, xg, gu, act, back, order, src_tok, dest_pos)
    return y

  @staticmethod
  def backward(ctx, dy):
    from ..ops import kernels as kk
    weights, w_gate, w_up, w_down, xg, gu, act, back, order, src_tok, dest_pos = ctx.saved_tensors
    epm, plan, fused = ctx.epm, ctx.plan, ctx.fused
    t, k = ctx.tk
    dy = dy.contiguous()
    a2a_d, a2a_r = epm._push_pair(t, k, dy.shape[-1], dy.device)
    dweights = moe_ops.combine_dw(back, dest_pos, dy) if ctx.needs_input_grad[1] else None
    w_sorted = weights.reshape(-1)[order].float().contiguous()
    d_back = moe_ops.gather_rows(dy, src_tok, w_sorted)
    d_rows = a2a_d.exchange_blocks(d_back, plan.dispatch, plan.dispatch_blocks, plan.n_pad, plan.zero_rows)
    deliver = moe_ops._deliver_wgrad
    if plan.n_pad > 0:
      f = gu.shape[1] // 2
      dact = moe_ops.grouped_gemm_rows(d_rows, w_down, plan, b_mn=False)
      g_down = deliver(w_down, lambda out, acc: moe_ops.grouped_gemm_wgrad(act, d_rows, plan, out, acc))
      dgu = kk.swiglu_bwd(dact, gu)
      if fused:
        d_xg = moe_ops.grouped_gemm_rows(dgu, w_gate, plan, b_mn=False)
        g_gate = deliver(w_gate, lambda out, acc: moe_ops.grouped_gemm_wgrad(xg, dgu, plan, out, acc))
        g_up = None
      else:
        dg, du = dgu[:, :f], dgu[:, f:]
        d_xg = moe_ops.grouped_gemm_rows(dg, w_gate, plan, b_mn=False)
        moe_ops.grouped_gemm_rows(du, w_up, plan, b_mn=False, epi=_lib.EPI_BF16_ACC, out=d_xg)
        g_gate = deliver(w_gate, lambda out, acc: moe_ops.grouped_gemm_wgrad(xg, dg, plan, out, acc))
        g_up = deliver(w_up, lambda out, acc: moe_ops.grouped_gemm_wgrad(xg, du, plan, out, acc))
    else:
      d_xg = d_rows
      zero = lambda out, acc: None if acc else out.zero_()   # noqa: E731
      g_down, g_gate = deliver(w_down, zero), deliver(w_gate, zero)
      g_up = None if fused else deliver(w_up, zero)
    d_send = a2a_r.exchange_blocks(d_xg, plan.ret, plan.ret_blocks, t * k)
    dx = moe_ops.combine_rows(d_send, dest_pos, None) if ctx.needs_input_grad[0] else None
    return dx, dweights, g_gate, g_up, g_down, None, None, None


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
      self._push[key] = (PushAllToAll(self.group, self.ep * t * k + self.local_experts * 256, dim, device),
                         PushAllToAll(self.group, t * k, dim, device))
    return self._push[key]

  def grouped_mlp(self, x, weights, idx, w_gate, w_up, w_down, capacity=None, rows_per_group=None,
                  fused_gate_up=False):
    """Same contract as :func:`ops.moe.grouped_mlp` but ``w_*`` hold only the local experts."""
    t, k = idx.shape
    e, el = self.num_experts, self.local_experts
    if (self.fused_exchange and capacity is None and x.is_cuda and x.dtype == torch.bfloat16
        and x.shape[-1] % 64 == 0 and w_down.shape[1] % 64 == 0 and dist.get_backend(self.group) == "nccl"
        and moe_ops._kernels_ok(x, w_gate, w_down)):
      wu = w_gate if fused_gate_up else w_up
      return _EPGroupedMLPFn.apply(x.contiguous(), weights.float().contiguous(), w_gate, wu, w_down, self,
                                   idx, fused_gate_up)
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
