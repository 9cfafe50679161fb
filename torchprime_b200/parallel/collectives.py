"""Autograd-aware collectives used by the tensor / expert / context parallel code paths.

The reference never writes these: XLA's SPMD partitioner inserts them from sharding annotations
(docs/sharding.md:12-16).  With one process per GPU they are explicit, and each has the matching
collective as its backward (all-reduce <-> identity, all-gather <-> reduce-scatter,
all-to-all <-> all-to-all).  All of them work on NCCL and on gloo (CPU test ranks).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def _size(group) -> int:
  return dist.get_world_size(group) if (dist.is_initialized() and group is not None) else 1


class _AllReduceFwd(torch.autograd.Function):
  """forward: sum over the group; backward: identity (row-parallel linear output)."""

  @staticmethod
  def forward(ctx, x, group):
    y = x.contiguous().clone()
    dist.all_reduce(y, group=group)
    return y

  @staticmethod
  def backward(ctx, g):
    return g, None


class _AllReduceBwd(torch.autograd.Function):
  """forward: identity; backward: sum over the group (input of a column-parallel linear)."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return x

  @staticmethod
  def backward(ctx, g):
    g = g.contiguous().clone()
    dist.all_reduce(g, group=ctx.group)
    return g, None


def reduce_from_tp(x, group):
  return x if _size(group) == 1 else _AllReduceFwd.apply(x, group)


def copy_to_tp(x, group):
  return x if _size(group) == 1 else _AllReduceBwd.apply(x, group)


def _all_gather_cat(x, group, dim):
  n = _size(group)
  parts = [torch.empty_like(x) for _ in range(n)]
  dist.all_gather(parts, x.contiguous(), group=group)
  return torch.cat(parts, dim=dim)


class _AllGatherDim(torch.autograd.Function):
  """forward: concatenate the group's tensors along ``dim``; backward: sum and keep the own slice."""

  @staticmethod
  def forward(ctx, x, group, dim):
    ctx.group, ctx.dim, ctx.n = group, dim, x.shape[dim]
    return _all_gather_cat(x, group, dim)

  @staticmethod
  def backward(ctx, g):
    n = _size(ctx.group)
    r = dist.get_rank(ctx.group)
    g = g.contiguous().clone()
    dist.all_reduce(g, group=ctx.group)
    return g.narrow(ctx.dim, r * ctx.n, ctx.n).contiguous(), None, None


def all_gather_dim(x, group, dim):
  return x if _size(group) == 1 else _AllGatherDim.apply(x, group, dim)


class _AllToAllRows(torch.autograd.Function):
  """Variable-size all-to-all over rows (dim 0); backward swaps the split lists."""

  @staticmethod
  def forward(ctx, x, in_splits, out_splits, group):
    ctx.group, ctx.in_splits, ctx.out_splits = group, in_splits, out_splits
    out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
    dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits,
                           group=group)
    return out

  @staticmethod
  def backward(ctx, g):
    out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
    dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.in_splits, input_split_sizes=ctx.out_splits,
                           group=ctx.group)
    return out, None, None, None


def all_to_all_rows(x, in_splits, out_splits, group):
  if dist.get_backend(group) == "gloo":
    return _AllToAllRowsGloo.apply(x, in_splits, out_splits, group)
  return _AllToAllRows.apply(x, in_splits, out_splits, group)


def _gloo_a2a(x, in_splits, out_splits, group):
  """gloo has no all_to_all_single: emulate with an all-gather of padded chunks."""
  n = dist.get_world_size(group)
  r = dist.get_rank(group)
  all_in = [None] * n
  dist.all_gather_object(all_in, list(in_splits), group=group)
  mx = max(max(s) if s else 0 for s in all_in)
  pad = x.new_zeros((n, mx) + tuple(x.shape[1:]))
  off = 0
  for j, s in enumerate(in_splits):
    pad[j, :s] = x[off:off + s]
    off += s
  gathered = [torch.empty_like(pad) for _ in range(n)]
  dist.all_gather(gathered, pad, group=group)
  return torch.cat([gathered[src][r, :all_in[src][r]] for src in range(n)], dim=0)


class _AllToAllRowsGloo(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, in_splits, out_splits, group):
    ctx.group, ctx.in_splits, ctx.out_splits = group, in_splits, out_splits
    return _gloo_a2a(x, in_splits, out_splits, group)

  @staticmethod
  def backward(ctx, g):
    return _gloo_a2a(g.contiguous(), ctx.out_splits, ctx.in_splits, ctx.group), None, None, None
