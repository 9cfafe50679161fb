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


class ExpertParallelMLP:
  def __init__(self, mesh, num_experts: int):
    self.group = mesh.group("expert")
    self.ep = mesh.size("expert")
    self.rank = mesh.index("expert")
    self.num_experts = num_experts
    assert num_experts % self.ep == 0, f"{num_experts} experts not divisible by expert axis {self.ep}"
    self.local_experts = num_experts // self.ep

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
    rows = all_to_all_rows(send_rows, in_splits, out_splits, self.group)
    experts = all_to_all_rows(send_expert.view(-1, 1), in_splits, out_splits, self.group).view(-1)
    ones = torch.ones(rows.shape[0], 1, dtype=torch.float32, device=x.device)
    if rows.shape[0] > 0:
      y_rows = moe_ops.grouped_mlp(rows, ones, experts.view(-1, 1).to(torch.int32), w_gate, w_up, w_down,
                                   fused_gate_up=fused_gate_up)
    else:
      y_rows = rows.new_zeros(rows.shape) + 0.0 * (w_gate.sum() + w_down.sum() + (0 if fused_gate_up else w_up.sum()))
    back = all_to_all_rows(y_rows, out_splits, in_splits, self.group)
    # weighted combine on the source rank
    w_flat = weights.reshape(-1)[order].to(back.dtype)
    out = torch.zeros(t, x.shape[-1], dtype=torch.float32, device=x.device)
    out.index_add_(0, order // k, (back * w_flat[:, None]).float())
    return out.to(x.dtype)
