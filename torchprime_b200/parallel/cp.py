"""Context parallelism: query rows are sharded over the ``context`` axis, K/V are gathered.

Same flavour as the reference (K/V replicated along the sequence, Q sharded:
configs/model/sharding/llama-fsdp-tp-cp.yaml:22-24, utils/kernel_utils.py:287-316), including
the optional load-balanced (zig-zag) layout in which rank r owns chunks r and 2cp-1-r.  Here
each rank gathers the other ranks' K/V over NVLink (backward: the matching reduce-scatter of
dK/dV), restores the natural key order for the zig-zag layout and calls the attention kernel
with the absolute positions of its own query rows, so the kernel's block skipping sees the
true causal structure.  Works for forward and backward (the reference's custom wrapper is
forward-only, kernel_utils.py:124-131).
"""

from __future__ import annotations

import torch

from ..ops import functional as ops
from ..utils.parallelism_utils import reorder_sequence
from .collectives import all_gather_dim


class ContextParallelAttention:
  def __init__(self, mesh, load_balanced: bool = False):
    self.group = mesh.group("context")
    self.cp = mesh.size("context")
    self.rank = mesh.index("context")
    self.load_balanced = load_balanced
    self._pos_cache = {}

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
