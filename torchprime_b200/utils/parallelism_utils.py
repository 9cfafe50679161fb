"""Context-parallel sequence layout helpers.

Load-balanced ("zig-zag") context parallelism splits the sequence into ``2*cp`` chunks
and gives rank r the chunks ``r`` and ``2*cp-1-r`` so every rank owns the same amount of
causal attention work.  Same layout and function names as the reference
(torchprime/utils/parallelism_utils.py:14-205): ``reorder_sequence(...,
to_contiguous=False)`` applies the permutation ``[0, 2cp-1, 1, 2cp-2, ...]`` over chunks,
``to_contiguous=True`` applies its inverse; ``reorder_mask`` is the numpy twin.
``LoadBalancedCausalMask`` describes the resulting mask (query row ids permuted, key ids
in natural order) for kernels and oracles.
"""

from __future__ import annotations

import numpy as np
import torch


def _zigzag_chunks(cp_size: int) -> list[int]:
  order = []
  for r in range(cp_size):
    order += [r, 2 * cp_size - 1 - r]
  return order


def _check(shape, seq_dim: int, cp_size: int):
  if cp_size % 2 != 0:
    raise ValueError(f"cp_size={cp_size} must be a multiple of 2.")
  if shape[seq_dim] % (cp_size * 2) != 0:
    raise ValueError(f"tensor.shape={tuple(shape)} is not a multiple of cp_size*2={cp_size * 2}")


def chunk_permutation(cp_size: int, to_contiguous: bool) -> list[int]:
  fwd = _zigzag_chunks(cp_size)
  if not to_contiguous:
    return fwd
  inv = [0] * len(fwd)
  for dst, src in enumerate(fwd):
    inv[src] = dst
  return inv


def reorder_sequence(tensor: torch.Tensor, cp_size: int, seq_dim: int = 1, to_contiguous: bool = False):
  """Permute ``2*cp_size`` equal chunks of ``seq_dim`` into (or out of) the zig-zag order."""
  if tensor is None:
    return None
  seq_dim = seq_dim % tensor.dim()
  _check(tensor.shape, seq_dim, cp_size)
  shape = tensor.shape
  chunks = tensor.reshape(*shape[:seq_dim], 2 * cp_size, shape[seq_dim] // (2 * cp_size), *shape[seq_dim + 1:])
  index = torch.tensor(chunk_permutation(cp_size, to_contiguous), device=tensor.device)
  return torch.index_select(chunks, seq_dim, index).reshape(shape)


def reorder_mask(array: np.ndarray, cp_size: int, seq_dim: int):
  """numpy version of the forward permutation (used on position-id vectors)."""
  seq_dim = seq_dim % array.ndim
  _check(array.shape, seq_dim, cp_size)
  shape = array.shape
  chunks = array.reshape(*shape[:seq_dim], 2 * cp_size, shape[seq_dim] // (2 * cp_size), *shape[seq_dim + 1:])
  return np.take(chunks, np.asarray(_zigzag_chunks(cp_size)), axis=seq_dim).reshape(shape)


class LoadBalancedCausalMask:
  """Causal mask for zig-zag ordered queries against naturally ordered keys:
  ``mask[i, j] = q_sequence[i] >= j`` with ``q_sequence = zigzag(arange(S))``."""

  def __init__(self, shape: tuple[int, int], offset: int = 0, shard_count: int = 1, cp_size: int = 4):
    self.shape = tuple(shape)
    self.offset = offset
    self.shard_count = shard_count
    self.cp_size = cp_size
    self.q_sequence = reorder_mask(np.arange(shape[0], dtype=np.int32), cp_size, 0)

  def as_array(self) -> np.ndarray:
    kv = np.arange(self.shape[1], dtype=np.int32)
    return (self.q_sequence[:, None] + self.offset) >= kv[None, :]

  def __eq__(self, other):
    return (isinstance(other, LoadBalancedCausalMask) and self.shape == other.shape and self.offset == other.offset
            and np.array_equal(self.q_sequence, other.q_sequence))

  def __hash__(self):
    return hash((type(self), self.shape, self.offset, self.q_sequence.tobytes()))


def cp_enabled(config) -> bool:
  return "context" in config.ici_mesh and config.ici_mesh.context > 1


def lb_cp_enabled(config) -> bool:
  return cp_enabled(config) and bool(config.model.get("load_balance_cp", False))
