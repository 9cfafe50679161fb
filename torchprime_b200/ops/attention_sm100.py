"""Python side of the sm_100a flash-attention kernels (csrc/attention_sm100.cu)."""

from __future__ import annotations


def supported(q, k, v, causal, window, q_segment_ids, softcap, q_positions, kv_positions) -> bool:
  return False


def attention(q, k, v, **kwargs):
  raise NotImplementedError
