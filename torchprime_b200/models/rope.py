"""Rotary-embedding frequency schedules and cos/sin tables.

Schedules: plain (``theta^(-2i/d)``), Llama-3.1 band-wise rescaling and YaRN
(DeepSeek).  Same numerical definitions as the reference's
torchprime/rope/rope.py:22-177; tables here are fp32 ``[max_pos, d/2]`` and are
consumed by the RoPE kernel (the reference materialises ``cat(freqs, freqs)`` in
the activation dtype, torchprime/torch_xla_models/model/llama/model.py:68-88).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass(kw_only=True)
class RopeScaling:
  """Llama-3.1 defaults."""
  factor: float = 8.0
  low_freq_factor: float = 1.0
  high_freq_factor: float = 4.0
  original_context_len: int = 8192


def default_rope_frequencies(head_dim: int, theta: float = 10000.0) -> torch.Tensor:
  exponent = torch.arange(0, head_dim, 2, dtype=torch.int64, device="cpu").float() / head_dim
  return 1.0 / (theta ** exponent)


def llama3_rope_frequencies(head_dim: int, theta: float = 10000.0, scaling: RopeScaling | None = None):
  """Long wavelengths are slowed by ``factor``, short ones untouched, and the band in
  between is blended linearly in 1/wavelength."""
  freqs = default_rope_frequencies(head_dim, theta)
  if scaling is None:
    return freqs
  lo_wl = scaling.original_context_len / scaling.low_freq_factor
  hi_wl = scaling.original_context_len / scaling.high_freq_factor
  assert lo_wl >= hi_wl, f"low_freq_wavelen {lo_wl} must be greater or equal to high_freq_wavelen {hi_wl}"
  wavelen = 2 * math.pi / freqs
  slowed = freqs / scaling.factor
  blend = (scaling.original_context_len / wavelen - scaling.low_freq_factor) / (
    scaling.high_freq_factor - scaling.low_freq_factor)
  mid = (1 - blend) * slowed + blend * freqs
  out = torch.where(wavelen > lo_wl, slowed, freqs)
  in_band = (wavelen >= hi_wl) & (wavelen <= lo_wl)
  return torch.where(in_band, mid, out)


def _yarn_mscale(scale: float, m: float = 1.0) -> float:
  return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0


def yarn_rope_frequencies(config) -> tuple[torch.Tensor, float]:
  """YaRN inverse frequencies and the attention (cos/sin) scale factor for a DeepSeek-style
  config with ``rope_scaling.{factor, beta_fast, beta_slow, mscale, mscale_all_dim,
  original_max_position_embeddings}``."""
  rs = config.rope_scaling
  assert rs is not None and rs.get("rope_type", rs.get("type")) == "yarn", "rope_scaling must be of type yarn"
  base = float(config.rope_theta)
  head_dim = config.get("head_dim", None) or config.hidden_size // config.num_attention_heads
  dim = int(head_dim * config.get("partial_rotary_factor", 1.0))
  factor = rs["factor"]
  if "original_max_position_embeddings" in rs:
    orig = rs["original_max_position_embeddings"]
    factor = config.max_position_embeddings / orig
  else:
    orig = config.max_position_embeddings
  attn_factor = rs.get("attention_factor")
  if attn_factor is None:
    ms, msa = rs.get("mscale"), rs.get("mscale_all_dim")
    attn_factor = float(_yarn_mscale(factor, ms) / _yarn_mscale(factor, msa)) if (ms and msa) else _yarn_mscale(factor)
  beta_fast = rs.get("beta_fast") or 32
  beta_slow = rs.get("beta_slow") or 1

  def corr_dim(rot):
    return (dim * math.log(orig / (rot * 2 * math.pi))) / (2 * math.log(base))

  low = max(math.floor(corr_dim(beta_fast)), 0)
  high = min(math.ceil(corr_dim(beta_slow)), dim - 1)
  if low == high:
    high += 0.001
  pos = base ** (torch.arange(0, dim, 2, device="cpu").float() / dim)
  ramp = torch.clamp((torch.arange(dim // 2, dtype=torch.float32, device="cpu") - low) / (high - low), 0, 1)
  extrap_w = 1 - ramp
  inv_freq = (1.0 / (factor * pos)) * (1 - extrap_w) + (1.0 / pos) * extrap_w
  return inv_freq, attn_factor


def rope_tables(inv_freq: torch.Tensor, max_pos: int, device, attention_factor: float = 1.0):
  """fp32 cos/sin tables ``[max_pos, d/2]``."""
  ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv_freq.to(device)[None, :].float()
  return (ang.cos() * attention_factor).contiguous(), (ang.sin() * attention_factor).contiguous()
