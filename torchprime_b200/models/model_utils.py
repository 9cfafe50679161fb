"""Model construction helpers: class lookup by config string, default dtype scope, model
size parsing and the per-component parameter report.

Counterparts in the reference: ``initialize_model_class``, ``set_default_dtype``,
``extract_model_size_from_model_name``, ``log_parameter_breakdown``
(torchprime/torch_xla_models/model/model_utils.py:138-245).
"""

from __future__ import annotations

import importlib
import logging
import re
from contextlib import contextmanager

import torch

_ALIASES = {
  "llama": "llama", "mixtral": "mixtral", "deepseek_v3": "deepseek_v3", "llama4": "llama4",
  "model.llama": "llama", "model.mixtral": "mixtral", "model.deepseek_v3": "deepseek_v3", "model.llama4": "llama4",
}


def resolve_model_class(model_class: str):
  """``"llama.LlamaForCausalLM"`` -> class (module looked up in this package)."""
  module_name, cls_name = model_class.rsplit(".", 1)
  short = _ALIASES.get(module_name, module_name.split(".")[-1])
  try:
    module = importlib.import_module(f"torchprime_b200.models.{short}")
  except ModuleNotFoundError as e:
    raise ImportError(f"Failed to import model module '{module_name}' (looked for torchprime_b200.models.{short})") from e
  if not hasattr(module, cls_name):
    raise ImportError(f"Class '{cls_name}' not found in module '{module.__name__}'")
  return getattr(module, cls_name)


def initialize_model_class(model_config, device: str | torch.device | None = None, dtype=None):
  """Instantiate ``model_config.model_class``.  ``device="meta"`` builds the skeleton only;
  the FSDP engine then materialises and initialises each rank's shard on its GPU."""
  cls = resolve_model_class(model_config.model_class)
  if device is None and dtype is None:
    return cls(model_config)
  with set_default_dtype(dtype or torch.get_default_dtype()):
    if device is None:
      return cls(model_config)
    with torch.device(device):
      return cls(model_config)


@contextmanager
def set_default_dtype(dtype: torch.dtype):
  old = torch.get_default_dtype()
  torch.set_default_dtype(dtype)
  try:
    yield
  finally:
    torch.set_default_dtype(old)


def extract_model_size_from_model_name(name: str) -> float | int:
  """Billions of parameters parsed from names like ``llama-3.1-70b`` or ``mixtral-8x7b``; -1 if absent."""
  m = re.search(r"(?:(\d+)x)?(\d+(?:\.\d+)?)b\b", name.lower())
  if not m:
    return -1
  try:
    size = float(m.group(2)) * (int(m.group(1)) if m.group(1) else 1)
  except ValueError:
    return -1
  return int(size) if size == int(size) else size


def log_parameter_breakdown(model: torch.nn.Module, logger: logging.Logger) -> None:
  total = sum(p.numel() for p in model.parameters())
  logger.info("Model total size: %s parameters", f"{total:,}")
  groups = {"mlp": 0, "attention": 0, "embedding": 0, "lm_head": 0, "norm": 0, "other": 0}
  for name, p in model.named_parameters():
    if "mlp" in name:
      key = "mlp"
    elif "self_attn" in name or "attention" in name:
      key = "attention"
    elif "embed" in name:
      key = "embedding"
    elif "lm_head" in name:
      key = "lm_head"
    elif "norm" in name:
      key = "norm"
    else:
      key = "other"
    groups[key] += p.numel()
  for key, n in groups.items():
    logger.info("  %-10s: %s params (%.2f%%)", key, f"{n:,}", 100.0 * n / max(total, 1))
