"""Base class of every causal LM: weight init, export / load in the HF-compatible
sharded-safetensors layout, and the description of FSDP units.

Public behaviour mirrors the reference's BaseCausalLM
(torchprime/torch_xla_models/model/base_causal_lm.py:29-185): ``forward(input_ids,
labels=None, attention_mask=None) -> (logits, loss)``, ``export(dir)``,
``from_pretrained(path_or_repo)``, ``_maybe_save_checkpoint(config)``.
"""

from __future__ import annotations

import json
import logging
import os
import time

import torch
import torch.nn as nn

from ..config import Config, to_container

logger = logging.getLogger(__name__)


class BaseCausalLM(nn.Module):
  config: Config

  def _init_weights(self, module: nn.Module):
    std = self.config.initializer_range
    if isinstance(module, nn.Linear):
      module.weight.data.normal_(mean=0.0, std=std)
      if module.bias is not None:
        module.bias.data.zero_()
    elif isinstance(module, nn.Embedding):
      module.weight.data.normal_(mean=0.0, std=std)
      if module.padding_idx is not None:
        module.weight.data[module.padding_idx].zero_()

  def forward(self, input_ids, labels=None, attention_mask=None):
    raise NotImplementedError("Subclasses must implement forward")

  # ---------------------------------------------------------------- FSDP units
  def fsdp_units(self) -> list[tuple[str, nn.Module]]:
    """Modules whose parameters are gathered / released together, in execution order.
    Default: embedding, every decoder layer, then (final norm + lm_head)."""
    units = [("model.embed_tokens", self.model.embed_tokens)]
    for i, layer in enumerate(self.model.layers):
      units.append((f"model.layers.{i}", layer))
    units.append(("head", self.head_unit()))
    return units

  def head_unit(self) -> nn.Module:
    return self._head

  # ---------------------------------------------------------------- export / load
  def export(self, save_directory: str):
    from ..checkpoint import safetensors_io
    os.makedirs(save_directory, exist_ok=True)
    state = {k: v.detach().cpu() for k, v in self.state_dict().items()}
    safetensors_io.save_sharded_safetensors_by_layer(state, save_directory)
    with open(os.path.join(save_directory, "config.json"), "w") as f:
      json.dump(to_container(self.config), f, indent=2)

  def from_pretrained(self, model_path_or_repo: str):
    from ..checkpoint import safetensors_io
    with safetensors_io.model_dir(model_path_or_repo) as model_dir:
      state = safetensors_io.load_safetensors_to_state_dict(model_dir)
    state = self.convert_loaded_state_dict(state)
    self.load_state_dict(state, strict=True)
    return self

  def convert_loaded_state_dict(self, state: dict) -> dict:
    """Hook for models whose in-memory layout differs from the HF checkpoint layout."""
    return state

  def _maybe_save_checkpoint(self, config, engine=None) -> None:
    """Export the trained weights (SFT).  Writes a distributed checkpoint with every rank's
    shards and, when ``task.convert_to_safetensors`` is on, converts it on rank 0 to the
    HF-style sharded safetensors directory, then meets at a barrier."""
    from ..checkpoint import dcp_io, safetensors_io
    from ..dist import runtime as rt
    folder = config.task.get("export_checkpoint_path", None)
    if folder is None:
      logger.info("Skipping model export, task.export_checkpoint_path is not set")
      return
    save_dir = os.path.join(config.output_dir, folder)
    t0 = time.perf_counter()
    if torch.cuda.is_available():
      torch.cuda.synchronize()
    if rt.rank() == 0:
      os.makedirs(save_dir, exist_ok=True)
      safetensors_io.copy_hf_config_files(config.model.get("pretrained_model", None), save_dir)
      safetensors_io.save_hf_tokenizer(config.model.get("tokenizer_name", None), save_dir)
    rt.barrier()
    state = None if engine is not None else {k: v for k, v in self.state_dict().items()}
    dcp_io.save_distributed_checkpoint(state, save_dir, engine=engine)
    rt.barrier()
    if config.task.get("convert_to_safetensors", False) and rt.rank() == 0:
      dcp_io.convert_to_safetensors_on_cpu(save_dir, save_dir)
      if not os.path.exists(os.path.join(save_dir, "config.json")):
        with open(os.path.join(save_dir, "config.json"), "w") as f:
          json.dump(to_container(self.config), f, indent=2)
    rt.barrier()
    logger.info("Model export to %s finished in %.2f s", save_dir, time.perf_counter() - t0)
