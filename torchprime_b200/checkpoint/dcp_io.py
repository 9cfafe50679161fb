"""Distributed checkpoint directory ("format B") and its conversion to safetensors.

The reference saves ``{"model": state_dict}`` with ``torch.distributed.checkpoint`` from
every host and converts on rank 0 (torchprime/torch_xla_models/model/model_utils.py:
284-351).  Here every rank writes its flat parameter shard plus the shard layout as one
``__<rank>_0.distcp`` file, rank 0 writes ``.metadata``; conversion reassembles full
tensors on CPU from those files, deletes them and writes the sharded safetensors.
"""

from __future__ import annotations

import glob
import json
import logging
import os

import torch

from ..dist import runtime as rt
from . import safetensors_io

logger = logging.getLogger(__name__)


def save_distributed_checkpoint(state: dict, save_dir: str, engine=None) -> None:
  os.makedirs(save_dir, exist_ok=True)
  if engine is None:
    # un-sharded model: rank 0 writes everything
    if rt.is_main():
      torch.save({"model": {k: v.detach().cpu() for k, v in state.items()}, "kind": "full"},
                 os.path.join(save_dir, "__0_0.distcp"))
      with open(os.path.join(save_dir, ".metadata"), "w") as f:
        json.dump({"kind": "full", "world_size": 1}, f)
    return
  payload = {"kind": "flat", "flat_param": state["flat_param"].detach().cpu(), "layout": state["layout"],
             "fsdp": state["fsdp"], "fsdp_rank": state["fsdp_rank"], "tp": state["tp"], "tp_rank": state["tp_rank"]}
  # replicas along data/context hold identical shards: only the first replica writes
  if engine.mesh.index(("data", "context")) == 0:
    torch.save(payload, os.path.join(save_dir, f"__{rt.rank()}_0.distcp"))
  if rt.is_main():
    with open(os.path.join(save_dir, ".metadata"), "w") as f:
      json.dump({"kind": "flat", "world_size": rt.world_size(), "fsdp": state["fsdp"], "tp": state["tp"]}, f)


def load_full_state_from_distcp(ckpt_dir: str) -> dict:
  files = sorted(glob.glob(os.path.join(ckpt_dir, "__*_0.distcp")))
  if not files:
    raise FileNotFoundError(f"no *.distcp files in {ckpt_dir}")
  parts = [torch.load(f, map_location="cpu", weights_only=False) for f in files]
  if parts[0]["kind"] == "full":
    return parts[0]["model"]
  fsdp, tp = parts[0]["fsdp"], parts[0]["tp"]
  by_coord = {(p["tp_rank"], p["fsdp_rank"]): p for p in parts}
  out = {}
  layout = parts[0]["layout"]
  for t in range(tp):
    for u in layout:
      pieces = [by_coord[(t, r)]["flat_param"][u["shard_offset"]:u["shard_offset"] + u["shard_size"]]
                for r in range(fsdp)]
      full = torch.cat(pieces)
      for s in u["slots"]:
        n = 1
        for d in s["shape"]:
          n *= d
        val = full[s["offset"]:s["offset"] + n].view(s["shape"]).clone()
        if s["tp_dim"] is None:
          out[s["name"]] = val
        else:
          out.setdefault(s["name"], [None] * tp)[t] = val
  for u in layout:
    for s in u["slots"]:
      if s["tp_dim"] is not None:
        out[s["name"]] = torch.cat(out[s["name"]], dim=s["tp_dim"])
  return out


def convert_to_safetensors_on_cpu(ckpt_dir: str, save_dir: str) -> None:
  state = load_full_state_from_distcp(ckpt_dir)
  for f in glob.glob(os.path.join(ckpt_dir, "*.distcp")):
    os.remove(f)
  meta = os.path.join(ckpt_dir, ".metadata")
  if os.path.exists(meta):
    os.remove(meta)
  safetensors_io.save_sharded_safetensors_by_layer(state, save_dir)
  logger.info("Converted distributed checkpoint in %s to safetensors in %s", ckpt_dir, save_dir)
