"""Resumable training-state checkpoints (a capability the reference does not have: it only
exports weights at the end of SFT, model/base_causal_lm.py:131-185).

Every rank writes its own flat shards — fp32 master weights, optimizer state, the bf16
compute copy is rebuilt from the master — plus step, LR-schedule position, data cursor and
RNG state.  Loading requires the same mesh (shards are positional)."""

from __future__ import annotations

import json
import os

import torch

from ..dist import runtime as rt


def _rank_file(path: str) -> str:
  return os.path.join(path, f"rank_{rt.rank():05d}.pt")


def save(path: str, trainer, step: int) -> None:
  os.makedirs(path, exist_ok=True)
  e = trainer.engine
  payload = {
    "step": step,
    "flat_master": (e.flat_master if e.flat_master is not None else e.flat_param).detach().cpu(),
    "optimizer": {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v)
                  for k, v in trainer.optimizer.state_dict().items()},
    "lr_scheduler": trainer.lr_scheduler.state_dict(),
    "loader": trainer._loader.state_dict() if getattr(trainer, "_loader", None) is not None else {"cursor": step},
    "rng_cpu": torch.get_rng_state(),
    "rng_cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
    "mesh": dict(trainer.mesh.shape), "world_size": rt.world_size(), "total_shard": e.total_shard,
  }
  tmp = _rank_file(path) + ".tmp"
  torch.save(payload, tmp)
  os.replace(tmp, _rank_file(path))
  rt.barrier()
  if rt.is_main():
    with open(os.path.join(path, "meta.json"), "w") as f:
      json.dump({"step": step, "world_size": rt.world_size(), "mesh": dict(trainer.mesh.shape)}, f)


def load(path: str, trainer) -> int:
  f = _rank_file(path)
  if not os.path.exists(f):
    raise FileNotFoundError(f"no training-state shard for rank {rt.rank()} in {path}")
  payload = torch.load(f, map_location="cpu", weights_only=False)
  e = trainer.engine
  if payload["world_size"] != rt.world_size() or payload["total_shard"] != e.total_shard or payload["mesh"] != dict(
      trainer.mesh.shape):
    raise RuntimeError(f"checkpoint {path} was written for mesh {payload['mesh']} / world {payload['world_size']}; "
                       f"current mesh is {dict(trainer.mesh.shape)} / world {rt.world_size()}")
  master = e.flat_master if e.flat_master is not None else e.flat_param
  e.params_will_change()
  master.copy_(payload["flat_master"].to(master.device))
  if e.master_weights:
    e.flat_param.copy_(master)
  e.params_changed()
  opt_sd = {k: (v.to(e.device) if isinstance(v, torch.Tensor) else v) for k, v in payload["optimizer"].items()}
  trainer.optimizer.load_state_dict(opt_sd)
  trainer.lr_scheduler.load_state_dict(payload["lr_scheduler"])
  torch.set_rng_state(payload["rng_cpu"])
  if payload.get("rng_cuda") is not None and torch.cuda.is_available():
    torch.cuda.set_rng_state(payload["rng_cuda"])
  return int(payload["step"])
