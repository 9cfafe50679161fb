"""Distributed checkpoint directory ("format B") and its conversion to safetensors.

The reference saves ``{"model": state_dict}`` with ``torch.distributed.checkpoint`` from
every host and converts on rank 0 (torchprime/torch_xla_models/model/model_utils.py:
284-351).  This module writes the same kind of directory (``.metadata`` plus
``__<rank>_<n>.distcp`` files that ``torch.distributed.checkpoint.load`` reads, top-level
key ``"model"``, one entry per parameter under its state-dict name).

The engine's shards are slices of flat per-unit buffers, which cut parameters at arbitrary
element offsets, so they are not expressible as sharded tensors of the checkpoint format.
Instead every parameter is written whole by exactly one rank: the ranks walk the model unit
by unit, all take part in the gathers (over the fsdp, tensor and expert groups), and rank
``i`` keeps the parameters whose position in the model is ``i`` modulo the world size.  Host
memory per rank is therefore 1/world of the model, and the files are written in parallel.
"""

from __future__ import annotations

import glob
import logging
import os

import torch
import torch.distributed.checkpoint as dcp

from ..dist import runtime as rt
from . import safetensors_io

logger = logging.getLogger(__name__)


def _owned_state(engine) -> dict:
  """This rank's share of the un-sharded parameters (whole tensors on CPU)."""
  names = [s.name for u in engine.units for s in u.slots]
  world, rank = rt.world_size(), rt.rank()
  owner = {n: i % world for i, n in enumerate(names)}
  return engine.full_state_dict(to_cpu=True, keep=lambda name: owner[name] == rank)


def save_distributed_checkpoint(state: dict | None, save_dir: str, engine=None) -> None:
  """Collective.  ``state`` is a plain ``{name: tensor}`` dict for an un-sharded model (then only
  rank 0 holds data); with ``engine`` the parameters come from its shards."""
  os.makedirs(save_dir, exist_ok=True)
  if engine is not None:
    model_state = _owned_state(engine)
  else:
    model_state = {k: v.detach().cpu() for k, v in state.items()} if rt.is_main() else {}
  import torch.distributed as dist
  dcp.save({"model": model_state}, storage_writer=dcp.FileSystemWriter(save_dir, thread_count=4),
           no_dist=not dist.is_initialized())


def load_full_state_from_distcp(ckpt_dir: str) -> dict:
  """Read every tensor under ``"model"`` into CPU memory (single process, no process group)."""
  if not os.path.exists(os.path.join(ckpt_dir, ".metadata")):
    raise FileNotFoundError(f"no distributed checkpoint (.metadata) in {ckpt_dir}")
  reader = dcp.FileSystemReader(ckpt_dir)
  meta = reader.read_metadata()
  state = {}
  for key, tm in meta.state_dict_metadata.items():
    if not key.startswith("model.") or not hasattr(tm, "size"):
      continue
    state[key] = torch.empty(tuple(tm.size), dtype=tm.properties.dtype)
  dcp.load(state, storage_reader=reader, no_dist=True)
  return {k[len("model."):]: v for k, v in state.items()}


def convert_to_safetensors_on_cpu(ckpt_dir: str, save_dir: str) -> None:
  state = load_full_state_from_distcp(ckpt_dir)
  for f in glob.glob(os.path.join(ckpt_dir, "*.distcp")):
    os.remove(f)
  meta = os.path.join(ckpt_dir, ".metadata")
  if os.path.exists(meta):
    os.remove(meta)
  safetensors_io.save_sharded_safetensors_by_layer(state, save_dir)
  logger.info("Converted distributed checkpoint in %s to safetensors in %s", ckpt_dir, save_dir)
