"""Process-level distributed runtime: one process per GPU, ``torch.distributed`` for the
plumbing (NCCL on GPUs, gloo on CPU ranks).

Replaces the reference's single-process-per-host SPMD runtime
(``xr.use_spmd()``, torchprime/torch_xla_models/train.py:25-26) and its rank /
topology discovery calls (trainer/base_trainer.py:175-183).  Rendezvous always
uses the MASTER_ADDR given by the launcher (127.0.0.1 on one box).
"""

from __future__ import annotations

import datetime
import logging
import os

import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)
_STATE = {"initialized_here": False, "device": None}


def env_rank() -> int:
  return int(os.environ.get("RANK", "0"))


def env_world_size() -> int:
  return int(os.environ.get("WORLD_SIZE", "1"))


def env_local_rank() -> int:
  return int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))


def init(backend: str | None = None, timeout_s: float = 600.0, device: str | None = None) -> torch.device:
  """Initialise the default process group (if WORLD_SIZE > 1) and pick this rank's device."""
  use_cuda = torch.cuda.is_available() and device != "cpu"
  if use_cuda:
    dev = torch.device("cuda", env_local_rank() % torch.cuda.device_count())
    torch.cuda.set_device(dev)
  else:
    dev = torch.device("cpu")
  _STATE["device"] = dev
  if env_world_size() > 1 and not dist.is_initialized():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    backend = backend or ("nccl" if use_cuda else "gloo")
    kwargs = {}
    if backend == "nccl":
      kwargs["device_id"] = dev
    dist.init_process_group(backend=backend, rank=env_rank(), world_size=env_world_size(),
                            timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    _STATE["initialized_here"] = True
  return dev


def shutdown():
  if dist.is_initialized() and _STATE["initialized_here"]:
    dist.destroy_process_group()
    _STATE["initialized_here"] = False


def device() -> torch.device:
  if _STATE["device"] is None:
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
  return _STATE["device"]


def rank() -> int:
  return dist.get_rank() if dist.is_initialized() else 0


def world_size() -> int:
  return dist.get_world_size() if dist.is_initialized() else 1


def is_main() -> bool:
  return rank() == 0


def barrier(group=None):
  if dist.is_initialized():
    if dist.get_backend(group) == "nccl":
      dist.barrier(group=group, device_ids=[torch.cuda.current_device()])
    else:
      dist.barrier(group=group)


def all_reduce_max_float(value: float, group=None) -> float:
  """Max of a host float over ranks (used for "max over ranks" timings)."""
  if not dist.is_initialized():
    return value
  t = torch.tensor([value], dtype=torch.float64, device=device() if dist.get_backend(group) == "nccl" else "cpu")
  dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
  return float(t.item())
