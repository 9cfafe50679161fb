"""Resolves ``model.remat.*`` into engine options.

Reference: ``add_activation_checkpointing_and_scan`` and ``add_optimization_barriers``
(torchprime/torch_xla_models/model_rewriting/rematerialization_utils.py:28-155) rewrite the
module tree with checkpoint wrappers, ``scan_layers`` and backward optimisation barriers.
In this framework the FSDP engine owns recomputation (a unit is re-run in backward from
its saved inputs), the compile-once layer loop is CUDA-graph replay of a layer segment and
host offload is an async copy of the saved unit input, so the same config keys are only
*validated and translated* here:

  activation_checkpoint_layers  -> classes whose units are recomputed in backward
  scan_layers                   -> path of the homogeneous stack replayed from a graph
  offload_tensors               -> ``decoder_input``: saved unit inputs live in pinned host memory
  optimization_barrier_layers   -> accepted (no compiler to restrain), class names checked

The constraints of the reference are kept: offloading needs scan and exactly one remat
class, and that class must be the class of the scanned layers.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch.nn as nn


@dataclass
class RematPlan:
  remat_classes: tuple = ()
  scan_path: str | None = None
  scan_start: int = 0
  offload_tensors: tuple = ()
  barrier_classes: tuple = ()


def get_classes_by_names(model: nn.Module, names) -> tuple:
  """Classes present in ``model`` whose ``__name__`` is in ``names``; unknown names raise."""
  found = {}
  for mod in model.modules():
    n = type(mod).__name__
    if n in names:
      found[n] = type(mod)
  missing = [n for n in names if n not in found]
  assert not missing, f"Some classes can't be found in the model: {missing}"
  return tuple(found[n] for n in names)


def _resolve(model: nn.Module, path: str):
  mod = model
  for part in path.split("."):
    mod = getattr(mod, part)
  return mod


def add_activation_checkpointing_and_scan(model: nn.Module, config) -> RematPlan:
  remat = config.model.get("remat", {}) or {}
  ckpt_names = list(remat.get("activation_checkpoint_layers", []) or [])
  scan_path = remat.get("scan_layers", None)
  offload = list(remat.get("offload_tensors", []) or [])
  start = int(config.model.get("first_k_dense_replace", 0) or 0) if scan_path else 0
  classes = get_classes_by_names(model, ckpt_names) if ckpt_names else ()
  if offload:
    assert scan_path is not None, "Offloading requires scan_layers to be set"
    assert len(classes) == 1, "Offloading requires exactly one activation checkpoint layer class"
    unknown = [t for t in offload if t != "decoder_input"]
    if unknown:
      raise ValueError(f"unknown tensors in offload_tensors: {unknown} (layers tag: decoder_input)")
  if scan_path is not None:
    stack = _resolve(model, scan_path)
    layers = list(stack)[start:]
    kinds = {type(l) for l in layers}
    assert len(kinds) <= 1, f"scan_layers needs a homogeneous stack, found {sorted(k.__name__ for k in kinds)}"
    if classes and layers:
      assert len(classes) == 1 and classes[0] in kinds, (
        "the activation_checkpoint_layers class must be the class of the scanned layers")
  return RematPlan(remat_classes=tuple(c.__name__ for c in classes), scan_path=scan_path, scan_start=start,
                   offload_tensors=tuple(offload))


def add_optimization_barriers(model: nn.Module, config, plan: RematPlan | None = None):
  remat = config.model.get("remat", {}) or {}
  names = list(remat.get("optimization_barrier_layers", []) or [])
  classes = get_classes_by_names(model, names) if names else ()
  if plan is not None:
    plan.barrier_classes = tuple(c.__name__ for c in classes)
  return model
