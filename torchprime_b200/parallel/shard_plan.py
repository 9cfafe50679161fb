"""Turns the YAML partition specs into an explicit per-rank plan.

The reference hands the same YAML (``configs/model/sharding/*.yaml``) to the XLA GSPMD
partitioner as annotations (torchprime/sharding/shard_model.py:98-174,211-243) and
lets the compiler place every collective.  Here each process owns one GPU, so the specs
are *compiled* into decisions:

* a parameter dim mapped to ``tensor`` -> that dim is sliced over the tensor-parallel
  group (column- vs row-parallel linear follows from which dim it is);
* a dim mapped to ``expert`` -> the leading expert dim is placed over the expert group;
* a dim mapped to ``fsdp`` -> the parameter takes part in ZeRO-3: its (tensor/expert-
  local) values live in the flat shard of its FSDP unit.  The engine shards flat
  buffers, so *which* dim carries ``fsdp`` only matters for the export layout;
* module-output specs are recorded and checked (batch dim over data x fsdp, hidden dim
  over tensor, sequence over context) and select the activation layout of the TP / CP
  code paths instead of being annotations.

Pattern grammar is the reference's: integer path components are written ``*``, a
``[i]`` suffix addresses element i of a tuple output, nested lists name several axes for
one dim, and every key must match a parameter or a module.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Callable

import torch.nn as nn

_AXES = {"data", "fsdp", "tensor", "expert", "context"}


def _to_tuple(obj):
  if isinstance(obj, (list, tuple)):
    return tuple(_to_tuple(o) for o in obj)
  return obj


def process_sharding_name(name: str) -> str:
  """``model.layers.3.mlp`` -> ``model.layers.*.mlp``."""
  return ".".join("*" if part.isdigit() else part for part in name.split("."))


_TAIL_INDEX = re.compile(r"^(.*)\[(\d+)\]$")


def split_tail_index(key: str) -> tuple[str, int | None]:
  m = _TAIL_INDEX.match(key)
  return (m.group(1), int(m.group(2))) if m else (key, None)


def _axes_of(entry) -> tuple:
  if entry is None:
    return ()
  if isinstance(entry, (list, tuple)):
    return tuple(entry)
  return (entry,)


@dataclass
class ParamPlacement:
  name: str
  spec: tuple
  tp_dim: int | None = None
  ep_dim: int | None = None
  fsdp_dim: int | None = None


@dataclass
class ShardPlan:
  params: dict = field(default_factory=dict)     # full param name -> ParamPlacement
  modules: dict = field(default_factory=dict)    # module name -> (spec, tuple index or None)
  raw: dict = field(default_factory=dict)

  @classmethod
  def from_config(cls, model: nn.Module, sharding: dict | None, strict: bool = True) -> "ShardPlan":
    plan = cls(raw=dict(sharding or {}))
    if not sharding:
      return plan
    patterns = {}
    for key, spec in sharding.items():
      base, idx = split_tail_index(key)
      patterns[base] = (key, _to_tuple(spec), idx)
    seen = set()
    param_names = {n for n, _ in model.named_parameters()}
    for name in param_names:
      pat = process_sharding_name(name)
      if pat in patterns:
        key, spec, _ = patterns[pat]
        seen.add(key)
        pl = ParamPlacement(name=name, spec=spec)
        for d, entry in enumerate(spec):
          axes = _axes_of(entry)
          for a in axes:
            assert a in _AXES, f"unknown mesh axis '{a}' in sharding spec for {key}"
          if "tensor" in axes:
            pl.tp_dim = d
          if "expert" in axes:
            pl.ep_dim = d
          if "fsdp" in axes:
            pl.fsdp_dim = d
        plan.params[name] = pl
    for name, _ in model.named_modules():
      pat = process_sharding_name(name)
      if pat in patterns and pat not in {process_sharding_name(p) for p in param_names}:
        key, spec, idx = patterns[pat]
        seen.add(key)
        plan.modules[name] = (spec, idx)
    if strict:
      want = set(sharding.keys())
      missing = want - seen
      assert not missing, (
        f"Requested to shard these names: {sorted(want)}, but only sharded these: {sorted(seen)}.\n\n"
        "These names were not found in the model:\n" + "\n".join(sorted(missing)))
    return plan

  # ------------------------------------------------------------------ queries
  def tp_dim(self, param_name: str) -> int | None:
    p = self.params.get(param_name)
    return p.tp_dim if p else None

  def ep_dim(self, param_name: str) -> int | None:
    p = self.params.get(param_name)
    return p.ep_dim if p else None

  def uses_axis(self, axis: str) -> bool:
    for p in self.params.values():
      for entry in p.spec:
        if axis in _axes_of(entry):
          return True
    for spec, _ in self.modules.values():
      for entry in spec:
        if axis in _axes_of(entry):
          return True
    return False

  def activation_axes(self, module_name: str, dim: int) -> tuple:
    spec, _ = self.modules.get(module_name, ((), None))
    return _axes_of(spec[dim]) if dim < len(spec) else ()


# ---------------------------------------------------------------------------
# Functional API with the reference's shape (used by tests and by other backends):
# callbacks receive (tensor_or_output, spec) and return the transformed object.
# ---------------------------------------------------------------------------
class ShardedModule(nn.Module):
  """Wraps a module so that ``mark_sharding(output, spec)`` runs on what it returns."""

  def __init__(self, mod: nn.Module, mark_sharding: Callable, spec: tuple):
    super().__init__()
    self._orig_mod = mod
    self.mark_sharding = mark_sharding
    self.spec = spec

  def forward(self, *args, **kwargs):
    return self.mark_sharding(self._orig_mod(*args, **kwargs), self.spec)


def wrap_module(mod: nn.Module, transform: Callable[[nn.Module, str], nn.Module], prefix: tuple = ()) -> nn.Module:
  """Bottom-up module rewrite: children first, then the module itself."""
  for name, child in list(mod.named_children()):
    new_child = wrap_module(child, transform, prefix + (name,))
    if new_child is not child:
      setattr(mod, name, new_child)
  return transform(mod, ".".join(prefix))


def shard_model(model: nn.Module, shard_weight: Callable, shard_activation: Callable) -> nn.Module:
  state = {name: shard_weight(p, name) for name, p in model.state_dict().items()}
  model.load_state_dict(state, assign=True)
  return wrap_module(model, shard_activation)


def shard_model_from_config(model: nn.Module, config: dict, shard_output: Callable,
                            shard_param: Callable | None = None) -> nn.Module:
  """Apply ``shard_param(tensor, spec)`` to matching parameters and wrap matching modules
  so ``shard_output(output, spec)`` runs on their results.  All keys must match."""
  shard_param = shard_param or shard_output
  table, out_fns = {}, {}
  for key, spec in config.items():
    base, idx = split_tail_index(key)
    table[base] = _to_tuple(spec)
    if idx is not None:
      def make(index):
        def on_element(outputs, spec):
          outputs = list(outputs) if isinstance(outputs, (list, tuple)) else outputs
          outputs[index] = shard_output(outputs[index], spec)
          return tuple(outputs) if isinstance(outputs, list) else outputs
        return on_element
      out_fns[base] = make(idx)
  seen = set()

  def on_weight(param, name):
    pat = process_sharding_name(name)
    if pat in table:
      seen.add(pat)
      return shard_param(param, table[pat])
    return param

  def on_module(mod, name):
    pat = process_sharding_name(name)
    if pat in table and pat not in seen:
      seen.add(pat)
      return ShardedModule(mod, out_fns.get(pat, shard_output), table[pat])
    if pat in table and isinstance(mod, nn.Module) and not any(
        process_sharding_name(n) == pat for n, _ in model.named_parameters()):
      return ShardedModule(mod, out_fns.get(pat, shard_output), table[pat])
    return mod

  model = shard_model(model, on_weight, on_module)
  want = set(table.keys())
  missing = want - seen
  assert not missing, (
    f"Requested to shard these names: {sorted(want)}, but only sharded these: {sorted(seen)}.\n\n"
    "These names were not found in the model:\n" + "\n".join(sorted(missing)))
  return model
