"""Five-axis logical device mesh over the GPUs of one NVSwitch box.

Axis names and the row-major rank <-> coordinate rule follow the reference
(``("data","fsdp","tensor","expert","context")``, ``xs.Mesh(range(n), shape, names)``,
torchprime/torch_xla_models/topology.py:93-120).  Differences that come from the
hardware: every GPU pair has the same NVLink bandwidth through the switch, so there is no
physical device ordering to optimise (the reference's 64x4 TPU ring mesh,
torchprime/mesh/custom_mesh.py:34-123, has no counterpart and
:func:`maybe_get_custom_mesh` returns None); cross-box ``dcn_mesh`` axes must be 1.

``expert_axis_mode="folded"`` lays the expert-parallel group over the same ranks as
data x fsdp (so ``fsdp=8 expert=8`` is valid on 8 GPUs): dense weights are sharded over
fsdp while expert weights are placed by expert index over the very same ranks.
"""

from __future__ import annotations

import itertools
import math
from dataclasses import dataclass, field

import torch.distributed as dist

AXES = ("data", "fsdp", "tensor", "expert", "context")


def is_1d_sharding(mesh_shape) -> bool:
  """True when at most one axis is larger than 1 (reference: topology.py is_1d_sharding)."""
  return sum(1 for v in mesh_shape if v > 1) <= 1


def maybe_get_custom_mesh(*_args, **_kwargs):
  """NVSwitch gives a uniform topology; there is never a custom physical ordering."""
  return None


def get_num_slices() -> int:
  """Number of cross-box slices.  Always 1: this framework runs on one NVSwitch domain."""
  return 1


@dataclass
class Mesh:
  shape: dict                      # axis -> size, in AXES order
  rank: int = 0
  world_size: int = 1
  expert_mode: str = "orthogonal"  # or "folded"
  _groups: dict = field(default_factory=dict, repr=False)

  # ----------------------------------------------------------------- geometry
  @property
  def grid_axes(self) -> tuple:
    """Axes that span distinct ranks (the folded expert axis does not)."""
    return tuple(a for a in AXES if not (a == "expert" and self.expert_mode == "folded"))

  def grid_shape(self) -> tuple:
    return tuple(self.shape[a] for a in self.grid_axes)

  def coords_of(self, rank: int) -> dict:
    out, rem = {}, rank
    for a, n in reversed(list(zip(self.grid_axes, self.grid_shape()))):
      out[a] = rem % n
      rem //= n
    if self.expert_mode == "folded":
      out["expert"] = self.expert_rank_of(rank)
    return out

  def rank_of(self, coords: dict) -> int:
    r = 0
    for a, n in zip(self.grid_axes, self.grid_shape()):
      r = r * n + coords[a]
    return r

  @property
  def coords(self) -> dict:
    return self.coords_of(self.rank)

  def size(self, axis) -> int:
    if isinstance(axis, (list, tuple)):
      return math.prod(self.size(a) for a in axis)
    return self.shape[axis]

  def index(self, axis) -> int:
    """Position of this rank along ``axis`` (or along a row-major tuple of axes)."""
    if isinstance(axis, (list, tuple)):
      i = 0
      for a in axis:
        i = i * self.shape[a] + self.coords[a]
      return i
    return self.coords[axis]

  # ------------------------------------------------------------ expert folding
  def _fold_base_axes(self) -> tuple:
    return ("data", "fsdp")

  def expert_rank_of(self, rank: int) -> int:
    c = {}
    rem = rank
    for a, n in reversed(list(zip(self.grid_axes, self.grid_shape()))):
      c[a] = rem % n
      rem //= n
    flat = c["data"] * self.shape["fsdp"] + c["fsdp"]
    return flat % self.shape["expert"]

  # ------------------------------------------------------------------- groups
  def ranks_in_group(self, axes, rank: int | None = None) -> list[int]:
    """Ranks that share every coordinate with ``rank`` except along ``axes``."""
    rank = self.rank if rank is None else rank
    axes = (axes,) if isinstance(axes, str) else tuple(axes)
    if self.expert_mode == "folded" and "expert" in axes:
      assert axes == ("expert",), "a folded expert axis cannot be combined with other axes"
      base = self.ranks_in_group(self._fold_base_axes(), rank)
      e = self.shape["expert"]
      pos = base.index(rank)
      start = (pos // e) * e
      return base[start:start + e]
    me = self.coords_of(rank)
    free = [a for a in self.grid_axes if a in axes]
    ranges = [range(self.shape[a]) for a in free]
    out = []
    for combo in itertools.product(*ranges):
      c = dict(me)
      c.update(dict(zip(free, combo)))
      out.append(self.rank_of(c))
    return out

  def group(self, axes):
    """Process group over ``axes`` (None when it would contain only this rank or when
    torch.distributed is not initialised).  Creation is collective: every rank creates
    every group of the family in the same order."""
    axes = (axes,) if isinstance(axes, str) else tuple(axes)
    if axes in self._groups:
      return self._groups[axes]
    mine = None
    if dist.is_initialized() and self.size(axes) > 1:
      seen = set()
      for r in range(self.world_size):
        members = tuple(self.ranks_in_group(axes, r))
        if members in seen:
          continue
        seen.add(members)
        if len(members) == self.world_size:
          g = dist.group.WORLD
        else:
          g = dist.new_group(ranks=list(members))
        if self.rank in members:
          mine = g
    self._groups[axes] = mine
    return mine

  def describe(self) -> str:
    return "Mesh(" + ", ".join(f"{a}={self.shape[a]}" for a in AXES) + f", expert_mode={self.expert_mode})"


def get_mesh(config, rank: int | None = None, world_size: int | None = None) -> Mesh:
  """Build the mesh from ``config.ici_mesh`` / ``config.dcn_mesh``.

  Like the reference (topology.py:53-121) the product of the axis sizes must equal the
  number of devices; cross-box axes must all be 1 on a single NVSwitch box."""
  from . import runtime as rt
  rank = rt.rank() if rank is None else rank
  world_size = rt.world_size() if world_size is None else world_size
  ici = {a: int(config.ici_mesh.get(a, 1)) for a in AXES}
  dcn = {a: int(config.get("dcn_mesh", {}).get(a, 1)) for a in AXES}
  assert all(v == 1 for v in dcn.values()), (
    f"dcn_mesh axes must all be 1 on a single NVSwitch box, got {dcn}")
  mode = config.get("expert_axis_mode", "orthogonal")
  assert mode in ("orthogonal", "folded"), f"unknown expert_axis_mode {mode}"
  grid = math.prod(v for a, v in ici.items() if not (a == "expert" and mode == "folded"))
  assert grid == world_size, (
    f"Mesh is not using all the available devices. The mesh shape is {tuple(ici.values())} "
    f"(expert_axis_mode={mode}) = {grid} ranks while there are {world_size} devices")
  if mode == "folded":
    base = ici["data"] * ici["fsdp"]
    assert base % ici["expert"] == 0, f"folded expert axis {ici['expert']} must divide data*fsdp = {base}"
  return Mesh(shape=ici, rank=rank, world_size=world_size, expert_mode=mode)
