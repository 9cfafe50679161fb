"""Mesh + shard-plan set-up for a model.

Reference: ``setup_sharding_and_mesh(model, config) -> (model, input_sharding_spec,
minibatch)`` (torchprime/torch_xla_models/model_rewriting/sharding_initialization.py:22-69)
creates the global SPMD mesh, decides whether each host loads only its part of the batch
("minibatch") and annotates the model.  Here it returns the explicit pieces the engine and
the data loader need: the :class:`Mesh`, the compiled :class:`ShardPlan`, the tuple of mesh
axes the batch dimension is split over (``("data","fsdp")`` plus ``"expert"`` when that
axis is orthogonal, as in the reference's MoE configs) and the sequence axis
(``"context"`` when context parallelism is on).
"""

from __future__ import annotations

from dataclasses import dataclass

from ..config import to_container
from ..dist.mesh import Mesh, get_mesh, is_1d_sharding
from ..parallel.shard_plan import ShardPlan


@dataclass
class ShardingSetup:
  mesh: Mesh
  plan: ShardPlan
  batch_axes: tuple
  seq_axis: str | None
  minibatch: bool

  @property
  def input_sharding_spec(self):
    return (self.batch_axes, self.seq_axis)


def setup_sharding_and_mesh(model, config, mesh: Mesh | None = None) -> ShardingSetup:
  mesh = mesh or get_mesh(config)
  sharding = config.model.get("sharding", None)
  plan = ShardPlan.from_config(model, to_container(sharding) if sharding else None)
  batch_axes = ("data", "fsdp")
  if mesh.expert_mode == "orthogonal" and mesh.size("expert") > 1:
    batch_axes = ("data", "fsdp", "expert")
  seq_axis = "context" if mesh.size("context") > 1 else None
  minibatch = is_1d_sharding(tuple(mesh.shape.values()))
  return ShardingSetup(mesh=mesh, plan=plan, batch_axes=batch_axes, seq_axis=seq_axis, minibatch=minibatch)
