"""Mesh geometry, shard plan, zig-zag permutations, safetensors layout."""

import json
import os

import numpy as np
import pytest
import torch
import torch.nn as nn

from torchprime_b200.checkpoint import safetensors_io as sio
from torchprime_b200.config import compose, to_container
from torchprime_b200.dist.mesh import Mesh, get_mesh, is_1d_sharding, maybe_get_custom_mesh
from torchprime_b200.models.model_utils import extract_model_size_from_model_name, initialize_model_class
from torchprime_b200.parallel.shard_plan import ShardPlan, ShardedModule, shard_model_from_config
from torchprime_b200.utils.parallelism_utils import (LoadBalancedCausalMask, chunk_permutation, reorder_mask,
                                                     reorder_sequence)


def test_reorder_golden_and_roundtrip():
  x = torch.arange(8)[None]
  y = reorder_sequence(x, cp_size=2, seq_dim=1)
  assert y.tolist() == [[0, 1, 6, 7, 2, 3, 4, 5]]
  assert reorder_sequence(y, cp_size=2, seq_dim=1, to_contiguous=True).tolist() == x.tolist()
  for cp in (2, 4, 8):
    t = torch.randn(2, 16 * cp, 3)
    back = reorder_sequence(reorder_sequence(t, cp, 1), cp, 1, to_contiguous=True)
    assert torch.equal(back, t)
  assert chunk_permutation(2, True) == [0, 2, 3, 1]
  with pytest.raises(ValueError, match="multiple of 2"):
    reorder_sequence(x, cp_size=3, seq_dim=1)
  with pytest.raises(ValueError, match="not a multiple"):
    reorder_sequence(torch.arange(6)[None], cp_size=2, seq_dim=1)
  assert reorder_mask(np.arange(8), 2, 0).tolist() == [0, 1, 6, 7, 2, 3, 4, 5]
  m = LoadBalancedCausalMask((8, 8), cp_size=2)
  assert m.q_sequence.tolist() == [0, 1, 6, 7, 2, 3, 4, 5]
  assert m.as_array()[2].tolist() == [True] * 7 + [False]
  assert m == LoadBalancedCausalMask((8, 8), cp_size=2) and hash(m) == hash(LoadBalancedCausalMask((8, 8), cp_size=2))


def test_mesh_geometry_and_groups():
  shape = {"data": 1, "fsdp": 4, "tensor": 2, "expert": 1, "context": 1}
  m = Mesh(shape, rank=5, world_size=8)
  assert m.coords["fsdp"] == 2 and m.coords["tensor"] == 1
  assert m.ranks_in_group("fsdp") == [1, 3, 5, 7] and m.ranks_in_group("tensor") == [4, 5]
  assert m.index(("data", "fsdp")) == 2 and m.size(("fsdp", "tensor")) == 8
  for r in range(8):
    assert m.rank_of(m.coords_of(r)) == r
  f = Mesh({"data": 1, "fsdp": 8, "tensor": 1, "expert": 4, "context": 1}, rank=5, world_size=8, expert_mode="folded")
  assert f.ranks_in_group("expert") == [4, 5, 6, 7] and f.coords["expert"] == 1
  assert is_1d_sharding((1, 4, 1, 1, 1)) and not is_1d_sharding((1, 2, 2, 1, 1))
  assert maybe_get_custom_mesh() is None


def test_get_mesh_checks():
  c = compose("default", ["ici_mesh.fsdp=4"])
  with pytest.raises(AssertionError, match="not using all the available devices"):
    get_mesh(c, rank=0, world_size=8)
  assert get_mesh(c, rank=0, world_size=4).size("fsdp") == 4
  c = compose("default", ["ici_mesh.fsdp=8", "ici_mesh.expert=8", "expert_axis_mode=folded"])
  assert get_mesh(c, rank=3, world_size=8).ranks_in_group("expert") == list(range(8))


class _Toy(nn.Module):
  def __init__(self):
    super().__init__()
    self.embed = nn.Embedding(8, 4)
    self.layers = nn.ModuleList([nn.Linear(4, 4) for _ in range(3)])

  def forward(self, x):
    h = self.embed(x)
    for l in self.layers:
      h = l(h)
    return h


def test_shard_plan_and_functional_api():
  toy = _Toy()
  cfg = {"embed.weight": ["fsdp", None], "layers.*.weight": ["tensor", "fsdp"], "layers.*": [["data", "fsdp"], None]}
  plan = ShardPlan.from_config(toy, cfg)
  assert plan.tp_dim("layers.1.weight") == 0 and plan.tp_dim("embed.weight") is None
  assert plan.modules["layers.2"][0] == (("data", "fsdp"), None)
  assert plan.uses_axis("tensor") and not plan.uses_axis("context")
  with pytest.raises(AssertionError, match="not found in the model"):
    ShardPlan.from_config(toy, {"nope.weight": ["fsdp"]})
  calls = []
  out = shard_model_from_config(_Toy(), cfg, lambda t, spec: (calls.append(("out", spec)), t)[1],
                                lambda t, spec: (calls.append(("param", spec)), t)[1])
  assert sum(1 for c in calls if c[0] == "param") == 4
  assert isinstance(out.layers[0], ShardedModule)
  out(torch.tensor([[1, 2]]))
  assert sum(1 for c in calls if c[0] == "out") == 3
  # [i] suffix shards one element of a tuple output
  class Tup(nn.Module):
    def __init__(self):
      super().__init__()
      self.inner = nn.Linear(2, 2)
    def forward(self, x):
      return self.inner(x), x
  class Wrap(nn.Module):
    def __init__(self):
      super().__init__()
      self.t = Tup()
    def forward(self, x):
      return self.t(x)
  seen = []
  w = shard_model_from_config(Wrap(), {"t[0]": ["fsdp", None]}, lambda t, spec: (seen.append(t.shape), t * 2)[1])
  a, b = w(torch.ones(1, 2))
  assert len(seen) == 1 and torch.equal(b, torch.ones(1, 2))


def test_real_sharding_configs_match_models():
  for model in ("llama-tiny", "mixtral-tiny", "deepseek-tiny"):
    cfg = compose("default", ["model=" + model])
    m = initialize_model_class(cfg.model, device="meta")
    ShardPlan.from_config(m, to_container(cfg.model.sharding))


def test_group_keys_and_roundtrip(tmp_path):
  assert sio.get_param_group_key("model.layers.12.mlp.up_proj.weight") == "layers_12"
  assert sio.get_param_group_key("model.embed_tokens.weight") == "model"
  assert sio.get_param_group_key("model.norm.weight") == "model"
  assert sio.get_param_group_key("lm_head.weight") == "lm_head"
  assert sio.get_param_group_key("module.layer1.0.conv.weight") == "layer1_0"
  state = {"model.embed_tokens.weight": torch.randn(4, 2), "model.layers.0.a._orig_mod.weight": torch.randn(2, 2),
           "model.layers.1.a.weight": torch.randn(2, 2).to(torch.bfloat16), "lm_head.weight": torch.randn(4, 2)}
  sio.save_sharded_safetensors_by_layer(state, str(tmp_path))
  files = sorted(os.listdir(tmp_path))
  assert files == ["layers_0.safetensors", "layers_1.safetensors", "lm_head.safetensors", "model.safetensors",
                   "model.safetensors.index.json"]
  index = json.load(open(tmp_path / "model.safetensors.index.json"))
  assert set(index) == {"weight_map"} and index["weight_map"]["model.layers.0.a.weight"] == "layers_0.safetensors"
  back = sio.load_safetensors_to_state_dict(str(tmp_path))
  assert torch.equal(back["model.layers.0.a.weight"], state["model.layers.0.a._orig_mod.weight"])
  assert back["model.layers.1.a.weight"].dtype == torch.bfloat16
  with pytest.raises(FileNotFoundError):
    sio.load_safetensors_to_state_dict(str(tmp_path / "missing"))


def test_model_size_parsing():
  assert extract_model_size_from_model_name("llama-3.1-70b") == 70
  assert extract_model_size_from_model_name("mixtral-8x7b") == 56
  assert extract_model_size_from_model_name("llama-tiny") == -1


def test_homogeneous_sequential_passes_keyword_arguments_to_every_layer():
  import pytest
  import torch
  import torch.nn as nn
  from torchprime_b200.layers import HomogeneousSequential

  class Scale(nn.Module):
    def __init__(self, k):
      super().__init__()
      self.k = k

    def forward(self, x, bias=None):
      return x * self.k + bias

  stack = HomogeneousSequential(Scale(2.0), Scale(3.0))
  out = stack(torch.ones(2), bias=torch.full((2,), 1.0))
  assert torch.equal(out, torch.full((2,), 10.0))          # (1*2+1)*3+1
  with pytest.raises(AssertionError):
    HomogeneousSequential(Scale(1.0), nn.ReLU())


@pytest.mark.parametrize("scale,align", [(1, 128), (20, 256)])
def test_expert_exchange_plan_groups_rows_by_expert_and_returns_them(scale, align):
  """The host-side plan of the expert-parallel exchange, checked by replaying the block-push kernel's
  rule in Python: rows land at the owner grouped by expert in padded segments, padding rows are the
  ones listed for zeroing, and the return blocks bring every row back to its place."""
  import random

  import torch
  from torchprime_b200.parallel.ep import _ExchangePlan
  random.seed(0)
  ep, el = 4, 3
  E = ep * el
  C = [[scale * random.choice([0, 0, 1, 5, 130, 257]) for _ in range(E)] for _ in range(ep)]
  C[2] = [0] * E                                           # a rank that sends nothing
  plans = [_ExchangePlan(C, me, ep, el, "cpu") for me in range(ep)]
  assert all(p.row_align == align for p in plans)
  # the range-checked debug mode accepts what the plan produces (receive buffers sized as the engine sizes them)
  import os
  from torchprime_b200.ops import _debug
  pairs = max(sum(row) for row in C)
  os.environ["TPB_DEBUG_BOUNDS"] = "1"
  try:
    for p in plans:
      _debug.check_exchange_descriptors("dispatch", p.dispatch, p.dispatch_blocks, p.n_send, ep, ep * pairs + el * 256)
      _debug.check_exchange_descriptors("return", p.ret, p.ret_blocks, p.n_pad, ep, pairs)
  finally:
    os.environ.pop("TPB_DEBUG_BOUNDS")

  def push(src_rows, desc, nb, dst):
    start, rank, row0 = desc[:nb + 1].tolist(), desc[nb + 1:2 * nb + 1].tolist(), desc[2 * nb + 1:].tolist()
    for row, item in enumerate(src_rows):
      b = max(i for i in range(nb) if start[i] <= row)
      if rank[b] >= 0:
        dst[rank[b]][row0[b] + row - start[b]] = item

  send = [[(s, e, i) for e in range(E) for i in range(C[s][e])] for s in range(ep)]
  recv = [dict() for _ in range(ep)]
  for s in range(ep):
    assert plans[s].n_send == len(send[s])
    push(send[s], plans[s].dispatch, plans[s].dispatch_blocks, recv)
  for r in range(ep):
    p = plans[r]
    koff = p.k_offsets.tolist()
    assert p.n_pad == koff[-1] and all(v % p.row_align == 0 for v in koff) and p.row_align in (128, 256)
    assert p.tile_expert.tolist() == [j for j in range(el) for _ in range((koff[j + 1] - koff[j]) // 128)]
    filled = set(recv[r])
    zero = set(p.zero_rows.tolist()) if p.zero_rows is not None else set()
    assert filled | zero == set(range(p.n_pad)) and not (filled & zero)
    for j in range(el):
      seg = [recv[r][i] for i in range(koff[j], koff[j + 1]) if i in recv[r]]
      assert all(e == r * el + j for _, e, _ in seg)
      assert seg == sorted(seg)                          # sources in order, rows of a source in order
      assert len(seg) == sum(C[s][r * el + j] for s in range(ep))
  back = [dict() for _ in range(ep)]
  for r in range(ep):
    rows = [recv[r].get(i) for i in range(plans[r].n_pad)]
    push(rows, plans[r].ret, plans[r].ret_blocks, back)
  for s in range(ep):
    assert [back[s][i] for i in range(len(send[s]))] == send[s]


def test_fused_tensor_parallel_request_needs_the_kernel_path():
  """``linear(..., tp_reduce=...)`` promises that the output is already summed over the tensor group;
  on a path without kernels (CPU, fp32) that promise cannot be kept, so it raises instead of silently
  returning a partial sum."""
  import torch
  from torchprime_b200.ops import functional as ops

  class Reducer:
    def usable(self, m, n, k):
      return True

  x, w = torch.randn(4, 8), torch.randn(16, 8)
  with pytest.raises(RuntimeError):
    ops.linear(x, w, tp_reduce=Reducer())
  with pytest.raises(RuntimeError):
    ops.linear_swiglu(x, w, w.clone(), tp_reduce_grad=Reducer())
  assert ops.linear(x, w).shape == (4, 16)


def test_tp_slice_of_fused_blocks_round_trips():
  """A fused [gate | up] dimension is sliced half by half: every rank holds [gate_r | up_r]."""
  import torch
  from torchprime_b200.parallel.fsdp import tp_slice, tp_unslice
  w = torch.arange(2 * 3 * 8).view(2, 3, 8)              # last dim = [gate(4) | up(4)]
  parts = [tp_slice(w, 2, 2, r, blocks=2) for r in range(2)]
  assert parts[0][0, 0].tolist() == [0, 1, 4, 5] and parts[1][0, 0].tolist() == [2, 3, 6, 7]
  assert torch.equal(tp_unslice(parts, 2, blocks=2), w)
  plain = [tp_slice(w, 1, 3, r) for r in range(3)]
  assert plain[1].shape == (2, 1, 8) and torch.equal(tp_unslice(plain, 1), w)


def test_leftover_ranges_of_the_peer_reduce_scatter():
  """What the weight-gradient GEMMs did not push is copied to the owners, cut at shard boundaries."""
  from types import SimpleNamespace
  from torchprime_b200.parallel.fsdp_comm import PeerFsdpComm
  u = SimpleNamespace(total=400, shard_size=100, _pushed=[(120, 80), (0, 50), (250, 100)])
  got = PeerFsdpComm._leftover(None, u)
  assert got == [(0, 50, 50), (1, 100, 20), (2, 200, 50), (3, 350, 50)]
  covered = sorted([(a, a + n) for _, a, n in got] + [(a, a + n) for a, n in u._pushed])
  assert covered[0][0] == 0 and covered[-1][1] == 400 and all(x[1] == y[0] for x, y in zip(covered, covered[1:]))
  u2 = SimpleNamespace(total=200, shard_size=100, _pushed=[])
  assert PeerFsdpComm._leftover(None, u2) == [(0, 0, 100), (1, 100, 100)]


def test_expert_exchange_plan_matches_a_plain_restatement():
  """The vectorised plan of the expert-parallel exchange against a row-by-row restatement of its layout:
  send side sorted by expert; receive side expert-major, every segment padded, sources in rank order."""
  import random
  from torchprime_b200.parallel.ep import _ExchangePlan
  random.seed(0)
  for ep, el, big in ((2, 2, False), (4, 3, False), (2, 4, True)):
    E = ep * el
    C = [[random.randint(0, 40) + (1200 if big else 0) for _ in range(E)] for _ in range(ep)]
    C[0][1] = 0
    for me in range(ep):
      p = _ExchangePlan(C, me, ep, el, "cpu")
      al = p.row_align
      assert al == (256 if big else 128)
      tot = [[sum(C[s][r * el + j] for s in range(ep)) for j in range(el)] for r in range(ep)]
      pad = lambda v: (v + al - 1) // al * al
      offpad = [[sum(pad(x) for x in tot[r][:j]) for j in range(el + 1)] for r in range(ep)]
      d = p.dispatch.tolist()
      start, rank, row0 = d[:E + 1], d[E + 1:2 * E + 1], d[2 * E + 1:]
      assert start == [sum(C[me][:e]) for e in range(E + 1)] and rank == [e // el for e in range(E)]
      assert row0 == [offpad[e // el][e % el] + sum(C[s][e] for s in range(me)) for e in range(E)]
      r = p.ret.tolist()
      nb = el * (ep + 1)
      rstart, rrank, rrow0 = r[:nb + 1], r[nb + 1:2 * nb + 1], r[2 * nb + 1:]
      want_start, want_rank, want_row0, zero = [], [], [], []
      for j in range(el):
        e, pos = me * el + j, offpad[me][j]
        for s in range(ep):
          want_start.append(pos); want_rank.append(s); want_row0.append(sum(C[s][:e])); pos += C[s][e]
        want_start.append(pos); want_rank.append(-1); want_row0.append(0)
        zero.extend(range(pos, offpad[me][j + 1]))
      want_start.append(offpad[me][el])
      assert (rstart, rrank, rrow0) == (want_start, want_rank, want_row0)
      assert (p.zero_rows.tolist() if p.zero_rows is not None else []) == zero
      assert p.n_pad == offpad[me][el] and p.k_offsets.tolist() == offpad[me]
      assert p.tile_expert.tolist() == [j for j in range(el) for _ in range((offpad[me][j + 1] - offpad[me][j]) // 128)]
