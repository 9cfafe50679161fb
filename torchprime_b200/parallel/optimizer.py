"""Optimizers over the engine's flat shards, learning-rate schedules and gradient clipping.

The reference builds ``torch.optim.AdamW`` or HF ``Adafactor(relative_step=False,
scale_parameter=False)`` directly on bf16 parameters and clips with
``clip_grad_norm_`` / ``clip_grad_value_`` inside the compiled step
(torchprime/torch_xla_models/trainer/base_trainer.py:127-156,368-380).  Here the
optimizer state is sharded with the parameters (ZeRO-3): one fused AdamW launch updates
the fp32 master copy and both moments of this rank's shard and writes the bf16 compute
copy; the global gradient norm is a flat sum of squares plus a scalar all-reduce, and the
clip coefficient stays on the device (no host round trip inside the step).
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import functional as ops


_CHUNK = 1 << 27   # elements per slice in the plain-PyTorch optimizer path


def lr_lambda(kind: str, step: int, warmup: int, total: int) -> float:
  """Multiplier of the base learning rate at optimizer step ``step`` (0-based), matching
  ``transformers.get_scheduler`` for linear / cosine / constant(_with_warmup)."""
  if kind in ("constant",):
    return 1.0
  if step < warmup:
    return step / max(1, warmup)
  if kind == "constant_with_warmup":
    return 1.0
  if kind == "linear":
    return max(0.0, (total - step) / max(1, total - warmup))
  if kind == "cosine":
    prog = (step - warmup) / max(1, total - warmup)
    return max(0.0, 0.5 * (1.0 + math.cos(math.pi * prog)))
  raise ValueError(f"Unsupported lr_scheduler type: {kind}")


class LRScheduler:
  def __init__(self, base_lr: float, kind: str = "linear", warmup_steps: int = 0, total_steps: int = 1):
    self.base_lr, self.kind, self.warmup, self.total = base_lr, kind, warmup_steps, total_steps
    self.step_count = 0
    lr_lambda(kind, 0, warmup_steps, total_steps)  # validates `kind`

  def get_last_lr(self):
    return [self.base_lr * lr_lambda(self.kind, self.step_count, self.warmup, self.total)]

  def step(self):
    self.step_count += 1

  def state_dict(self):
    return {"step_count": self.step_count}

  def load_state_dict(self, sd):
    self.step_count = sd["step_count"]


class ShardedOptimizerBase:
  def __init__(self, engine):
    self.engine = engine
    dev = engine.device
    self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
    self._coef = torch.ones(1, dtype=torch.float32, device=dev)
    self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
    self.step_count = 0

  # ----------------------------------------------------------------- clipping
  def clip_gradients(self, max_norm: float | None, max_value: float | None = None) -> torch.Tensor:
    """Global L2 norm of all gradients (device scalar).  With ``max_norm`` > 0 the clip
    coefficient is stored for the next ``step``; ``max_value`` clamps element-wise first."""
    e = self.engine
    g = e.flat_grad
    use_k = e.is_cuda and ops.get_backend() != "torch"
    if max_value is not None and max_value > 0:
      g.clamp_(-max_value, max_value)
    def sumsq_into(acc, t):
      if t.numel() == 0:
        return
      if use_k:
        from ..ops import kernels as k
        k.sumsq_(t, acc)
      else:
        for lo in range(0, t.numel(), _CHUNK):   # bounded temporaries
          acc.add_(torch.linalg.vector_norm(t[lo:lo + _CHUNK], dtype=torch.float32).pow(2))

    # Dense shards are disjoint over the fsdp group; expert-parallel slices (the tail of the flat
    # buffers) are disjoint over the expert group, which need not be the same set of ranks.
    n_dense = getattr(e, "sharded_total", g.numel())
    local_sq = None
    if n_dense < g.numel():
      local_sq = torch.zeros_like(self._sumsq)
      sumsq_into(local_sq, g[n_dense:])
      ep_grp = e.mesh.group("expert") if (dist.is_initialized() and e.mesh is not None) else None
      if ep_grp is not None:
        dist.all_reduce(local_sq, group=ep_grp)
      tp_grp = e.mesh.group("tensor") if (dist.is_initialized() and e.mesh is not None) else None
      if tp_grp is not None and any(s.local and s.tp_dim is not None for u in e.units for s in u.slots):
        # expert weights are sliced over the tensor group as well (all of them, or none)
        assert all(s.tp_dim is not None for u in e.units for s in u.slots if s.local), (
          "expert-parallel parameters must be all tensor-parallel or all replicated over the tensor axis")
        dist.all_reduce(local_sq, group=tp_grp)
      g = g[:n_dense]
    self._sumsq.zero_()
    sumsq_into(self._sumsq, g)
    if dist.is_initialized() and e.mesh is not None:
      tp_grp = e.mesh.group("tensor")
      if tp_grp is not None:
        # tensor-parallel slices are disjoint over the tensor group, everything else is replicated
        # there: all-reduce only the sliced part so replicated gradients are counted once
        sliced = torch.zeros_like(self._sumsq)
        for start, n in self._tp_pieces():
          sumsq_into(sliced, g[start:start + n])
        self._sumsq.sub_(sliced)
        dist.all_reduce(sliced, group=tp_grp)
        self._sumsq.add_(sliced)
      fsdp_grp = e.mesh.group("fsdp")
      if fsdp_grp is not None:
        dist.all_reduce(self._sumsq, group=fsdp_grp)
    if local_sq is not None:
      self._sumsq.add_(local_sq)
    if use_k:
      from ..ops import kernels as k
      k.clip_coef_(self._sumsq, max_norm or 0.0, self._coef, self._norm)
    else:
      self._norm.copy_(self._sumsq.sqrt())
      if max_norm is not None and max_norm > 0:
        self._coef.copy_(torch.clamp(max_norm / (self._norm + 1e-6), max=1.0))
      else:
        self._coef.fill_(1.0)
    return self._norm

  def _tp_pieces(self):
    """(start, length) ranges of this rank's flat shard that belong to tensor-parallel sliced parameters."""
    if getattr(self, "_tp_piece_cache", None) is None:
      e = self.engine
      pieces = []
      for u in e.units:
        lo, hi = e.fsdp_rank * u.shard_size, (e.fsdp_rank + 1) * u.shard_size
        for s in u.slots:
          if s.tp_dim is None or s.local:
            continue
          a, b = max(lo, s.offset), min(hi, s.offset + s.numel)
          if a < b:
            pieces.append((u.shard_offset + a - lo, b - a))
      self._tp_piece_cache = pieces
    return self._tp_piece_cache

  def zero_grad(self):
    self.engine.zero_grad()


class ShardedAdamW(ShardedOptimizerBase):
  def __init__(self, engine, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
    super().__init__(engine)
    self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
    n = engine.total_shard
    self.exp_avg = torch.zeros(n, dtype=torch.float32, device=engine.device)
    self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=engine.device)

  def step(self, lr: float | None = None):
    e = self.engine
    lr = self.lr if lr is None else lr
    self.step_count += 1
    master = e.flat_master if e.flat_master is not None else e.flat_param
    p16 = e.flat_param if e.master_weights else None
    e.params_will_change()
    if e.is_cuda and ops.get_backend() != "torch" and master.dtype == torch.float32 and master.numel() % 4 == 0:
      from ..ops import kernels as k
      k.adamw_(master, self.exp_avg, self.exp_avg_sq, e.flat_grad, p16, lr, self.betas[0], self.betas[1],
               self.eps, self.weight_decay, self.step_count, clip_coef=self._coef)
    else:
      from ..ops import reference as ref
      for lo in range(0, master.numel(), _CHUNK):   # bounded temporaries
        sl = slice(lo, lo + _CHUNK)
        p32 = master[sl] if master.dtype == torch.float32 else master[sl].float()
        ref.adamw_step(p32, e.flat_grad[sl], self.exp_avg[sl], self.exp_avg_sq[sl], lr, self.betas[0],
                       self.betas[1], self.eps, self.weight_decay, self.step_count, grad_scale=self._coef)
        if master.dtype != torch.float32:
          master[sl].copy_(p32)
        if p16 is not None:
          p16[sl].copy_(master[sl])
    e.params_changed()

  def state_dict(self):
    return {"exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq, "step": self.step_count}

  def load_state_dict(self, sd):
    self.exp_avg.copy_(sd["exp_avg"])
    self.exp_avg_sq.copy_(sd["exp_avg_sq"])
    self.step_count = int(sd["step"])


class ShardedAdafactor(ShardedOptimizerBase):
  """Adafactor with a fixed learning rate (``relative_step=False, scale_parameter=False``,
  no momentum, ``clip_threshold=1.0``, ``decay_rate=-0.8``, eps (1e-30, 1e-3)) as the
  reference configures HF's implementation (base_trainer.py:143-152).

  Second moments are factored per parameter *shard piece*: the piece of a >=2-D parameter
  that lives in this rank's flat shard is viewed as whole rows of its last dimension;
  row statistics are local and column statistics are summed over the fsdp group, so the
  factored estimate equals the un-sharded one.  Ragged leftovers (a shard boundary that
  cuts a row) and 1-D parameters use the un-factored second moment."""

  def __init__(self, engine, lr: float, eps=(1e-30, 1e-3), clip_threshold: float = 1.0, decay_rate: float = -0.8,
               weight_decay: float = 0.0):
    super().__init__(engine)
    if weight_decay:
      raise ValueError("Adafactor does not support weight decay.")
    self.lr, self.eps, self.clip_threshold, self.decay_rate = lr, eps, clip_threshold, decay_rate
    self.pieces = self._plan_pieces()

  def _plan_pieces(self):
    """Flat (un-factored) pieces plus, for every >=2-D parameter, one entry per rank describing the
    whole rows of it (possibly none) that live in this rank's shard.  Every rank lists every
    factored parameter in the same order so the statistics exchange is one uniform all-reduce."""
    e = self.engine
    pieces = []
    for u in e.units:
      lo, hi = e.fsdp_rank * u.shard_size, (e.fsdp_rank + 1) * u.shard_size
      for s in u.slots:
        cols = s.shape[-1] if len(s.shape) >= 2 else None
        if s.local:
          start = e.sharded_total + s.local_offset
          if cols is None:
            pieces.append({"kind": "flat", "start": start, "n": s.numel, "v": None})
          else:
            pieces.append({"kind": "rows", "start": start, "rows": s.numel // cols, "cols": cols,
                           "total_rows": s.numel // cols, "vr": None, "vc": None, "shared": False})
          continue
        a, b = max(lo, s.offset), min(hi, s.offset + s.numel)
        has = a < b
        start = u.shard_offset + (a - lo)
        rel0, rel1 = a - s.offset, b - s.offset
        if cols is None:
          if has:
            pieces.append({"kind": "flat", "start": start, "n": b - a, "v": None})
          continue
        first_row = -(-rel0 // cols) if has else 0
        last_row = rel1 // cols if has else 0
        head_n = (min(first_row * cols, rel1) - rel0) if has else 0
        if head_n > 0:
          pieces.append({"kind": "flat", "start": start, "n": head_n, "v": None})
        pieces.append({"kind": "rows", "start": start + head_n, "rows": max(0, last_row - first_row), "cols": cols,
                       "total_rows": s.numel // cols, "vr": None, "vc": None, "shared": e.fsdp > 1})
        if has:
          tail0 = max(last_row, first_row) * cols
          if rel1 > tail0 and tail0 >= rel0 + head_n:
            pieces.append({"kind": "flat", "start": start + (tail0 - rel0), "n": rel1 - tail0, "v": None})
    return pieces

  def step(self, lr: float | None = None):
    e = self.engine
    lr = self.lr if lr is None else lr
    self.step_count += 1
    beta2t = 1.0 - math.pow(self.step_count, self.decay_rate)
    master = e.flat_master if e.flat_master is not None else e.flat_param
    coef = self._coef
    dev = e.flat_grad.device
    grp = e.fsdp_group if e.fsdp > 1 else None
    e.params_will_change()

    def apply(sl, upd, n):
      rms = upd.norm(2) / math.sqrt(n)
      upd = upd / torch.clamp(rms / self.clip_threshold, min=1.0)
      master[sl].add_(upd.to(master.dtype), alpha=-lr)

    # phase 1: local statistics; factored pieces queue their column sums and row-moment sums
    shared_stats, work = [], []
    for pc in self.pieces:
      if pc["kind"] == "flat":
        sl = slice(pc["start"], pc["start"] + pc["n"])
        g = e.flat_grad[sl].float() * coef
        upd = g * g + self.eps[0]
        if pc["v"] is None:
          pc["v"] = torch.zeros_like(upd)
        pc["v"].mul_(beta2t).add_(upd, alpha=1.0 - beta2t)
        apply(sl, g * pc["v"].rsqrt(), pc["n"])
        continue
      r, c = pc["rows"], pc["cols"]
      if pc["vr"] is None:
        pc["vr"] = torch.zeros(r, dtype=torch.float32, device=dev)
        pc["vc"] = torch.zeros(c, dtype=torch.float32, device=dev)
      g = None
      col_sum = torch.zeros(c, dtype=torch.float32, device=dev)
      if r > 0:
        sl = slice(pc["start"], pc["start"] + r * c)
        g = (e.flat_grad[sl].float() * coef).view(r, c)
        sq = g * g + self.eps[0]
        col_sum = sq.sum(0)
        pc["vr"].mul_(beta2t).add_(sq.mean(-1), alpha=1.0 - beta2t)
      stat = torch.cat([col_sum, pc["vr"].sum().reshape(1)])
      if pc["shared"]:
        shared_stats.append(stat)
      work.append((pc, g, stat))
    if shared_stats and grp is not None:
      flat = torch.cat(shared_stats)
      dist.all_reduce(flat, group=grp)
      off = 0
      for i, (pc, g, stat) in enumerate(work):
        if pc["shared"]:
          n = stat.numel()
          work[i] = (pc, g, flat[off:off + n])
          off += n
    # phase 2: factored update
    for pc, g, stat in work:
      c = pc["cols"]
      pc["vc"].mul_(beta2t).add_(stat[:c] / pc["total_rows"], alpha=1.0 - beta2t)
      if g is None:
        continue
      row_mean = stat[c] / pc["total_rows"]
      r_factor = (pc["vr"] / row_mean).rsqrt().unsqueeze(-1)
      c_factor = pc["vc"].rsqrt().unsqueeze(0)
      upd = (g * r_factor * c_factor).reshape(-1)
      apply(slice(pc["start"], pc["start"] + upd.numel()), upd, upd.numel())
    if e.master_weights:
      e.flat_param.copy_(master)
    e.params_changed()

  def state_dict(self):
    return {"step": self.step_count, "pieces": [{k: v for k, v in p.items() if k in ("v", "vr", "vc")}
                                                for p in self.pieces]}

  def load_state_dict(self, sd):
    self.step_count = int(sd["step"])
    for p, saved in zip(self.pieces, sd["pieces"]):
      p.update(saved)


def create_optimizer(task_config, engine):
  """``adamw`` or ``adafactor`` from ``task.optimizer`` (same keys and errors as the
  reference's ``Trainer._create_optimizer``)."""
  oc = task_config.optimizer
  kind = str(oc.type).lower()
  if kind == "adamw":
    kw = {}
    if oc.get("weight_decay", None) is not None:
      kw["weight_decay"] = float(oc.weight_decay)
    if oc.get("betas", None) is not None:
      kw["betas"] = tuple(oc.betas)
    return ShardedAdamW(engine, lr=float(oc.learning_rate), **kw)
  if kind == "adafactor":
    if oc.get("weight_decay", None):
      raise ValueError("Adafactor does not support weight decay.")
    return ShardedAdafactor(engine, lr=float(oc.learning_rate))
  raise ValueError(f"Unsupported optimizer type: {oc.type}. Supported types are 'adafactor' and 'adamw'.")
