"""Per-rank input pipeline: sharded sampling, collation, pinned staging and asynchronous
host-to-device copies on a side stream.

Replaces the reference's ``DistributedSampler`` + ``pl.MpDeviceLoader(input_sharding=...)``
(torchprime/torch_xla_models/trainer/base_trainer.py:171-211).  Every rank loads only the
rows of the global batch that belong to its (data, fsdp[, expert]) coordinate — the
"minibatch" mode of the reference; ranks of one tensor/context group read the same rows.
Like the reference the sampler shuffles with a fixed seed and is never re-seeded per
epoch, the last incomplete batch is dropped, and the iterator restarts when exhausted.
"""

from __future__ import annotations

import torch
from torch.utils.data import Dataset


def default_collate(samples: list[dict]) -> dict:
  out = {}
  for k in samples[0]:
    vals = [s[k] for s in samples]
    out[k] = torch.stack([v if isinstance(v, torch.Tensor) else torch.as_tensor(v) for v in vals])
  return out


class ShardedBatchLoader:
  def __init__(self, dataset: Dataset, global_batch_size: int, num_replicas: int, replica_rank: int,
               device: torch.device, shuffle: bool = True, seed: int = 0, prefetch: bool = True, collate=None):
    assert global_batch_size % num_replicas == 0, (
      f"global batch {global_batch_size} must be divisible by the number of batch shards {num_replicas}")
    self.dataset = dataset
    self.local_batch = global_batch_size // num_replicas
    self.global_batch = global_batch_size
    self.num_replicas, self.replica_rank = num_replicas, replica_rank
    self.device = torch.device(device)
    self.shuffle, self.seed = shuffle, seed
    self.collate = collate or default_collate
    self.epoch_batches = len(dataset) // global_batch_size
    assert self.epoch_batches > 0, "dataset smaller than one global batch"
    self.copy_stream = torch.cuda.Stream(device=self.device) if (self.device.type == "cuda" and prefetch) else None
    self._order = None
    self._cursor = 0          # global batches consumed in total (resumable)
    self._staged = None
    self.h2d_bytes_last = 0

  # ------------------------------------------------------------------ ordering
  def _epoch_order(self):
    if self._order is None:
      n = len(self.dataset)
      if self.shuffle:
        g = torch.Generator()
        g.manual_seed(self.seed)
        self._order = torch.randperm(n, generator=g).tolist()
      else:
        self._order = list(range(n))
    return self._order

  def _indices(self, batch_no: int) -> list[int]:
    order = self._epoch_order()
    b = batch_no % self.epoch_batches
    base = b * self.global_batch + self.replica_rank * self.local_batch
    return order[base:base + self.local_batch]

  # ------------------------------------------------------------------ staging
  def _load_host(self, batch_no: int) -> dict:
    batch = self.collate([self.dataset[i] for i in self._indices(batch_no)])
    if self.device.type == "cuda":
      batch = {k: v.pin_memory() for k, v in batch.items()}
    return batch

  def _to_device(self, host: dict):
    if self.device.type != "cuda":
      return host, None
    nbytes = sum(v.numel() * v.element_size() for v in host.values())
    if self.copy_stream is None:
      dev = {k: v.to(self.device, non_blocking=True) for k, v in host.items()}
      return dev, nbytes
    with torch.cuda.stream(self.copy_stream):
      dev = {k: v.to(self.device, non_blocking=True) for k, v in host.items()}
      ev = torch.cuda.Event()
      ev.record(self.copy_stream)
    return (dev, ev, host), nbytes

  def next_batch(self) -> dict:
    """The next local batch on the device.  The following batch is already being read and
    copied while the caller computes."""
    if self._staged is None:
      self._staged = self._to_device(self._load_host(self._cursor))
    staged, nbytes = self._staged
    self.h2d_bytes_last = nbytes or 0
    self._cursor += 1
    if self.copy_stream is not None:
      dev, ev, _host = staged
      torch.cuda.current_stream().wait_event(ev)
      for v in dev.values():
        v.record_stream(torch.cuda.current_stream())
      batch = dev
    else:
      batch = staged
    self._staged = self._to_device(self._load_host(self._cursor)) if self.copy_stream is not None else None
    return batch

  def __iter__(self):
    while True:
      yield self.next_batch()

  @property
  def epoch(self) -> float:
    return self._cursor / self.epoch_batches

  def state_dict(self):
    return {"cursor": self._cursor}

  def load_state_dict(self, sd):
    self._cursor = int(sd["cursor"])
    self._staged = None
