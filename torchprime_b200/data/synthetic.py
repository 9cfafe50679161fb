"""Synthetic pre-training data: uniform-random token ids derived from a seed.

Needs no tokenizer, dataset download or network, which is the default for benchmarks.
Each sample is generated from ``(seed, index)`` so every rank can produce exactly the
rows it needs and the stream is identical for any world size.
"""

from __future__ import annotations

import torch
from torch.utils.data import Dataset


class SyntheticTokenDataset(Dataset):
  def __init__(self, vocab_size: int, block_size: int, num_samples: int = 4096, seed: int = 42):
    self.vocab_size, self.block_size, self.num_samples, self.seed = vocab_size, block_size, num_samples, seed

  def __len__(self):
    return self.num_samples

  def __getitem__(self, idx: int):
    g = torch.Generator()
    g.manual_seed((self.seed * 1000003 + idx) & 0x7FFFFFFF)
    ids = torch.randint(0, self.vocab_size, (self.block_size,), generator=g, dtype=torch.int64)
    return {"input_ids": ids, "labels": ids.clone()}


def make_synthetic_dataset(*, vocab_size: int, block_size: int, num_samples: int = 4096, seed: int = 42, **_unused):
  return SyntheticTokenDataset(vocab_size, block_size, num_samples, seed)
