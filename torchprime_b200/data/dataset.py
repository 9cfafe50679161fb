"""Pre-training text datasets: tokenise a ``text`` column, concatenate and cut into fixed blocks.

Same entry point and sources as the reference's ``make_train_dataset``
(torchprime/data/dataset.py:98-191): a HuggingFace hub dataset, a dataset saved with
``save_to_disk`` (local or ``gs://``; ``is_preprocessed`` skips tokenisation) or a JSONL file with
a ``text`` field.  ``labels`` are a copy of ``input_ids`` (the model shifts).  The ``datasets``
package is imported lazily so synthetic-data runs do not need it.
"""

from __future__ import annotations

import json
import logging
from itertools import chain

import torch
from torch.utils.data import Dataset

logger = logging.getLogger(__name__)


class TokenBlockDataset(Dataset):
  """In-memory list of equal-length token blocks."""

  def __init__(self, blocks: list[list[int]], extra: dict | None = None):
    self.blocks = blocks
    self.extra = extra or {}

  def __len__(self):
    return len(self.blocks)

  def __getitem__(self, i):
    ids = torch.tensor(self.blocks[i], dtype=torch.int64)
    out = {"input_ids": ids, "labels": ids.clone()}
    for k, col in self.extra.items():
      out[k] = torch.tensor(col[i], dtype=torch.int64)
    return out


def group_texts(token_lists, block_size: int) -> list[list[int]]:
  """Concatenate all token lists and split into blocks of ``block_size`` (remainder dropped)."""
  flat = list(chain.from_iterable(token_lists))
  usable = (len(flat) // block_size) * block_size
  return [flat[i:i + block_size] for i in range(0, usable, block_size)]


def _read_jsonl(path: str) -> list[dict]:
  import fsspec
  rows = []
  with fsspec.open(path, "r") as f:
    for line in f:
      line = line.strip()
      if line:
        rows.append(json.loads(line))
  return rows


def _load_hf_dataset(name: str, config, split: str, cache_dir):
  import datasets
  if name.startswith("gs://") or name.startswith("/"):
    data = datasets.load_from_disk(name)
    if isinstance(data, datasets.DatasetDict):
      data = data[split]
    return data
  return datasets.load_dataset(name, config, split=split, cache_dir=cache_dir)


def load_hf_or_json_dataset(hf_dataset_name=None, hf_dataset_config_name=None, file_dataset_path=None,
                            split="train", cache_dir=None):
  """Rows as an indexable sequence of dicts from exactly one of the two sources."""
  if hf_dataset_name and file_dataset_path:
    raise ValueError("Only one of `hf_dataset_name` or `file_dataset_path` should be provided.")
  if hf_dataset_name:
    return _load_hf_dataset(hf_dataset_name, hf_dataset_config_name, split, cache_dir)
  if file_dataset_path:
    return _read_jsonl(file_dataset_path)
  raise ValueError("Either `hf_dataset_name` or `file_dataset_path` must be provided.")


def make_train_dataset(hf_dataset_name=None, hf_dataset_config_name=None, file_dataset_path=None,
                       is_preprocessed: bool = False, split: str = "train", cache_dir=None, *, tokenizer,
                       block_size: int, **_ignored) -> Dataset:
  if is_preprocessed:
    if not hf_dataset_name:
      raise ValueError("A path must be provided via `hf_dataset_name` when `is_preprocessed` is True.")
    data = _load_hf_dataset(hf_dataset_name, None, split, cache_dir)
    cols = getattr(data, "column_names", None) or list(data[0].keys())
    if "input_ids" not in cols:
      raise ValueError(f"Pre-processed dataset has no `input_ids` column (columns: {cols})")
    return TokenBlockDataset([list(r["input_ids"]) for r in data])
  rows = load_hf_or_json_dataset(hf_dataset_name, hf_dataset_config_name, file_dataset_path, split, cache_dir)
  texts = (r["text"] for r in rows)
  token_lists = (tokenizer(t)["input_ids"] for t in texts)
  blocks = group_texts(token_lists, block_size)
  logger.info("Built %d blocks of %d tokens", len(blocks), block_size)
  return TokenBlockDataset(blocks)
