"""Supervised fine-tuning datasets: prompt/completion and chat formats, loss masking,
truncation, padding or sample-wise packing.

Semantics follow the reference (torchprime/data/sft_dataset.py:34-384):

* ``prompt_completion`` rows may use ``prompt``/``completion``, ``question``/``answer``
  (wrapped as ``"Question:\\n...\\n\\n\\nAnswer:\\n"``), ``text`` or ``completion`` alone;
* ``chat`` rows hold ``messages``; every message is rendered with the tokenizer's chat template
  and split on whitespace into tokens;
* ``compute_loss_on``: ``all`` | ``completion`` (last message / the completion) | ``assistant`` |
  ``last_assistant``; masked positions get label -100;
* EOS is always appended and trained on; over-long samples are cut on the ``right``, on the
  ``left`` or ``drop``-ped;
* samples are padded to ``block_size`` (pad id, else EOS; ``attention_mask`` marks real tokens) or
  packed greedily, never splitting a sample.

Extension: packed blocks also carry ``segment_ids`` so the attention kernels can keep samples from
attending to each other (the reference packs without such a mask).
"""

from __future__ import annotations

import torch
from torch.utils.data import Dataset

from .dataset import _load_hf_dataset, load_hf_or_json_dataset

IGNORE = -100


def _truncate(ids, labels, max_length, truncation):
  if len(ids) <= max_length:
    return ids, labels
  if truncation == "drop":
    return None, None
  if truncation == "left":
    return ids[-max_length:], labels[-max_length:]
  return ids[:max_length], labels[:max_length]


def _finish(ids, labels, tokenizer, max_length, truncation):
  if tokenizer.eos_token_id is not None:
    ids = ids + [tokenizer.eos_token_id]
    labels = labels + [tokenizer.eos_token_id]
  ids, labels = _truncate(ids, labels, max_length, truncation)
  return None if ids is None else {"input_ids": ids, "labels": labels}


def _tokenize_prompt_completion(example: dict, tokenizer, *, compute_loss_on, max_length, truncation):
  if "prompt" in example and "completion" in example:
    prompt, completion = example.get("prompt", ""), example.get("completion", "")
  elif "question" in example and "answer" in example:
    prompt = f"Question:\n{example.get('question', '')}\n\n\nAnswer:\n"
    completion = example.get("answer", "")
  elif "text" in example:
    prompt, completion = "", example["text"]
  elif "completion" in example:
    prompt, completion = "", example["completion"]
  else:
    raise ValueError(
      "Invalid input format: must contain 'prompt'/'completion' or 'question'/'answer' or 'text' fields.")
  p_ids = tokenizer.encode(prompt, add_special_tokens=False)
  c_ids = tokenizer.encode(completion, add_special_tokens=False)
  ids = p_ids + c_ids
  labels = list(ids)
  if compute_loss_on != "all":
    labels[:len(p_ids)] = [IGNORE] * len(p_ids)
  return _finish(ids, labels, tokenizer, max_length, truncation)


def _tokenize_chat(example: dict, tokenizer, *, compute_loss_on, max_length, truncation):
  messages = example["messages"]
  last_assistant = max((i for i, m in enumerate(messages) if m["role"] == "assistant"), default=None)
  ids, labels = [], []
  for i, message in enumerate(messages):
    text = tokenizer.apply_chat_template([message], tokenize=False).strip()
    m_ids = [tokenizer.convert_tokens_to_ids(tok) for tok in text.split()]
    ids.extend(m_ids)
    if compute_loss_on == "all":
      masked = False
    elif compute_loss_on == "assistant":
      masked = message["role"] != "assistant"
    elif compute_loss_on == "last_assistant":
      masked = not (message["role"] == "assistant" and i == last_assistant)
    else:
      masked = i != len(messages) - 1
    labels.extend([IGNORE] * len(m_ids) if masked else m_ids)
  return _finish(ids, labels, tokenizer, max_length, truncation)


def _pad_and_maybe_pack_samples(examples: dict, tokenizer, block_size: int, *, pack: bool) -> dict:
  """``examples``: columns ``input_ids`` / ``labels`` (lists of token lists).  Returns columns
  ``input_ids``, ``labels``, ``attention_mask`` (and ``segment_ids`` when packing)."""
  pad_id = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else tokenizer.eos_token_id
  out = {"input_ids": [], "labels": [], "attention_mask": []}
  if pack:
    out["segment_ids"] = []

  def emit(ids, labs, segs=None):
    n = len(ids)
    out["input_ids"].append(ids + [pad_id] * (block_size - n))
    out["labels"].append(labs + [IGNORE] * (block_size - n))
    out["attention_mask"].append([1] * n + [0] * (block_size - n))
    if pack:
      out["segment_ids"].append(segs + [0] * (block_size - n))

  if not pack:
    for ids, labs in zip(examples["input_ids"], examples["labels"], strict=True):
      emit(list(ids[:block_size]), list(labs[:block_size]))
    return out
  cur_ids, cur_labs, cur_seg, seg = [], [], [], 1
  for ids, labs in zip(examples["input_ids"], examples["labels"], strict=True):
    ids, labs = list(ids[:block_size]), list(labs[:block_size])
    if len(cur_ids) + len(ids) > block_size:
      emit(cur_ids, cur_labs, cur_seg)
      cur_ids, cur_labs, cur_seg, seg = [], [], [], 1
    cur_ids += ids
    cur_labs += labs
    cur_seg += [seg] * len(ids)
    seg += 1
    if len(cur_ids) == block_size:
      emit(cur_ids, cur_labs, cur_seg)
      cur_ids, cur_labs, cur_seg, seg = [], [], [], 1
  if cur_ids:
    emit(cur_ids, cur_labs, cur_seg)
  return out


class ColumnDataset(Dataset):
  def __init__(self, columns: dict, keys=("input_ids", "labels", "attention_mask")):
    self.columns = {k: columns[k] for k in keys if k in columns}
    self.n = len(next(iter(self.columns.values()))) if self.columns else 0

  def __len__(self):
    return self.n

  def __getitem__(self, i):
    return {k: torch.tensor(v[i], dtype=torch.int64) for k, v in self.columns.items()}

  @property
  def column_names(self):
    return list(self.columns)


def make_sft_dataset(hf_dataset_name=None, hf_dataset_config_name=None, file_dataset_path=None,
                     is_preprocessed: bool = False, split: str = "train", cache_dir=None,
                     format: str = "prompt_completion", compute_loss_on: str = "completion",
                     pack_samples: bool = False, truncation: str = "right", emit_segment_ids: bool = False, *,
                     tokenizer, block_size: int, **_ignored) -> Dataset:
  if is_preprocessed:
    if not hf_dataset_name:
      raise ValueError("A path must be provided via `hf_dataset_name` when `is_preprocessed` is True.")
    data = _load_hf_dataset(hf_dataset_name, None, split, cache_dir)
    cols = getattr(data, "column_names", None) or list(data[0].keys())
    required = ["input_ids", "labels", "attention_mask"]
    if not all(c in cols for c in required):
      raise ValueError("Pre-processed SFT dataset is missing one of the required columns:"
                       f" {required}. Available columns: {list(cols)}")
    return ColumnDataset({c: [list(r[c]) for r in data] for c in required})
  rows = load_hf_or_json_dataset(hf_dataset_name, hf_dataset_config_name, file_dataset_path, split, cache_dir)
  tok = _tokenize_prompt_completion if format == "prompt_completion" else _tokenize_chat
  ids, labels = [], []
  for ex in rows:
    out = tok(dict(ex), tokenizer, compute_loss_on=compute_loss_on, max_length=block_size, truncation=truncation)
    if out is not None:
      ids.append(out["input_ids"])
      labels.append(out["labels"])
  cols = _pad_and_maybe_pack_samples({"input_ids": ids, "labels": labels}, tokenizer, block_size, pack=pack_samples)
  keys = ["input_ids", "labels", "attention_mask"] + (["segment_ids"] if (pack_samples and emit_segment_ids) else [])
  return ColumnDataset(cols, keys)
