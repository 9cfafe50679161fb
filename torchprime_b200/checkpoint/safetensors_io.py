"""HF-compatible sharded safetensors export / import ("format A").

On-disk layout (kept byte-for-byte compatible with what the reference writes,
torchprime/torch_xla_models/model/model_utils.py:35-135,248-281, so exported models load
in HF / vLLM and the reference's own loader):

* one ``<group>.safetensors`` per parameter group: ``layers_<i>`` for
  ``{model,encoder,decoder}.layers.<i>.*``, ``<block>_<i>`` for any ``<block>.<i>.*``,
  otherwise the first path component — so ``model.embed_tokens.weight`` and
  ``model.norm.weight`` land in a shard literally named ``model.safetensors``;
* ``model.safetensors.index.json`` = ``{"weight_map": {param: file}}`` (no metadata
  block); a loader that finds the index uses it, else reads a single
  ``model.safetensors``;
* wrapper infixes (``._orig_mod``) are stripped from keys; tensors keep their dtype.
"""

from __future__ import annotations

import json
import logging
import contextlib
import os
import shutil
import tempfile
from collections import defaultdict
from concurrent.futures import ThreadPoolExecutor
from contextlib import contextmanager

import torch

logger = logging.getLogger(__name__)
INDEX_NAME = "model.safetensors.index.json"
SINGLE_NAME = "model.safetensors"


def get_param_group_key(param_name: str) -> str:
  parts = param_name.split(".")
  if parts and parts[0] == "module":
    parts = parts[1:]
  if len(parts) >= 3 and parts[0] in ("model", "encoder", "decoder") and parts[1] == "layers" and parts[2].isdigit():
    return f"layers_{parts[2]}"
  if len(parts) >= 2 and parts[1].isdigit():
    return f"{parts[0]}_{parts[1]}"
  return parts[0]


def _clean_key(k: str) -> str:
  return k.replace("._orig_mod", "")


def save_sharded_safetensors_by_layer(state_dict: dict, save_dir: str, tmp_dir: str | None = None,
                                      max_workers: int = 24) -> None:
  """Write one shard per parameter group plus the index.  With ``tmp_dir`` shards are
  written there first and then moved (useful when ``save_dir`` is a slow mount)."""
  from safetensors.torch import save_file
  os.makedirs(save_dir, exist_ok=True)
  work_dir = tmp_dir or save_dir
  os.makedirs(work_dir, exist_ok=True)
  groups: dict[str, dict] = defaultdict(dict)
  for k, v in state_dict.items():
    key = _clean_key(k)
    groups[get_param_group_key(key)][key] = v.detach().contiguous().cpu()
  weight_map = {}

  def write(item):
    group, tensors = item
    fname = f"{group}.safetensors"
    save_file(tensors, os.path.join(work_dir, fname))
    return fname, list(tensors)

  with ThreadPoolExecutor(max_workers=max(1, min(max_workers, len(groups)))) as ex:
    for fname, keys in ex.map(write, groups.items()):
      for k in keys:
        weight_map[k] = fname
  with open(os.path.join(work_dir, INDEX_NAME), "w") as f:
    json.dump({"weight_map": weight_map}, f, indent=2)
  if work_dir != save_dir:
    for fname in set(weight_map.values()) | {INDEX_NAME}:
      shutil.move(os.path.join(work_dir, fname), os.path.join(save_dir, fname))


def load_safetensors_to_state_dict(model_dir: str) -> dict:
  """Read every tensor of an exported / HF model directory (index-aware)."""
  from safetensors import safe_open
  state = {}
  index = os.path.join(model_dir, INDEX_NAME)
  if os.path.exists(index):
    with open(index) as f:
      weight_map = json.load(f)["weight_map"]
    for fname in sorted(set(weight_map.values())):
      with safe_open(os.path.join(model_dir, fname), framework="pt", device="cpu") as sf:
        for k in sf.keys():
          state[k] = sf.get_tensor(k)
    return state
  single = os.path.join(model_dir, SINGLE_NAME)
  if os.path.exists(single):
    with safe_open(single, framework="pt", device="cpu") as sf:
      for k in sf.keys():
        state[k] = sf.get_tensor(k)
    return state
  raise FileNotFoundError(f"No *.safetensors found in {model_dir}")


@contextmanager
def local_path_from_gcs(path_or_repo: str, temp_dir: str | None = None):
  """``gs://`` paths are copied to a temporary local directory with ``gsutil``; anything
  else is passed through.  The copy is removed when the context exits."""
  if not str(path_or_repo).startswith("gs://"):
    yield path_or_repo
    return
  import subprocess
  local = tempfile.mkdtemp(dir=temp_dir)
  try:
    subprocess.run(["gsutil", "-m", "cp", "-r", path_or_repo.rstrip("/") + "/*", local], check=True)
    yield local
  finally:
    shutil.rmtree(local, ignore_errors=True)


@contextlib.contextmanager
def model_dir(path_or_repo: str):
  """Context manager yielding a local directory with the model files of a local directory, a
  ``gs://`` prefix (copied to a temporary directory that is removed on exit) or an HF hub repo id."""
  if os.path.isdir(path_or_repo):
    yield path_or_repo
  elif str(path_or_repo).startswith("gs://"):
    with local_path_from_gcs(path_or_repo) as local:
      yield local
  else:
    from ..utils.retry import retry
    import huggingface_hub
    yield retry(lambda: huggingface_hub.snapshot_download(
      repo_id=path_or_repo, allow_patterns=["*.safetensors*", "config.json", "generation_config.json"]))


def copy_hf_config_files(pretrained: str | None, save_dir: str) -> None:
  """Copy ``config.json`` / ``generation_config.json`` of the base model next to the export."""
  if not pretrained:
    return
  try:
    with model_dir(pretrained) as src:
      for name in ("config.json", "generation_config.json"):
        p = os.path.join(src, name)
        if os.path.exists(p):
          shutil.copy(p, os.path.join(save_dir, name))
  except Exception as e:  # noqa: BLE001 - offline boxes cannot reach the hub
    logger.warning("could not fetch HF config files of %s: %s", pretrained, e)


def save_hf_tokenizer(tokenizer_name: str | None, save_dir: str) -> None:
  if not tokenizer_name:
    return
  try:
    from transformers import AutoTokenizer
    AutoTokenizer.from_pretrained(tokenizer_name).save_pretrained(save_dir)
  except Exception as e:  # noqa: BLE001
    logger.warning("could not save tokenizer %s: %s", tokenizer_name, e)
