"""Snapshot tokenizer / model / dataset assets from the HF hub into a directory tree.

  python -m torchprime_b200.launcher.save_hf_assets --repo-id meta-llama/Meta-Llama-3-8B \
      --dest /data/assets --file-type tokenizer model
  python -m torchprime_b200.launcher.save_hf_assets --dataset-name wikitext --dataset-config wikitext-2-raw-v1 \
      --dest /data/assets --tokenizer meta-llama/Meta-Llama-3-8B --block-size 8192

Counterpart of the reference's launcher/save_hf_assets_to_gcs.py:1-187 (snapshot-download, then
``gsutil cp``): the destination here is a directory that the training job reads through
``model.pretrained_model`` / ``dataset.file_dataset_path``; shipping it to object storage is
left to whatever the site uses.  Needs network access and ``huggingface_hub`` / ``datasets``.
"""

from __future__ import annotations

import argparse
import os

TOKENIZER_PATTERNS = ["tokenizer*", "special_tokens_map.json", "*.model", "vocab.*", "merges.txt"]
MODEL_PATTERNS = ["*.safetensors*", "config.json", "generation_config.json"]


def save_repo(repo_id: str, dest: str, file_types, token=None) -> str:
  from huggingface_hub import snapshot_download
  patterns = []
  if "tokenizer" in file_types:
    patterns += TOKENIZER_PATTERNS
  if "model" in file_types:
    patterns += MODEL_PATTERNS
  out = os.path.join(dest, repo_id.replace("/", "--"))
  snapshot_download(repo_id=repo_id, allow_patterns=patterns, local_dir=out, token=token)
  return out


def save_dataset(name: str, config: str | None, dest: str, split: str, tokenizer: str | None, block_size: int | None):
  """Raw copy, or (with ``tokenizer`` and ``block_size``) the tokenised and packed dataset the
  trainer loads with ``dataset.is_preprocessed=true``."""
  import datasets
  out = os.path.join(dest, "datasets", name.replace("/", "--") + (f"--{config}" if config else ""))
  if tokenizer and block_size:
    from transformers import AutoTokenizer

    from ..data.dataset import make_train_dataset
    tok = AutoTokenizer.from_pretrained(tokenizer)
    blocks = make_train_dataset(name, config, split=split, tokenizer=tok, block_size=block_size)
    ds = datasets.Dataset.from_dict({"input_ids": [list(map(int, blocks[i]["input_ids"])) for i in range(len(blocks))]})
    out += f"--bs{block_size}"
  else:
    ds = datasets.load_dataset(name, config, split=split)
  ds.save_to_disk(out)
  return out


def main(argv=None):
  ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
  ap.add_argument("--repo-id")
  ap.add_argument("--file-type", nargs="+", default=["tokenizer", "model"], choices=["tokenizer", "model"])
  ap.add_argument("--dataset-name")
  ap.add_argument("--dataset-config")
  ap.add_argument("--split", default="train")
  ap.add_argument("--tokenizer")
  ap.add_argument("--block-size", type=int)
  ap.add_argument("--dest", required=True)
  ap.add_argument("--token", default=os.environ.get("HF_TOKEN"))
  a = ap.parse_args(argv)
  if not a.repo_id and not a.dataset_name:
    ap.error("give --repo-id and/or --dataset-name")
  os.makedirs(a.dest, exist_ok=True)
  if a.repo_id:
    print("saved", save_repo(a.repo_id, a.dest, a.file_type, a.token))
  if a.dataset_name:
    print("saved", save_dataset(a.dataset_name, a.dataset_config, a.dest, a.split, a.tokenizer, a.block_size))


if __name__ == "__main__":
  main()
