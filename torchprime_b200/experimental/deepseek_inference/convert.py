"""Convert a Hugging Face DeepSeek-V3 / V2-Lite checkpoint to this framework's layout.

  python -m torchprime_b200.experimental.deepseek_inference.convert --hf-ckpt-path <dir> \
      --save-path <dir> --model deepseek-v2-lite

Capability reference: torchprime/experimental/torchax_models/deepseek_v3/convert.py:32-95, which
renames HF keys to its inference model's names and splits experts over model-parallel ranks.
Here the training model keeps the HF names, so conversion is: read the (bf16) shards, fold the
per-expert ``mlp.experts.<i>.{gate,up,down}_proj`` matrices into the grouped tensors the grouped
GEMM consumes, drop multi-token-prediction layers beyond ``num_hidden_layers``, and write one
safetensors shard per layer plus the index.  Expert-parallel placement happens at load time
from the sharding config, not in the file layout.
"""

from __future__ import annotations

import argparse
import json
import os
import re

import torch


def convert_state_dict(hf_state: dict, config) -> dict:
  from ...models.deepseek_v3 import convert_hf_state_dict_for_grouped_moe
  n = int(config.num_hidden_layers)
  kept = {}
  for k, v in hf_state.items():
    m = re.match(r"model\.layers\.(\d+)\.", k)
    if m and int(m.group(1)) >= n:
      continue                                   # multi-token-prediction heads
    if k.endswith("rotary_emb.inv_freq"):
      continue
    kept[k] = v
  return convert_hf_state_dict_for_grouped_moe(kept, config)


def main(hf_ckpt_path: str, save_path: str, model: str) -> dict:
  from ...checkpoint import safetensors_io
  from ...config import compose, to_container
  cfg = compose("default", [f"model={model}"]).model
  state = safetensors_io.load_safetensors_to_state_dict(hf_ckpt_path)
  if any(t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) for t in state.values()):
    raise ValueError("the checkpoint holds fp8 weights: run fp8_cast_bf16 first")
  out = convert_state_dict(state, cfg)
  safetensors_io.save_sharded_safetensors_by_layer(out, save_path)
  with open(os.path.join(save_path, "config.json"), "w") as f:
    json.dump(to_container(cfg), f, indent=2)
  for extra in ("tokenizer.json", "tokenizer_config.json", "generation_config.json"):
    src = os.path.join(hf_ckpt_path, extra)
    if os.path.exists(src):
      with open(src, "rb") as a, open(os.path.join(save_path, extra), "wb") as b:
        b.write(a.read())
  return {"tensors": len(out)}


if __name__ == "__main__":
  ap = argparse.ArgumentParser()
  ap.add_argument("--hf-ckpt-path", required=True)
  ap.add_argument("--save-path", required=True)
  ap.add_argument("--model", default="deepseek-v2-lite")
  a = ap.parse_args()
  print(main(a.hf_ckpt_path, a.save_path, a.model))
