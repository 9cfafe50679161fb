"""Cast a block-scaled FP8 (e4m3) DeepSeek checkpoint to bf16.

  python -m torchprime_b200.experimental.deepseek_inference.fp8_cast_bf16 \
      --input-fp8-hf-path <dir> --output-bf16-hf-path <dir>

The published DeepSeek-V3 weights store every 2-D weight as float8_e4m3fn plus a companion
``<name>_scale_inv`` of one fp32 factor per 128x128 block.  Capability reference:
torchprime/experimental/torchax_models/deepseek_v3/fp8_cast_bf16.py:12-113, which walks the
shards of the index, dequantises each fp8 weight with its scale, drops the scale entries and
rewrites the index; its dequantisation kernel is imported from a module the reference does not
ship, so the arithmetic here follows the checkpoint format itself.

Shards are processed one at a time; a scale living in another shard is fetched through the
index, and at most two foreign shards stay cached.
"""

from __future__ import annotations

import argparse
import glob
import json
import os

import torch

BLOCK = 128


def weight_dequant(weight: torch.Tensor, scale_inv: torch.Tensor, block: int = BLOCK,
                   out_dtype=torch.bfloat16) -> torch.Tensor:
  """``weight`` [M, N] (fp8 or any float) times the per-block factor
  ``scale_inv[ceil(M/block), ceil(N/block)]``."""
  assert weight.dim() == 2 and scale_inv.dim() == 2, (weight.shape, scale_inv.shape)
  m, n = weight.shape
  bm, bn = -(-m // block), -(-n // block)
  assert scale_inv.shape == (bm, bn), f"scale {tuple(scale_inv.shape)} does not tile weight {(m, n)}"
  s = scale_inv.float().repeat_interleave(block, 0)[:m].repeat_interleave(block, 1)[:, :n]
  return (weight.float() * s).to(out_dtype)


def weight_quant(weight: torch.Tensor, block: int = BLOCK):
  """Inverse used by the tests and for making fixtures: per-block absmax scaling to e4m3 (max 448)."""
  m, n = weight.shape
  bm, bn = -(-m // block), -(-n // block)
  pad = torch.zeros(bm * block, bn * block, dtype=torch.float32)
  pad[:m, :n] = weight.float()
  blocks = pad.view(bm, block, bn, block)
  amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
  scale_inv = amax / 448.0
  q = (blocks / scale_inv[:, None, :, None]).view(bm * block, bn * block)[:m, :n]
  return q.to(torch.float8_e4m3fn), scale_inv


def main(fp8_path: str, bf16_path: str) -> dict:
  from safetensors.torch import load_file, save_file
  os.makedirs(bf16_path, exist_ok=True)
  index_file = os.path.join(fp8_path, "model.safetensors.index.json")
  with open(index_file) as f:
    index = json.load(f)
  weight_map = index["weight_map"]
  cache: dict[str, dict] = {}

  def foreign(name):
    fname = weight_map[name]
    if fname not in cache:
      cache[fname] = load_file(os.path.join(fp8_path, fname), device="cpu")
      while len(cache) > 2:
        cache.pop(next(iter(cache)))
    return cache[fname][name]

  dropped = []
  for path in sorted(glob.glob(os.path.join(fp8_path, "*.safetensors"))):
    fname = os.path.basename(path)
    shard = load_file(path, device="cpu")
    out = {}
    for name, t in shard.items():
      if name.endswith("_scale_inv"):
        continue
      if t.element_size() == 1 and t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        sname = name + "_scale_inv"
        if sname in shard:
          scale = shard[sname]
        elif sname in weight_map:
          scale = foreign(sname)
        else:
          print(f"warning: no scale for {name}; plain cast")
          out[name] = t.to(torch.bfloat16)
          continue
        out[name] = weight_dequant(t, scale)
        dropped.append(sname)
      else:
        out[name] = t
    save_file(out, os.path.join(bf16_path, fname))
  new_map = {k: v for k, v in weight_map.items() if not k.endswith("_scale_inv")}
  new_index = {"metadata": index.get("metadata", {}), "weight_map": new_map}
  with open(os.path.join(bf16_path, "model.safetensors.index.json"), "w") as f:
    json.dump(new_index, f, indent=2)
  for extra in ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json"):
    src = os.path.join(fp8_path, extra)
    if os.path.exists(src):
      with open(src, "rb") as a, open(os.path.join(bf16_path, extra), "wb") as b:
        b.write(a.read())
  return {"tensors": len(new_map), "dequantised": len(dropped)}


if __name__ == "__main__":
  ap = argparse.ArgumentParser()
  ap.add_argument("--input-fp8-hf-path", required=True)
  ap.add_argument("--output-bf16-hf-path", required=True)
  a = ap.parse_args()
  print(main(a.input_fp8_hf_path, a.output_bf16_hf_path))
