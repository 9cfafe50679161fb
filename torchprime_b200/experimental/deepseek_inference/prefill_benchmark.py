"""Time the prefill (and optionally decode steps) of a randomly initialised DeepSeek model.

  python -m torchprime_b200.experimental.deepseek_inference.prefill_benchmark \
      [--model deepseek-v2-lite] [--layers 6] [--seqlen 2048] [--batch-size 1] [--attn-impl naive] \
      [--decode-steps 0] [--iters 5]

Capability reference: torchprime/experimental/torchax_models/deepseek_v3/prefill_benchmark.py:141-197
(random weights, sharded KV cache, three timed forward calls at a given sequence length and batch
size).  Here the timing is taken with CUDA events after warm-up and one JSON line is printed.
"""

from __future__ import annotations

import argparse
import json
import time

import torch

from .engine import DeepseekInferenceEngine


def run(model_name="deepseek-v2-lite", layers=None, seqlen=2048, batch_size=1, attn_impl="naive", decode_steps=0,
        iters=5, overrides=()):
  from ...config import compose
  from ...models.model_utils import initialize_model_class
  ov = [f"model={model_name}"] + list(overrides)
  if layers:
    ov.append(f"model.num_hidden_layers={layers}")
  cfg = compose("default", ov).model
  cuda = torch.cuda.is_available()
  dev = "cuda" if cuda else "cpu"
  torch.manual_seed(0)
  model = initialize_model_class(cfg, device=dev, dtype=torch.bfloat16 if cuda else torch.float32)
  engine = DeepseekInferenceEngine(model, batch_size, seqlen + decode_steps + 1, attn_impl)
  tokens = torch.randint(0, cfg.vocab_size, (batch_size, seqlen), device=dev)

  def timed(fn):
    if cuda:
      s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      torch.cuda.synchronize()
      s.record()
      fn()
      e.record()
      torch.cuda.synchronize()
      return s.elapsed_time(e)
    t0 = time.perf_counter()
    fn()
    return (time.perf_counter() - t0) * 1e3

  for _ in range(2):
    engine.forward(tokens, 0)
  prefill = sorted(timed(lambda: engine.forward(tokens, 0)) for _ in range(iters))[iters // 2]
  out = {"model": model_name, "layers": int(cfg.num_hidden_layers), "seqlen": seqlen, "batch_size": batch_size,
         "attn_impl": attn_impl, "prefill_ms": round(prefill, 3),
         "prefill_tokens_per_s": round(batch_size * seqlen / prefill * 1e3, 1),
         "cache_mb": round(engine.cache_bytes() / 2**20, 1)}
  if decode_steps:
    nxt = torch.randint(0, cfg.vocab_size, (batch_size, 1), device=dev)
    engine.forward(nxt, seqlen)
    total = timed(lambda: [engine.forward(nxt, seqlen + i) for i in range(decode_steps)])
    out["decode_ms_per_token"] = round(total / decode_steps, 3)
  return out


if __name__ == "__main__":
  ap = argparse.ArgumentParser()
  ap.add_argument("--model", default="deepseek-v2-lite")
  ap.add_argument("--layers", type=int, default=None)
  ap.add_argument("--seqlen", type=int, default=2048)
  ap.add_argument("--batch-size", type=int, default=1)
  ap.add_argument("--attn-impl", choices=["naive", "absorb"], default="naive")
  ap.add_argument("--decode-steps", type=int, default=0)
  ap.add_argument("--iters", type=int, default=5)
  a = ap.parse_args()
  print(json.dumps(run(a.model, a.layers, a.seqlen, a.batch_size, a.attn_impl, a.decode_steps, a.iters)))
