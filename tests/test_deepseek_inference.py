"""Cached DeepSeek inference (naive and absorbed MLA caches), generation, fp8 cast, HF conversion."""

import json
import os

import pytest
import torch

from torchprime_b200.config import compose
from torchprime_b200.experimental.deepseek_inference import convert, fp8_cast_bf16
from torchprime_b200.experimental.deepseek_inference.engine import (DeepseekInferenceEngine,
                                                                     full_forward_last_logits)
from torchprime_b200.experimental.deepseek_inference.generate import generate, sample
from torchprime_b200.models.model_utils import initialize_model_class


def _tiny():
  cfg = compose("default", ["model=deepseek-tiny"]).model
  torch.manual_seed(0)
  return cfg, initialize_model_class(cfg).eval()


@pytest.mark.parametrize("impl", ["naive", "absorb"])
def test_cached_forward_matches_the_training_model(impl):
  cfg, model = _tiny()
  eng = DeepseekInferenceEngine(model, max_batch_size=2, max_seq_len=32, attn_impl=impl)
  ids = torch.randint(0, cfg.vocab_size, (2, 12))
  want = full_forward_last_logits(model, ids)
  got = eng.forward(ids, 0)
  assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()
  # prefill 7, then one token at a time: the cache must reproduce the full forward at every step
  eng.forward(ids[:, :7], 0)
  for t in range(7, 12):
    step = eng.forward(ids[:, t:t + 1], t)
    assert torch.allclose(step, full_forward_last_logits(model, ids[:, :t + 1]), atol=2e-4)


def test_absorbed_cache_is_smaller_than_the_naive_one():
  _, model = _tiny()
  naive = DeepseekInferenceEngine(model, 1, 64, "naive").cache_bytes()
  absorb = DeepseekInferenceEngine(model, 1, 64, "absorb").cache_bytes()
  a = model.model.layers[0].self_attn
  ratio = a.num_heads * (a.qk_head_dim + a.v_head_dim) / (a.kv_lora_rank + a.qk_rope_head_dim)
  assert naive / absorb == pytest.approx(ratio)


def test_greedy_generation_equals_repeated_full_forward():
  cfg, model = _tiny()
  eng = DeepseekInferenceEngine(model, 2, 32, "absorb")
  prompts = [[5, 9, 17, 3], [7, 2]]
  outs = generate(eng, prompts, max_new_tokens=5, eos_id=-5, temperature=0.0)
  for p, o in zip(prompts, outs):
    seq = list(p)
    for tok in o:
      nxt = int(full_forward_last_logits(model, torch.tensor([seq])).argmax())
      assert tok == nxt
      seq.append(tok)
    assert len(o) == 5
  stop = outs[0][2]
  cut = generate(eng, prompts[:1], max_new_tokens=5, eos_id=stop, temperature=0.0)[0]
  assert cut == outs[0][: outs[0].index(stop)]


def test_sampling_follows_the_distribution():
  g = torch.Generator().manual_seed(0)
  logits = torch.tensor([[0.0, 1.0, 2.0]]).repeat(20000, 1)
  draws = sample(logits, 1.0, g)
  freq = torch.bincount(draws, minlength=3).float() / draws.numel()
  assert torch.allclose(freq, torch.softmax(logits[0], -1), atol=0.02)
  assert int(sample(torch.tensor([[0.0, 5.0, 1.0]]), 1e-6, g)) == 1


def test_fp8_block_dequant_and_checkpoint_cast(tmp_path):
  from safetensors.torch import load_file, save_file
  torch.manual_seed(0)
  w = torch.randn(200, 300) * 0.1
  q, s = fp8_cast_bf16.weight_quant(w)
  assert q.dtype == torch.float8_e4m3fn and s.shape == (2, 3)
  back = fp8_cast_bf16.weight_dequant(q, s, out_dtype=torch.float32)
  assert (back - w).abs().max() <= 0.07 * w.abs().max()          # e4m3: 3 mantissa bits
  src, dst = tmp_path / "fp8", tmp_path / "bf16"
  os.makedirs(src)
  norm = torch.ones(300, dtype=torch.bfloat16)
  save_file({"a.weight": q, "norm.weight": norm}, str(src / "s1.safetensors"))
  save_file({"a.weight_scale_inv": s}, str(src / "s2.safetensors"))     # the scale lives in another shard
  with open(src / "model.safetensors.index.json", "w") as f:
    json.dump({"metadata": {}, "weight_map": {"a.weight": "s1.safetensors", "norm.weight": "s1.safetensors",
                                              "a.weight_scale_inv": "s2.safetensors"}}, f)
  info = fp8_cast_bf16.main(str(src), str(dst))
  assert info == {"tensors": 2, "dequantised": 1}
  out = load_file(str(dst / "s1.safetensors"))
  assert out["a.weight"].dtype == torch.bfloat16 and torch.allclose(out["a.weight"].float(), back, atol=2e-3)
  idx = json.load(open(dst / "model.safetensors.index.json"))["weight_map"]
  assert "a.weight_scale_inv" not in idx and set(idx) == {"a.weight", "norm.weight"}


def test_hf_checkpoint_conversion_loads_into_the_model(tmp_path):
  from torchprime_b200.checkpoint import safetensors_io
  from torchprime_b200.models.deepseek_v3 import revert_grouped_moe_to_hf_state_dict
  cfg, model = _tiny()
  hf = revert_grouped_moe_to_hf_state_dict(model.state_dict(), cfg)
  hf[f"model.layers.{cfg.num_hidden_layers}.embed_tokens.weight"] = torch.zeros(2, 2)   # an MTP layer
  hf["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(4)
  safetensors_io.save_sharded_safetensors_by_layer(hf, str(tmp_path / "hf"))
  convert.main(str(tmp_path / "hf"), str(tmp_path / "ours"), "deepseek-tiny")
  fresh = initialize_model_class(cfg)
  fresh.from_pretrained(str(tmp_path / "ours"))
  for k, v in model.state_dict().items():
    assert torch.equal(fresh.state_dict()[k], v), k


def test_prefill_benchmark_reports_prefill_and_decode_times():
  from torchprime_b200.experimental.deepseek_inference.prefill_benchmark import run
  out = run("deepseek-tiny", None, 32, 2, "absorb", decode_steps=2, iters=3)
  assert out["prefill_ms"] > 0 and out["decode_ms_per_token"] > 0 and out["layers"] == 3
