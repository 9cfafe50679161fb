"""Numerics of the model definitions against independent implementations (CPU, fp32)."""

import math

import pytest
import torch

from torchprime_b200.config import compose
from torchprime_b200.models import rope
from torchprime_b200.models.model_utils import initialize_model_class
from torchprime_b200.ops import reference as ref


def test_llama_matches_huggingface():
  tf = pytest.importorskip("transformers")
  cfg = compose("default", ["model=llama-tiny", "model.num_hidden_layers=2"]).model
  hf_cfg = tf.LlamaConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                          intermediate_size=cfg.intermediate_size, num_hidden_layers=cfg.num_hidden_layers,
                          num_attention_heads=cfg.num_attention_heads, num_key_value_heads=cfg.num_key_value_heads,
                          rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta, attention_bias=False,
                          max_position_embeddings=2048, tie_word_embeddings=False, attn_implementation="eager")
  torch.manual_seed(0)
  hf = tf.LlamaForCausalLM(hf_cfg).float()
  ours = initialize_model_class(cfg)
  ours.load_state_dict(hf.state_dict())
  for seq in (8, 128):
    ids = torch.randint(0, cfg.vocab_size, (2, seq))
    out = hf(input_ids=ids, labels=ids)
    logits, loss = ours(ids, labels=ids)
    assert torch.allclose(logits, out.logits, atol=2e-5), (logits - out.logits).abs().max()
    assert abs(loss.item() - out.loss.item()) < 1e-5
  hf.zero_grad(); ours.zero_grad()
  out.loss.backward(); loss.backward()
  hg = dict(hf.named_parameters())
  for n, p in ours.named_parameters():
    assert torch.allclose(p.grad, hg[n].grad, atol=2e-5), n


def test_llama31_rope_scaling_matches_huggingface():
  tf = pytest.importorskip("transformers")
  from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
  hf_cfg = tf.LlamaConfig(hidden_size=4096, num_attention_heads=32, rope_theta=500000.0, max_position_embeddings=131072,
                          rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                        "high_freq_factor": 4.0, "original_max_position_embeddings": 8192})
  try:
    want, _ = ROPE_INIT_FUNCTIONS["llama3"](hf_cfg, "cpu")
  except Exception:  # noqa: BLE001 - signature drift between transformers versions
    pytest.skip("ROPE_INIT_FUNCTIONS signature changed")
  got = rope.llama3_rope_frequencies(128, 500000.0, rope.RopeScaling())
  assert torch.allclose(got, want, rtol=1e-5)


def test_rope_against_scalar_loop():
  inv = rope.default_rope_frequencies(8, 10000.0)
  for i in range(4):
    assert inv[i].item() == pytest.approx(10000.0 ** (-2 * i / 8))
  cos, sin = rope.rope_tables(inv, 5, "cpu")
  x = torch.randn(1, 5, 1, 8)
  y = ref.rope_apply(x, torch.cat([cos, cos], -1), torch.cat([sin, sin], -1))
  for p in range(5):
    for i in range(4):
      a, b = x[0, p, 0, i].item(), x[0, p, 0, i + 4].item()
      ang = p * inv[i].item()
      assert y[0, p, 0, i].item() == pytest.approx(a * math.cos(ang) - b * math.sin(ang), abs=1e-5)
      assert y[0, p, 0, i + 4].item() == pytest.approx(b * math.cos(ang) + a * math.sin(ang), abs=1e-5)


def test_yarn_frequencies_interpolate_between_regimes():
  cfg = compose("default", ["model=deepseek-v3"]).model
  inv, factor = rope.yarn_rope_frequencies(cfg)
  base = 1.0 / (10000 ** (torch.arange(0, 64, 2).float() / 64))
  assert inv.shape == (32,) and torch.allclose(inv[0], base[0]) and factor == pytest.approx(1.0)
  scale = cfg.max_position_embeddings / cfg.rope_scaling.original_max_position_embeddings
  assert torch.allclose(inv[-1], base[-1] / scale)


def test_eager_attention_masks():
  torch.manual_seed(0)
  q, k, v = torch.randn(1, 6, 2, 4), torch.randn(1, 6, 1, 4), torch.randn(1, 6, 1, 4)
  o = ref.attention(q, k, v, causal=True)
  o_first = ref.attention(q[:, :1], k[:, :1], v[:, :1], causal=True)
  assert torch.allclose(o[:, :1], o_first, atol=1e-6)
  seg = torch.tensor([[0, 0, 0, 1, 1, 1]])
  o_seg = ref.attention(q, k, v, causal=True, q_segment_ids=seg)
  assert torch.allclose(o_seg[:, 3:], ref.attention(q[:, 3:], k[:, 3:], v[:, 3:], causal=True), atol=1e-6)
  o_win = ref.attention(q, k, v, causal=True, window=1)
  assert torch.allclose(o_win, v.expand(1, 6, 2, 4), atol=1e-6)


def test_deepseek_grouped_checkpoint_conversion_round_trip():
  from torchprime_b200.models.deepseek_v3 import (convert_hf_state_dict_for_grouped_moe,
                                                   revert_grouped_moe_to_hf_state_dict)
  cfg = compose("default", ["model=deepseek-tiny"]).model
  torch.manual_seed(0)
  m = initialize_model_class(cfg)
  sd = m.state_dict()
  hf = revert_grouped_moe_to_hf_state_dict(sd, cfg)
  assert "model.layers.1.mlp.experts.0.gate_proj.weight" in hf and "model.layers.1.mlp.grouped.W_gate" not in hf
  assert hf["model.layers.1.mlp.experts.3.down_proj.weight"].shape == (cfg.hidden_size, cfg.moe_intermediate_size)
  back = convert_hf_state_dict_for_grouped_moe(hf, cfg)
  assert back.keys() == sd.keys() and all(torch.equal(back[k], sd[k]) for k in sd)
  m2 = initialize_model_class(cfg)
  m2.load_state_dict(m2.convert_loaded_state_dict(hf))


def test_mixtral_dropping_matches_dense_when_capacity_is_large():
  base = ["model=mixtral-tiny", "model.capacity_factor=100.0"]
  torch.manual_seed(0)
  a = initialize_model_class(compose("default", base + ["model.moe_implementation=gmm"]).model)
  b = initialize_model_class(compose("default", base + ["model.moe_implementation=dropping"]).model)
  b.load_state_dict(a.state_dict())
  ids = torch.randint(0, 256, (2, 32))
  la, _ = a(ids)
  lb, loss_b = b(ids, labels=ids)
  assert torch.allclose(la, lb, atol=1e-5)
  tight = initialize_model_class(compose("default", ["model=mixtral-tiny", "model.capacity_factor=0.25",
                                                     "model.moe_implementation=dropping"]).model)
  tight.load_state_dict(a.state_dict())
  lt, _ = tight(ids)
  assert not torch.allclose(la, lt, atol=1e-4)   # tokens were dropped
