"""The side models and adapters the reference ships next to the LLM trainer: ResNet-18 classification
(torchprime/torch_xla_vision_models/train.py, torchprime/models/resnet18), the TransAct forward
benchmark model (torchprime/models/transact), the benchmark model registry and the HuggingFace
``run_clm.py`` command adapter (torchprime/hf_models/train.py)."""

import csv
import sys

import pytest
import torch

from torchprime_b200.config import compose


def test_registry_models_run_forward():
  from torchprime_b200.models import registry
  assert set(registry) == {"pinterest/transformer_user_action", "resnet18"}
  for name, factory in registry.items():
    m = factory().eval()
    args, kwargs = m.get_sample_inputs(2)
    with torch.no_grad():
      out = m(*args, **kwargs)
    assert out.shape[0] == 2 and torch.isfinite(out).all(), name


def test_transact_output_layout_and_masking():
  from torchprime_b200.models.transact import TransAct, TransActConfig
  cfg = TransActConfig(seq_len=12, latest_n_emb=3, item_emb_dim=8, action_emb_dim=8, nhead=2, dim_feedforward=16)
  torch.manual_seed(0)
  m = TransAct(cfg).eval()
  b = 3
  act = torch.randint(0, 20, (b, 12))
  items, times = torch.rand(b, 12, 8), torch.randint(0, 100, (b, 12))
  req, cand = torch.randint(500, 1000, (b,)), torch.rand(b, 8)
  out = m(act, items, times, req, cand)
  d_model = 8 + 2 * 8
  assert out.shape == (b, d_model + 3 * d_model)          # max-pool head + the 3 latest positions
  # padded actions (-1 maps to the padding entry) are masked out of the attention: changing their
  # item embeddings must not change the output of the other positions' pooled summary
  act2 = act.clone()
  act2[:, 6:] = -1
  out_a = m(act2, items, times, req, cand)
  items_b = items.clone()
  items_b[:, 6:] += 10.0
  out_b = m(act2, items_b, times, req, cand)
  assert torch.allclose(out_a[:, d_model:], out_b[:, d_model:], atol=1e-5)


def test_resnet18_freeze_unfreeze_and_hash():
  from torchprime_b200.models.resnet18 import Resnet18ForClassification, state_dict_hash
  a = Resnet18ForClassification(num_classes=7, seed=1, pretrained=False)
  b = Resnet18ForClassification(num_classes=7, seed=1, pretrained=False)
  assert a.model_hash == b.model_hash == state_dict_hash(a.model)
  assert a(torch.randn(2, 3, 64, 64)).shape == (2, 7)
  a.freeze_backbone()
  trainable = [n for n, p in a.named_parameters() if p.requires_grad]
  assert trainable and all(n.startswith(("model.fc", "model.conv1", "model.bn1")) for n in trainable)
  a.unfreeze_all()
  assert all(p.requires_grad for p in a.parameters())


def test_vision_training_loop_learns_and_writes_csv(tmp_path):
  from torchprime_b200.vision.train import cosine_with_warmup, train
  assert cosine_with_warmup(0, 10, 100) == 0.0 and cosine_with_warmup(10, 10, 100) == 1.0
  assert cosine_with_warmup(100, 10, 100) == pytest.approx(0.0, abs=1e-9)
  out = tmp_path / "metrics.csv"
  rows = train(num_classes=4, epochs=2, freeze_epochs=1, batch_size=16, lr=3e-3, train_samples=64,
               out_csv=str(out), device="cpu", seed=0)
  assert len(rows) == 2 and rows[1]["train_loss"] < rows[0]["train_loss"]
  with open(out) as f:
    got = list(csv.DictReader(f))
  assert [r["epoch"] for r in got] == ["0", "1"] and set(got[0]) >= {"train_loss", "val_accuracy", "model_hash"}


def test_hf_adapter_builds_the_run_clm_command(tmp_path):
  from torchprime_b200.hf_models.train import build_command
  cfg = compose("default", ["task.global_batch_size=16", "ici_mesh.fsdp=4", "task.max_steps=7",
                            f"output_dir={tmp_path}", "+train_script.path=/opt/run_clm.py",
                            "+train_script.args.block_size=1024", "+train_script.args.bf16=false"])
  cmd, env = build_command(cfg)
  assert cmd[:2] == [sys.executable, "/opt/run_clm.py"]
  flags = dict(a[2:].split("=", 1) for a in cmd[2:])
  assert flags["block_size"] == "1024" and flags["per_device_train_batch_size"] == "4"
  assert flags["max_steps"] == "7" and flags["bf16"] == "False" and flags["fsdp"] == "full_shard auto_wrap"
  assert env["TORCHPRIME_OUTPUT_DIR"] == str(tmp_path)
  with pytest.raises(ValueError, match="train_script.path"):
    build_command(compose("default", []))
