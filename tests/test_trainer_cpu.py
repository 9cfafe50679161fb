"""Trainer behaviour on CPU: optimizer factory, loop length, clipping values, profiler window,
SFT hooks, export / reload round trip, NaN detection, engine recomputation and offload plumbing."""

import json
import math
import os

import pytest
import torch
import torch.nn as nn

from torchprime_b200.config import compose
from torchprime_b200.data.synthetic import make_synthetic_dataset
from torchprime_b200.metrics.metrics import MetricsLogger
from torchprime_b200.models.model_utils import initialize_model_class
from torchprime_b200.parallel.fsdp import FSDPEngine
from torchprime_b200.parallel.optimizer import LRScheduler, ShardedAdafactor, ShardedAdamW, lr_lambda
from torchprime_b200.trainer import SFTTrainer, Trainer, TRAINERS

BASE = ["model=llama-tiny", "dataset=synthetic", "dataset.block_size=32", "task.global_batch_size=2",
        "ici_mesh.fsdp=1", "profile_start_step=-1", "+engine.cpu_dtype=float32", "logging_steps=1"]


def make_trainer(tmp_path, extra=(), cls=Trainer):
  cfg = compose("default", BASE + [f"output_dir={tmp_path}/out", f"profile_dir={tmp_path}/prof"] + list(extra))
  torch.manual_seed(0)
  model = initialize_model_class(cfg.model, device="meta")
  data = make_synthetic_dataset(vocab_size=cfg.model.vocab_size, block_size=32, num_samples=32)
  return cls(model=model, config=cfg, train_dataset=data), cfg


def test_registry():
  assert TRAINERS["train"] is Trainer and TRAINERS["sft"] is SFTTrainer


def test_optimizer_factory(tmp_path):
  tr, _ = make_trainer(tmp_path, ["task.optimizer.type=adamw", "+task.optimizer.weight_decay=0.1"])
  assert isinstance(tr.optimizer, ShardedAdamW) and tr.optimizer.weight_decay == 0.1
  tr, _ = make_trainer(tmp_path, ["task.optimizer.type=adafactor"])
  assert isinstance(tr.optimizer, ShardedAdafactor)
  with pytest.raises(ValueError, match="does not support weight decay"):
    make_trainer(tmp_path, ["task.optimizer.type=adafactor", "+task.optimizer.weight_decay=0.1"])
  with pytest.raises(ValueError, match="Unsupported optimizer type"):
    make_trainer(tmp_path, ["task.optimizer.type=sgd"])
  # plain-parameter path (no engine): torch / transformers optimizers
  cfg = compose("default", ["task.optimizer.type=adamw"])
  lin = nn.Linear(2, 2)
  assert isinstance(Trainer._create_optimizer(cfg, lin.parameters()), torch.optim.AdamW)


def test_lr_schedules():
  assert lr_lambda("linear", 0, 0, 10) == 1.0 and lr_lambda("linear", 5, 0, 10) == 0.5
  assert lr_lambda("linear", 1, 2, 10) == 0.5 and lr_lambda("cosine", 10, 0, 10) == pytest.approx(0.0)
  assert lr_lambda("constant_with_warmup", 7, 2, 10) == 1.0
  with pytest.raises(ValueError):
    LRScheduler(1.0, "nope")
  s = LRScheduler(2.0, "linear", 0, 4)
  s.step()
  assert s.get_last_lr() == [1.5]


def test_train_loop_runs_exactly_max_steps_and_logs(tmp_path, caplog):
  tr, cfg = make_trainer(tmp_path, ["task.max_steps=6", "task.optimizer.type=adamw"])
  calls = []
  orig = tr.train_step
  tr.train_step = lambda batch: (calls.append(1), orig(batch))[1]
  import logging
  with caplog.at_level(logging.INFO):
    tr.train_loop()
  assert len(calls) == 6
  text = caplog.text
  assert "Finished training run" in text and "Max step: 6" in text and "Global batch size: 2" in text
  assert "Epoch: 0.0000, step: 0, loss:" in text and "grad_norm:" in text and "trace time:" in text
  ml = MetricsLogger()
  tr.finalize_training(ml)
  m = json.load(open(tmp_path / "out" / "train_metrics.json"))
  assert m["num_steps"] == 6 and m["step_execution_time"] > 0
  assert json.load(open(tmp_path / "out" / "train_config.json"))["task"]["max_steps"] == 6


class _Lin(nn.Module):
  """y = w . x with w = 1: loss = sum(y) gives d loss / d w = x."""

  def __init__(self):
    super().__init__()
    self.fc = nn.Linear(4, 1, bias=False)

  def forward(self, x):
    return self.fc(x).sum()


def _engine_with_grads(grads):
  torch.manual_seed(0)
  m = _Lin()
  eng = FSDPEngine(m, None, None, device="cpu", param_dtype=torch.float32)
  eng.flat_grad[:4] = torch.tensor(grads)
  return eng


def test_clip_by_norm_and_value_exact():
  cfg = compose("default", ["task.optimizer.type=adamw", "task.max_grad_norm=1.0"])
  eng = _engine_with_grads([1.0, 1.0, 1.0, 1.0])
  opt = ShardedAdamW(eng, lr=0.0)
  norm = opt.clip_gradients(1.0, None)
  assert norm.item() == pytest.approx(2.0)
  assert (eng.flat_grad[:4] * opt._coef).tolist() == pytest.approx([0.5] * 4, rel=1e-5)
  norm = opt.clip_gradients(None, None)          # only measured
  assert norm.item() == pytest.approx(2.0) and opt._coef.item() == 1.0
  eng = _engine_with_grads([3.0, -3.0, 0.1, 0.0])
  opt = ShardedAdamW(eng, lr=0.0)
  opt.clip_gradients(None, 0.5)
  assert eng.flat_grad[:4].tolist() == pytest.approx([0.5, -0.5, 0.1, 0.0])


def test_profiler_window_started_and_stopped_once(tmp_path, monkeypatch):
  tr, cfg = make_trainer(tmp_path, ["task.max_steps=10", "profile_start_step=2", "profile_end_step=4"])
  events = []
  monkeypatch.setattr(tr, "_start_profile", lambda: events.append("start"))
  monkeypatch.setattr(tr, "_stop_profile", lambda: events.append("stop"))
  tr.train_loop()
  assert events.count("start") == 1 and events[:2] == ["start", "stop"]


def test_nan_loss_raises(tmp_path):
  tr, _ = make_trainer(tmp_path, ["task.max_steps=3"])
  tr.train_step = lambda batch: (torch.tensor(float("nan")), torch.tensor(1.0))
  with pytest.raises(ValueError, match="Loss is NaN at step 0"):
    tr.train_loop()


def test_units_are_recomputed_in_backward(tmp_path):
  tr, _ = make_trainer(tmp_path, ["task.max_steps=1"])
  layer = tr.engine.units[1]
  assert layer.remat and type(layer.module).__name__ == "LlamaDecoderLayer"
  n = {"calls": 0}
  orig = layer.orig_forward
  def counting(*a, **k):
    n["calls"] += 1
    return orig(*a, **k)
  layer.orig_forward = counting
  loader = tr._get_train_dataloader()
  tr.train_step(tr._prepare_batch(loader.next_batch()))
  assert n["calls"] == 2   # forward under no_grad + recomputation inside backward


def test_remat_config_validation():
  from torchprime_b200.rewriting.rematerialization_utils import add_activation_checkpointing_and_scan, get_classes_by_names
  cfg = compose("default", ["model=llama-tiny", "model/remat=llama-scan-offload"])
  m = initialize_model_class(cfg.model, device="meta")
  plan = add_activation_checkpointing_and_scan(m, cfg)
  assert plan.remat_classes == ("LlamaDecoderLayer",) and plan.scan_path == "model.layers"
  assert plan.offload_tensors == ("decoder_input",)
  bad = compose("default", ["model=llama-tiny", "model.remat.offload_tensors=[decoder_input]"])
  with pytest.raises(AssertionError, match="requires scan_layers"):
    add_activation_checkpointing_and_scan(m, bad)
  worse = compose("default", ["model=llama-tiny", "model/remat=llama-scan-offload", "model.remat.offload_tensors=[foo]"])
  with pytest.raises(ValueError, match="unknown tensors"):
    add_activation_checkpointing_and_scan(m, worse)
  with pytest.raises(AssertionError, match="can't be found"):
    get_classes_by_names(m, ["NoSuchLayer"])


def test_auto_trace_and_pure_modules(tmp_path):
  from torchprime_b200.rewriting.auto_trace import auto_trace
  from torchprime_b200.utils import profiling
  seen = []
  class M(nn.Module):
    def __init__(self):
      super().__init__()
      self.a = nn.Linear(2, 2)
      self.b = nn.Sequential(nn.Linear(2, 2), nn.ReLU())
    def forward(self, x):
      return self.b(self.a(x))
  m = auto_trace(M())
  import contextlib
  real = profiling.trace_scope
  @contextlib.contextmanager
  def fake(name):
    seen.append(name)
    yield
  import torchprime_b200.rewriting.auto_trace as at
  at.trace_scope = fake
  try:
    x = torch.ones(1, 2)
    ref_out = M.forward(m, x)
    assert seen == ["a", "0"]
  finally:
    at.trace_scope = real
  tr, _ = make_trainer(tmp_path, ["model.pure_modules=[LlamaMLP]"])
  assert all(getattr(mod, "_pure_marked", False) for mod in tr.model.modules() if type(mod).__name__ == "LlamaMLP")
  with pytest.raises(AssertionError, match="can't be found"):
    make_trainer(tmp_path, ["model.pure_modules=[Nope]"])


def test_export_and_reload_round_trip(tmp_path):
  cfg = compose("default", ["model=llama-tiny"])
  torch.manual_seed(1)
  m = initialize_model_class(cfg.model)
  ids = torch.randint(0, 256, (1, 16))
  want, _ = m(ids)
  m.export(str(tmp_path / "exp"))
  files = os.listdir(tmp_path / "exp")
  assert "model.safetensors.index.json" in files and "config.json" in files and "layers_0.safetensors" in files
  torch.manual_seed(2)
  m2 = initialize_model_class(cfg.model)
  m2.from_pretrained(str(tmp_path / "exp"))
  got, _ = m2(ids)
  assert (got - want).abs().max() < 5e-3
  bad = compose("default", ["model=llama-tiny", "model.hidden_size=32", "model.num_attention_heads=2",
                            "model.num_key_value_heads=1"])
  with pytest.raises(RuntimeError, match="size mismatch"):
    initialize_model_class(bad.model).from_pretrained(str(tmp_path / "exp"))


def test_sft_trainer_loads_and_exports(tmp_path):
  cfg0 = compose("default", ["model=llama-tiny"])
  torch.manual_seed(3)
  src = initialize_model_class(cfg0.model)
  src.export(str(tmp_path / "pre"))
  tr, cfg = make_trainer(tmp_path, ["task=sft", "task.max_steps=2", "task.global_batch_size=2",
                                    f"model.pretrained_model={tmp_path}/pre", "model.tokenizer_name=null",
                                    "task.convert_to_safetensors=true"], cls=SFTTrainer)
  loaded = tr.engine.full_state_dict()
  for k, v in src.state_dict().items():
    assert torch.allclose(loaded[k], v, atol=1e-6), k
  tr.train_loop()
  exp = tmp_path / "out" / "export"
  assert (exp / "model.safetensors.index.json").exists() and not list(exp.glob("*.distcp"))
  m2 = initialize_model_class(cfg0.model)
  m2.from_pretrained(str(exp))
  after = tr.engine.full_state_dict()
  assert torch.allclose(m2.state_dict()["lm_head.weight"], after["lm_head.weight"], atol=1e-6)


def test_multicast_switch_and_abort_guard(tmp_path, monkeypatch):
  """engine.multicast=false turns every multicast binding off through the switches the fused kernels
  read; a watchdog that may end the process refuses to run with multicast bindings on several ranks."""
  import os
  from torchprime_b200.dist import runtime as rt
  for key in ("TPB_AG_MULTICAST", "TPB_TP_FUSED", "TPB_CP_MULTICAST"):
    monkeypatch.delenv(key, raising=False)
  tr, _ = make_trainer(tmp_path, ["engine.multicast=false"])
  assert not tr.multicast
  assert all(os.environ[k] == "0" for k in ("TPB_AG_MULTICAST", "TPB_TP_FUSED", "TPB_CP_MULTICAST"))
  with monkeypatch.context() as m:
    m.setattr(rt, "world_size", lambda: 2)
    with pytest.raises(ValueError, match="engine.multicast=false"):
      make_trainer(tmp_path, ["engine.watchdog_seconds=5", "engine.watchdog_abort=true"])
  tr, _ = make_trainer(tmp_path, ["engine.watchdog_seconds=5", "engine.watchdog_abort=true", "engine.multicast=false"])
  assert tr.watchdog.abort
  tr.watchdog.stop()


def test_device_timeout_is_raised_at_the_step_it_is_seen(tmp_path, monkeypatch):
  """A bounded device wait that gave up must stop the run at once (with the step number), not after the
  last step: consumers of that kernel read partial data."""
  from torchprime_b200.ops import _lib
  tr, _ = make_trainer(tmp_path, ["task.max_steps=6"])
  calls = {"n": 0}

  def fake_check(step, synchronize):
    calls["n"] += 1
    if step == 2:
      raise _lib.KernelError(f"at training step {step}: device-side bounded wait gave up")
  monkeypatch.setattr(tr, "_check_device_status", fake_check)
  with pytest.raises(_lib.KernelError, match="at training step 2"):
    tr.train_loop()
  assert calls["n"] >= 3
