"""Config composer, validator, profiling window, retry, metrics records, MFU goldens."""

import json
import math
from datetime import timedelta

import numpy as np
import pytest
import torch

from torchprime_b200.config import compose, parse_cli, to_container
from torchprime_b200.metrics.metrics import Metrics, MetricsLogger
from torchprime_b200.metrics.mfu import compute_mfu, get_num_chips_and_tflops_per_chip
from torchprime_b200.metrics.step_timer import StepTimer
from torchprime_b200.utils.config_utils import config_validator
from torchprime_b200.utils.profiling import ensure_profile_end_step
from torchprime_b200.utils.retry import retry


def test_default_composition_and_overrides():
  c = compose("default", ["model=llama-3.1-70b", "model/remat=llama-scan-offload", "task.max_steps=3",
                          "ici_mesh.fsdp=8", "+foo.bar=[a,b]", "task.max_grad_value=null"])
  assert c.model.model_id == "llama-3.1-70b"
  assert c.model.remat.scan_layers == "model.layers"
  assert c.model.remat.offload_tensors == ["decoder_input"]
  assert c.model.remat.activation_checkpoint_layers == ["LlamaDecoderLayer"]
  assert c.task.max_steps == 3 and c.ici_mesh.fsdp == 8 and c.foo.bar == ["a", "b"]
  assert c.task.max_grad_value is None
  assert "model.layers.*.self_attn.q_proj.weight" in c.model.sharding
  assert c.model.sharding["model.layers.*"] == [["data", "fsdp"], None, "tensor"]


def test_config_name_and_override_keyword():
  name, ov = parse_cli(["--config-name", "llama-3-8b-sft-w-gsm8k", "task.max_steps=7"])
  c = compose(name, ov)
  assert c.task.name == "sft" and c.dataset.hf_dataset_name == "gsm8k" and c.task.max_steps == 7
  assert c.model.pretrained_model == "meta-llama/Meta-Llama-3-8B"
  assert c.task.convert_to_safetensors is False


def test_unknown_key_needs_plus():
  with pytest.raises(KeyError):
    compose("default", ["task.not_a_key=1"])
  assert compose("default", ["+task.not_a_key=1"]).task.not_a_key == 1


def test_every_model_config_composes():
  import glob, os
  from torchprime_b200.config import CONFIG_ROOT
  for f in glob.glob(os.path.join(CONFIG_ROOT, "model", "*.yaml")):
    c = compose("default", ["model=" + os.path.basename(f)[:-5]])
    assert c.model.model_class and c.model.hidden_size > 0


def test_validator_messages():
  c = compose("default", ["task.global_batch_size=2", "ici_mesh.fsdp=4"])
  with pytest.raises(AssertionError, match="Global_batch_size"):
    config_validator(c)
  c = compose("default", ["+model.load_balance_cp=true"])
  with pytest.raises(RuntimeError, match="only be used when cp is enabled"):
    config_validator(c)
  c = compose("default", ["model=llama-3-8b-cp", "model.load_balance_cp=true", "ici_mesh.context=2",
                          "model.attention_kernel=flash_attention", "ici_mesh.fsdp=2"])
  with pytest.raises(RuntimeError, match="splash attention"):
    config_validator(c)
  c = compose("default", ["ici_mesh.context=2", "ici_mesh.fsdp=2"])
  with pytest.raises(RuntimeError, match="config.model as well"):
    config_validator(c)
  c = compose("default", ["model=llama-3-8b-cp", "ici_mesh.context=4", "ici_mesh.fsdp=1"])
  with pytest.raises(RuntimeError, match="should equal"):
    config_validator(c)
  c = compose("default", ["dcn_mesh.fsdp=2", "task.global_batch_size=8"])
  with pytest.raises(RuntimeError, match="dcn_mesh"):
    config_validator(c)
  config_validator(compose("default", ["model=llama-3-8b-cp", "ici_mesh.context=2", "ici_mesh.fsdp=2"]))


@pytest.mark.parametrize("start,end,max_steps,want", [
  (-1, None, 20, (-1, -1)), (3, None, 15, (3, 10)), (3, None, 100, (3, 23)), (3, 6, 100, (3, 6)),
  (14, None, 15, (-1, -1)), (8, None, 12, (8, 9)), (3, 50, 20, (3, 15)),
])
def test_profile_window(start, end, max_steps, want):
  c = compose("default", [f"profile_start_step={start}", f"task.max_steps={max_steps}"] +
              ([f"profile_end_step={end}"] if end is not None else []))
  ensure_profile_end_step(c)
  assert (c.profile_start_step, c.profile_end_step) == want


def test_retry():
  calls = []
  def flaky():
    calls.append(1)
    if len(calls) < 3:
      raise OSError("boom")
    return 7
  assert retry(flaky, retry_count=3, retry_delay=0.001) == 7
  with pytest.raises(OSError):
    retry(lambda: (_ for _ in ()).throw(OSError("x")), retry_count=2, retry_delay=0.001)


def test_metrics_roundtrip(tmp_path):
  m = Metrics(train_runtime=timedelta(seconds=12.5), step_execution_time=timedelta(seconds=0.25), mfu=0.4,
              tokens_per_second=1000.0, num_steps=5)
  p = tmp_path / "m.json"
  m.save(p)
  raw = json.loads(p.read_text())
  assert raw["train_runtime"] == 12.5 and raw["step_execution_time"] == 0.25
  assert Metrics.load(p) == m
  assert "mfu" in str(m)
  lg = MetricsLogger()
  lg.log_step_execution_time(0.5); lg.log_mfu(0.3); lg.log_tokens_per_second(10.0); lg.log_num_steps(4)
  out = lg.finalize()
  assert out.step_execution_time == timedelta(seconds=0.5) and out.num_steps == 4
  assert MetricsLogger().finalize().step_execution_time is None


GOLDEN = [("llama-3-8b", 1024, 4096, 2.801027417, "foobar-v5p-512", 0.6148650326),
          ("llama-3.1-70b", 128, 8192, 16.992, "abc-v6e-128-stuff", 0.2359197522),
          ("mixtral-8x7b", 1024, 4096, 5.04, "v6e-256", 0.2822763546),
          ("deepseek-v3", 512, 4096, 10.0, "v5p-256", 0.8939805997)]


@pytest.mark.parametrize("model,b,s,t,chip,want", GOLDEN)
def test_mfu_golden_values(model, b, s, t, chip, want):
  cfg = to_container(compose("default", ["model=" + model]).model)
  assert compute_mfu(cfg, b, s, t, chip).mfu == pytest.approx(want, rel=0.01, abs=0.005)


def test_accelerator_table():
  assert get_num_chips_and_tflops_per_chip("v4-8") == (4, 275)
  assert get_num_chips_and_tflops_per_chip("b200-8") == (8, 2250)
  with pytest.raises(ValueError):
    get_num_chips_and_tflops_per_chip("q9-1")
  cfg = to_container(compose("default", ["model=llama-3-8b"]).model)
  r = compute_mfu(cfg, 8, 8192, 1.0, "b200-8")
  assert r.model_tflops == pytest.approx(3373.16, rel=1e-3)


def test_step_timer_summary():
  assert StepTimer.summarize([]) is None
  assert StepTimer.summarize([1.0, 3.0]) == 2.0
  assert StepTimer.summarize([1.0, 9.0, 2.0]) == 2.0
  t = StepTimer(use_cuda=False)
  for i in range(4):
    t.mark(i)
  assert len(t.deltas()) == 3 and len(t.deltas(first_step=1)) == 2
