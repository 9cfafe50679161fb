"""Small tools that had no test of their own: FLOPs accounting, run_model, doctor, pure-module marking and
the argument parsers of the experimental scripts (reference: torchprime/metrics/train_flops.py,
launcher/run_model.py, launcher/doctor.py, model_rewriting/assume_pure.py, experimental/*)."""

import pytest
import torch
import torch.nn as nn

from torchprime_b200.config import compose
from torchprime_b200.metrics.train_flops import StepShape, shape_from_model_config, train_step_tflops


def _model_cfg(name):
  cfg = compose("default", [f"model={name}", "dataset=synthetic"])
  return {k: cfg.model[k] for k in cfg.model.keys()}


def test_dense_llama_flops_match_the_closed_form():
  """Llama-3-8B, one sequence of 8192: 6 x (parameters without the embedding) x tokens for the weights and
  half of the dense S^2 work for causal attention."""
  s = shape_from_model_config(_model_cfg("llama-3-8b"), batch_size=1, seq_len=8192)
  total, weights, attn = train_step_tflops(s)
  h, f, L, v, kv = 4096, 14336, 32, 128256, 1024
  params = L * (h * h * 2 + 2 * h * kv + 3 * h * f) + h * v          # projections, FFN, head
  assert weights == pytest.approx(6.0 * params * 8192 / 1e12, rel=1e-6)
  assert attn == pytest.approx(3.0 * L * 2.0 * 8192 * 8192 * h / 1e12, rel=1e-6)
  assert total == pytest.approx(weights + attn)
  assert 415 < total < 430       # the figure bench.py reports as model TFLOPs per step


def test_moe_flops_count_only_the_routed_experts():
  cfg = _model_cfg("mixtral-8x7b")
  s = shape_from_model_config(cfg, batch_size=2, seq_len=4096)
  assert (s.experts, s.top_k) == (8, 2)
  total, weights, attn = train_step_tflops(s)
  dense_like = shape_from_model_config({**cfg, "num_local_experts": 1, "model_id": "x"}, 2, 4096)
  _, w_dense, _ = train_step_tflops(dense_like)
  # two of eight experts per token (plus the router): about twice the FFN work of a one-expert model
  assert 1.5 * w_dense < weights < 2.1 * w_dense
  s2 = StepShape(**{**s.__dict__, "grad_accum": 4})
  assert train_step_tflops(s2)[0] == pytest.approx(4 * total)


def test_deepseek_flops_use_mla_and_dense_first_layers():
  s = shape_from_model_config(_model_cfg("deepseek-v2-lite"), batch_size=1, seq_len=4096)
  assert s.mla["kv_lora_rank"] > 0 and s.dense_layers >= 1 and s.shared_experts >= 1
  total, weights, attn = train_step_tflops(s)
  assert total > 0 and attn > 0 and weights > attn


def test_run_model_times_forward_passes_on_cpu(capsys):
  from torchprime_b200.launcher import run_model
  times = run_model.main(["--model", "resnet18", "--batch-size", "2", "--runs", "2"])
  assert len(times) == 2 and all(t > 0 for t in times)
  assert "run 1:" in capsys.readouterr().out
  with pytest.raises(SystemExit):
    run_model.main(["--model", "not-a-model"])


def test_doctor_reports_and_needs_compiler_and_library(capsys, monkeypatch):
  from torchprime_b200.launcher import doctor
  rc = doctor.run_checks()
  out = capsys.readouterr().out
  assert "torchprime_b200 doctor" in out and "nvcc" in out and "torch.distributed backends" in out
  assert rc in (0, 1)
  # a missing library fails the run whatever the GPUs say
  from torchprime_b200.ops import _lib
  monkeypatch.setattr(_lib, "available", lambda: False)
  assert doctor.run_checks() == 1
  assert "[FAIL] kernel library missing" in capsys.readouterr().out


def test_pure_modules_get_a_trace_scope_and_unknown_names_are_rejected():
  from torchprime_b200.rewriting.assume_pure import mark_pure_modules

  class Block(nn.Module):
    def __init__(self):
      super().__init__()
      self.lin = nn.Linear(4, 4)

    def forward(self, x):
      return self.lin(x)

  model = nn.Sequential(Block(), Block())
  x = torch.randn(2, 4)
  want = model(x)
  cfg = compose("default", ["dataset=synthetic", "+model.pure_modules=[Block]"])
  mark_pure_modules(model, cfg)
  assert all(getattr(b, "_pure_marked", False) for b in model)
  assert torch.equal(model(x), want)
  from torchprime_b200.utils import profiling
  profiling.set_tracing(True)           # scopes are only recorded while a capture is running
  try:
    with torch.profiler.profile() as prof:
      model(x)
  finally:
    profiling.set_tracing(False)
  assert any(e.key == "Block" for e in prof.key_averages())
  bad = compose("default", ["dataset=synthetic", "+model.pure_modules=[NoSuchClass]"])
  with pytest.raises(AssertionError, match="NoSuchClass"):
    mark_pure_modules(nn.Sequential(Block()), bad)


@pytest.mark.parametrize("module", ["torchprime_b200.experimental.hf_trainer_sft.run_sft_gsm8k",
                                    "torchprime_b200.experimental.vllm_deployment.deploy"])
def test_experimental_scripts_parse_their_arguments(module, capsys):
  """The scripts need weights and network access to run; their command lines are checked here."""
  import importlib
  mod = importlib.import_module(module)
  with pytest.raises(SystemExit) as e:
    mod.main(["--help"])
  assert e.value.code == 0
  assert "--model" in capsys.readouterr().out
  with pytest.raises(SystemExit) as e:
    mod.main([])                      # the required argument is missing
  assert e.value.code == 2


def test_setup_sharding_and_mesh_names_the_batch_and_sequence_axes():
  """Reference: model_rewriting/sharding_initialization.py:22-69 (input sharding spec and minibatch)."""
  from torchprime_b200.dist.mesh import get_mesh
  from torchprime_b200.models.model_utils import initialize_model_class
  from torchprime_b200.rewriting.sharding_initialization import setup_sharding_and_mesh
  base = ["model=llama-3-8b", "model.num_hidden_layers=1", "model.hidden_size=64", "model.intermediate_size=128",
          "model.num_attention_heads=4", "model.num_key_value_heads=2", "model.vocab_size=128", "dataset=synthetic"]
  cfg = compose("default", base + ["ici_mesh.fsdp=4"])
  model = initialize_model_class(cfg.model, device="meta")
  s = setup_sharding_and_mesh(model, cfg, mesh=get_mesh(cfg, rank=1, world_size=4))
  assert s.batch_axes == ("data", "fsdp") and s.seq_axis is None and s.minibatch
  assert s.input_sharding_spec == (("data", "fsdp"), None)
  assert s.plan is not None and s.mesh.size("fsdp") == 4
  # context parallelism names the sequence axis; two axes > 1 is no longer a 1-D sharding
  cfg = compose("default", base + ["ici_mesh.fsdp=2", "ici_mesh.context=2", "model/sharding=llama-fsdp-tp-cp"])
  s = setup_sharding_and_mesh(model, cfg, mesh=get_mesh(cfg, rank=0, world_size=4))
  assert s.seq_axis == "context" and not s.minibatch
  # an orthogonal expert axis also splits the batch; a folded one does not
  moe = ["model=mixtral-8x7b", "model.num_hidden_layers=1", "model.hidden_size=64", "model.intermediate_size=128",
         "model.num_attention_heads=4", "model.num_key_value_heads=2", "model.vocab_size=128", "dataset=synthetic",
         "model.num_local_experts=4"]
  cfg = compose("default", moe + ["ici_mesh.fsdp=2", "ici_mesh.expert=2", "expert_axis_mode=orthogonal",
                                  "model/sharding=mixtral-fsdp-ep"])
  mm = initialize_model_class(cfg.model, device="meta")
  assert setup_sharding_and_mesh(mm, cfg, mesh=get_mesh(cfg, rank=0, world_size=4)).batch_axes == ("data", "fsdp", "expert")
  cfg = compose("default", moe + ["ici_mesh.fsdp=2", "ici_mesh.expert=2", "expert_axis_mode=folded",
                                  "model/sharding=mixtral-fsdp-ep"])
  assert setup_sharding_and_mesh(mm, cfg, mesh=get_mesh(cfg, rank=0, world_size=2)).batch_axes == ("data", "fsdp")
