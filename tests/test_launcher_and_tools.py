"""Launcher plumbing, e2e checkers, system check, benchmark row — all on CPU."""

import datetime
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "e2e_testing"))

from torchprime_b200.dist import launcher as L
from torchprime_b200.launcher import benchmark_db_util, cli


def test_jobset_name_and_workload_args():
  name = cli.generate_jobset_name("My Run!", datetime.datetime(2025, 1, 2, 3, 4, 5))
  assert name.endswith("-20250102-030405") and name == name.lower() and len(name) <= 40
  args = cli.workload_args(["model=llama-3-8b"], {"artifact_dir": "/art"}, "js")
  assert "profile_dir=/art/js/profile/0-0" in args and "output_dir=/art/js/outputs/0-0" in args
  assert cli.workload_args(["output_dir=x"], {}, "js").count("output_dir=x") == 1
  env = cli.workload_env({"gpus": 8, "artifact_dir": "/art"}, "js", "note")
  assert env["TORCHPRIME_ACCELERATOR_TYPE"] == "b200-8" and env["TORCHPRIME_JOBSET_NAME"] == "js"


def test_tp_run_dry_run(tmp_path, monkeypatch):
  monkeypatch.chdir(tmp_path)
  assert cli.main(["run", "--gpus", "2", "--dry-run", "-m", "torchprime_b200.train", "model=llama-tiny"]) == 0


def test_launcher_propagates_failure_and_stops_peers(tmp_path):
  script = tmp_path / "w.py"
  script.write_text("import os, sys, time\nr = int(os.environ['RANK'])\nassert os.environ['MASTER_ADDR'] == '127.0.0.1'\n"
                    "if r == 1:\n  sys.exit(7)\ntime.sleep(60)\n")
  import time
  t0 = time.time()
  rc = L.launch([sys.executable, str(script)], nproc=3, grace_s=2.0)
  assert rc == 7 and time.time() - t0 < 30
  ok = tmp_path / "ok.py"
  ok.write_text("import os\nassert int(os.environ['WORLD_SIZE']) == 2\n")
  assert L.launch([sys.executable, str(ok)], nproc=2) == 0


def test_e2e_checkers(tmp_path):
  import checks
  log = tmp_path / "log.txt"
  log.write_text("Epoch: 0.0, step: 0, loss: 1.2352, grad_norm: 1.0\nEpoch: 0.1, step: 9, loss: 0.4826, grad_norm: 0.5\n"
                 "Finished training run\n")
  assert checks.check_logs(str(log)) == 0
  assert checks.check_loss(str(log), 0.4826, 0.001) == 0 and checks.check_loss(str(log), 0.6, 0.001) == 1
  (tmp_path / "p" / "a").mkdir(parents=True)
  assert checks.check_profile(str(tmp_path / "p")) == 1
  (tmp_path / "p" / "a" / "trace_rank0.json").write_text("{}")
  assert checks.check_profile(str(tmp_path / "p")) == 0
  out = tmp_path / "out"
  out.mkdir()
  (out / "train_metrics.json").write_text(json.dumps({"step_execution_time": 1.0}))
  bounds = tmp_path / "b.yaml"
  assert checks.update_bounds(str(bounds), "k", [0.95, 1.0, 1.05, 1.02]) == 0
  assert checks.check_step_time(str(out), "k", str(bounds)) == 0
  (out / "train_metrics.json").write_text(json.dumps({"step_execution_time": 9.0}))
  assert checks.check_step_time(str(out), "k", str(bounds)) == 1
  b = checks.compute_bounds([1.0, 1.0, 1.0])
  assert b["confidence_interval"] == pytest.approx(0.03)


def test_system_check_and_benchmark_row(tmp_path):
  from torchprime_b200.tools import system_check
  assert system_check.main([f"output_dir={tmp_path}", "--foo"]) == 0
  assert any(f.startswith("log-") for f in os.listdir(tmp_path))
  (tmp_path / "train_metrics.json").write_text(json.dumps({"step_execution_time": 0.5, "mfu": 0.3, "tokens_per_second": 10.0,
                                                           "num_steps": 3, "train_runtime": 9.0}))
  (tmp_path / "train_config.json").write_text(json.dumps({"model": {"model_id": "m"}, "ici_mesh": {"fsdp": 8, "data": 1},
                                                          "task": {"global_batch_size": 8}, "dataset": {"block_size": 128}}))
  row = benchmark_db_util.append_row(str(tmp_path), str(tmp_path / "db.jsonl"))
  assert row["hardware_num_chips"] == 8 and row["metrics_mfu"] == 0.3 and os.path.exists(tmp_path / "db.jsonl")


def test_aux_scripts_parse_arguments(tmp_path):
  """The asset snapshot tool and the comparison scripts are importable and explain themselves."""
  import importlib
  import pytest
  mod = importlib.import_module("torchprime_b200.launcher.save_hf_assets")
  with pytest.raises(SystemExit):
    mod.main(["--dest", str(tmp_path)])          # neither a repo nor a dataset given
  draw = importlib.import_module("torchprime_b200.experimental.hf_trainer_sft.draw_figure")
  log = tmp_path / "train.log"
  log.write_text("step 1 loss: 1.25\nstep 2 loss: 0.75 lr: 1e-4\n")
  assert draw.losses_from_log(str(log)) == [1.25, 0.75]


def test_interactive_mode_reruns_on_file_change(tmp_path):
  """``tp run -i``: a change to a watched source file stops the running workload and starts it again;
  ignored paths (.gitignore) and other file types do not."""
  from torchprime_b200.launcher import cli
  (tmp_path / ".gitignore").write_text("outputs/\n*.log\n")
  (tmp_path / "train.py").write_text("x = 1\n")
  (tmp_path / "outputs").mkdir()
  (tmp_path / "outputs" / "gen.py").write_text("ignored\n")
  w = cli.FileChangeWatcher(str(tmp_path))
  assert w.changed() == []
  (tmp_path / "outputs" / "gen.py").write_text("still ignored\n")
  (tmp_path / "notes.txt").write_text("not a source file\n")
  assert w.changed() == []
  os.utime(tmp_path / "train.py", ns=(1, 1))
  (tmp_path / "cfg.yaml").write_text("a: 1\n")
  assert w.changed() == ["cfg.yaml", "train.py"]

  class FakeProc:
    def __init__(self):
      self.returncode, self.stopped, self.pid = None, False, None
    def poll(self):
      return self.returncode
    def terminate(self):
      self.stopped, self.returncode = True, -15
    def wait(self, timeout=None):
      return self.returncode
    def kill(self):
      self.returncode = -9
  procs, ticks = [], [0]

  def start():
    procs.append(FakeProc())
    return procs[-1]

  def fake_sleep(_s):
    ticks[0] += 1
    if ticks[0] == 2:
      (tmp_path / "train.py").write_text("x = 2\n")     # edit while the first run is still going
    if ticks[0] == 4:
      procs[-1].returncode = 0                           # the second run finishes
  rc = cli.run_interactive(start, w, poll_s=0.0, max_runs=2, sleep=fake_sleep)
  assert rc == 0 and len(procs) == 2 and procs[0].stopped and not procs[1].stopped


def test_save_hf_verbs_call_the_asset_tool(tmp_path, monkeypatch):
  from torchprime_b200.launcher import cli, save_hf_assets
  calls = []
  monkeypatch.setattr(save_hf_assets, "save_repo", lambda repo, dest, types, token=None: calls.append(("repo", repo, dest, tuple(types))) or dest)
  monkeypatch.setattr(save_hf_assets, "save_dataset", lambda name, cfg, dest, split, tok, bs: calls.append(("ds", name, cfg, split, tok, bs)) or dest)
  assert cli.main(["save-hf-model-files", "--repo-id", "org/model", "--dest", str(tmp_path), "--file-type", "tokenizer"]) == 0
  assert cli.main(["save-hf-dataset", "--dataset-name", "wikitext", "--dataset-config", "wikitext-2-raw-v1",
                   "--dest", str(tmp_path), "--tokenizer", "org/model", "--block-size", "128"]) == 0
  assert calls == [("repo", "org/model", str(tmp_path), ("tokenizer",)),
                   ("ds", "wikitext", "wikitext-2-raw-v1", "train", "org/model", 128)]
