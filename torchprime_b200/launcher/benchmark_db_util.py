"""Summary row of a finished run for a benchmark database.

The reference uploads a ``WorkloadBenchmarkV2Schema`` row to BigQuery
(launcher/benchmark_db_util.py:1-120, upload_metrics_to_bq.py).  There is no network here, so the
row — same information: model id, hardware, batch, sequence, step time, MFU, tokens/s, config —
is appended to a local JSON-lines file that any uploader can ship later."""

from __future__ import annotations

import datetime
import json
import os
import uuid


def collect_metrics(output_dir: str) -> tuple[dict, dict]:
  with open(os.path.join(output_dir, "train_metrics.json")) as f:
    metrics = json.load(f)
  with open(os.path.join(output_dir, "train_config.json")) as f:
    config = json.load(f)
  return metrics, config


def build_row(output_dir: str, env=None) -> dict:
  env = env if env is not None else os.environ
  metrics, config = collect_metrics(output_dir)
  mesh = config.get("ici_mesh", {})
  n = 1
  for v in mesh.values():
    n *= int(v)
  return {
    "run_id": f"{env.get('TORCHPRIME_JOBSET_NAME', 'local')}-{uuid.uuid4().hex[:8]}",
    "model_id": config.get("model", {}).get("model_id"),
    "software_id": "torchprime_b200", "hardware_id": env.get("TORCHPRIME_ACCELERATOR_TYPE", f"b200-{n}"),
    "hardware_num_chips": n, "hardware_num_slices": 1, "user": env.get("TORCHPRIME_USER", ""),
    "comments": env.get("TORCHPRIME_COMMENTS", ""),
    "global_batch_size": config.get("task", {}).get("global_batch_size"),
    "max_seq_length": config.get("dataset", {}).get("block_size"),
    "metrics_step_time": metrics.get("step_execution_time"), "metrics_mfu": metrics.get("mfu"),
    "metrics_tokens_per_second": metrics.get("tokens_per_second"), "num_steps": metrics.get("num_steps"),
    "train_runtime": metrics.get("train_runtime"), "update_timestamp": datetime.datetime.now().isoformat(),
    "configs_framework": json.dumps(config),
  }


def append_row(output_dir: str, db_path: str) -> dict:
  row = build_row(output_dir)
  os.makedirs(os.path.dirname(os.path.abspath(db_path)), exist_ok=True)
  with open(db_path, "a") as f:
    f.write(json.dumps(row) + "\n")
  return row
