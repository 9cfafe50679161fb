"""End-to-end run checkers (local-filesystem versions of the reference's e2e_testing/*.py, which
read the same artefacts from a GCS bucket):

  python e2e_testing/checks.py logs      <log file>                       "Finished training run" present
  python e2e_testing/checks.py loss      <log file> <expected> <tol>      last logged loss within tolerance
  python e2e_testing/checks.py profile   <profile dir>                    exactly one trace per rank 0
  python e2e_testing/checks.py step_time <output dir> <benchmark key>     step time inside the recorded bounds
  python e2e_testing/checks.py update    <bounds.yaml> <key> t1 t2 ...    recompute bounds from samples
"""

from __future__ import annotations

import glob
import json
import math
import os
import re
import statistics
import sys

import yaml

BOUNDS_FILE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "step_time_bounds.yaml")
LOSS_RE = re.compile(r"loss:\s*([0-9]*\.?[0-9]+(?:[eE][-+]?\d+)?)")


def check_logs(path: str) -> int:
  text = open(path, errors="replace").read()
  if "Finished training run" in text:
    print("Found 'Finished training run'")
    return 0
  print("Error: the log does not contain 'Finished training run'", file=sys.stderr)
  return 1


def last_loss(text: str) -> float | None:
  hits = LOSS_RE.findall(text)
  return float(hits[-1]) if hits else None


def check_loss(path: str, expected: float, tolerance: float) -> int:
  loss = last_loss(open(path, errors="replace").read())
  if loss is None:
    print("Error: no 'loss:' entry in the log", file=sys.stderr)
    return 1
  print(f"final loss {loss:.4f} (expected {expected:.4f} +- {tolerance})")
  return 0 if abs(loss - expected) <= tolerance else 1


def check_profile(profile_dir: str) -> int:
  files = glob.glob(os.path.join(profile_dir, "**", "trace_rank0.json"), recursive=True)
  if len(files) != 1:
    print(f"Error: expected exactly one rank-0 trace under {profile_dir}, found {len(files)}", file=sys.stderr)
    return 1
  print(f"Found profile {files[0]}")
  return 0


def check_step_time(output_dir: str, key: str, bounds_file: str = BOUNDS_FILE) -> int:
  files = glob.glob(os.path.join(output_dir, "**", "train_metrics.json"), recursive=True)
  if len(files) != 1:
    print(f"Error: expected one train_metrics.json under {output_dir}, found {len(files)}", file=sys.stderr)
    return 1
  t = json.load(open(files[0])).get("step_execution_time")
  if t is None:
    print("Error: step_execution_time is None in metrics.", file=sys.stderr)
    return 1
  b = yaml.safe_load(open(bounds_file))["benchmarks"][key]
  lo, hi = b["step_time_lower_bound"], b["step_time_upper_bound"]
  print(f"Step execution time: {t:.4f} s, bounds [{lo:.4f}, {hi:.4f}]")
  return 0 if lo <= t <= hi else 1


# Student-t 99% two-sided critical values for small samples (df -> t)
_T99 = {1: 63.657, 2: 9.925, 3: 5.841, 4: 4.604, 5: 4.032, 6: 3.707, 7: 3.499, 8: 3.355, 9: 3.250, 10: 3.169,
        15: 2.947, 20: 2.845, 30: 2.750, 60: 2.660}


def compute_bounds(samples: list[float], relax: float = 2.0, min_rel: float = 0.015) -> dict:
  """99% Student-t interval of the samples, at least 1.5% of the mean and at least the observed
  range, then widened by ``relax`` (the rule of the reference's update_step_time.py:231-259)."""
  n = len(samples)
  mean = statistics.fmean(samples)
  sd = statistics.stdev(samples) if n > 1 else 0.0
  df = max(1, n - 1)
  tcrit = next(v for k, v in sorted(_T99.items()) if k >= df) if df <= 60 else 2.576
  half = tcrit * sd * math.sqrt(1 + 1 / n) if n > 1 else 0.0
  half = max(half, min_rel * mean, max(mean - min(samples), max(samples) - mean)) * relax
  return {"step_time_lower_bound": mean - half, "step_time_upper_bound": mean + half, "confidence_interval": half,
          "average": mean, "sample_size": n}


def update_bounds(bounds_file: str, key: str, samples: list[float]) -> int:
  doc = yaml.safe_load(open(bounds_file)) if os.path.exists(bounds_file) else {"benchmarks": {}}
  entry = doc["benchmarks"].get(key, {"name": key})
  entry.update(compute_bounds(samples))
  doc["benchmarks"][key] = entry
  yaml.safe_dump(doc, open(bounds_file, "w"), sort_keys=False)
  print(f"updated {key}: {entry}")
  return 0


def main(argv):
  if len(argv) < 2:
    print(__doc__)
    return 2
  cmd, args = argv[0], argv[1:]
  if cmd == "logs":
    return check_logs(args[0])
  if cmd == "loss":
    return check_loss(args[0], float(args[1]), float(args[2]))
  if cmd == "profile":
    return check_profile(args[0])
  if cmd == "step_time":
    return check_step_time(args[0], args[1], *(args[2:3]))
  if cmd == "update":
    return update_bounds(args[0], args[1], [float(x) for x in args[2:]])
  print(__doc__)
  return 2


if __name__ == "__main__":
  sys.exit(main(sys.argv[1:]))
