"""Model FLOPs Utilization.

``compute_mfu`` keeps the reference's signature (torchprime/metrics/mfu.py:37-146):
the accelerator is named by a string such as ``v6e-256`` (TPU table kept so published
numbers and the reference's golden values can be reproduced) or ``b200-8`` /
``b200`` for this framework's hardware.  For B200 the denominator is the dense bf16
spec peak (2250 TFLOP/s per GPU); the fraction of the locally measured cuBLAS rate is
available through :func:`measured_peak_tflops`.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import sys
from dataclasses import dataclass
from pathlib import Path

from .train_flops import shape_from_model_config, train_step_tflops

# Peak dense bf16 TFLOP/s per chip.
PEAK_TFLOPS = {"v4": 275, "v5p": 459, "v5e": 197, "v6e": 918, "b200": 2250, "h100": 989}
# TPU v4 / v5p names count TensorCores (two per chip).
_CORES_PER_CHIP = {"v4": 2, "v5p": 2}


@dataclass
class MFU:
  model_tflops: float
  """TFLOPs the model needs for one step."""
  hardware_tflops_per_step: float
  """TFLOPs the hardware could have delivered during one step."""
  per_chip_tflops_per_sec: float
  mfu: float


def parse_accelerator_name(name: str) -> tuple[str, int]:
  m = re.search(r"(v\d+[ep]?|b200|h100)(?:-(\d+))?", name.lower())
  if not m:
    raise ValueError(f"No matching pattern found in {name}")
  kind = m.group(1)
  count = int(m.group(2)) if m.group(2) else 1
  return kind, count


def get_num_chips_and_tflops_per_chip(name: str) -> tuple[float, int]:
  kind, count = parse_accelerator_name(name)
  if kind not in PEAK_TFLOPS:
    raise ValueError(f"Unsupported accelerator type {name}")
  return count / _CORES_PER_CHIP.get(kind, 1), PEAK_TFLOPS[kind]


def measured_peak_tflops(path: str | None = None) -> dict | None:
  """cuBLAS bf16 rate and copy bandwidth measured on this pool's B200s, if recorded."""
  path = path or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                              "MEASURED_PEAKS.json")
  try:
    return json.loads(Path(path).read_text())
  except (OSError, ValueError):
    return None


def compute_mfu(config: dict, batch_size: int, sequence_length: int, step_duration: float, tpu_name: str,
                num_slices: int = 1, gradient_accumulation_steps: int = 1, torch_dtype: str = "bfloat16") -> MFU:
  """MFU of a training config.  ``batch_size`` is the *global* batch, ``tpu_name`` the
  accelerator string (``v5p-128``, ``b200-8``)."""
  shape = shape_from_model_config(config, batch_size, int(sequence_length), gradient_accumulation_steps)
  total, _, _ = train_step_tflops(shape)
  assert torch_dtype == "bfloat16", f"Unsupported dtype {torch_dtype}"
  chips, peak = get_num_chips_and_tflops_per_chip(tpu_name)
  chips *= num_slices
  hw = step_duration * chips * peak
  return MFU(model_tflops=total, hardware_tflops_per_step=hw, per_chip_tflops_per_sec=total / step_duration / chips,
             mfu=total / hw)


def main(argv=None):
  ap = argparse.ArgumentParser(description="Compute MFU from a HuggingFace-style model config.")
  ap.add_argument("--config", required=True, help="JSON or YAML model config")
  ap.add_argument("--batch-size", type=int, required=True)
  ap.add_argument("--step-duration", type=float, required=True, help="seconds per step")
  ap.add_argument("--seq-len", type=float, required=True)
  ap.add_argument("--tpu-name", "--accelerator", dest="name", required=True, help="e.g. v5p-128 or b200-8")
  a = ap.parse_args(argv)
  text = Path(a.config).read_text()
  if a.config.endswith((".yaml", ".yml")):
    import yaml
    cfg = yaml.safe_load(text)
  else:
    cfg = json.loads(text)
  r = compute_mfu(cfg, a.batch_size, a.seq_len, a.step_duration, a.name)
  print(f"Model teraflops: {r.model_tflops}", file=sys.stderr)
  print(f"Hardware teraflops: {r.hardware_tflops_per_step}", file=sys.stderr)
  print(r.mfu)


if __name__ == "__main__":
  main()
