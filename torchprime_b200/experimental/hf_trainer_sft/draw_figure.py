"""Overlay two loss curves (this framework's SFT run and the HF Trainer run) in one PNG.

  python torchprime_b200/experimental/hf_trainer_sft/draw_figure.py outputs/train.log outputs/hf_trainer_sft/losses.json

The first file is a training log with ``loss: <float>`` per step, the second the JSON written by
``run_sft_gsm8k.py``.  Same purpose as the reference's experimental/torchrun_gpu_sft/draw_figure.py.
"""

from __future__ import annotations

import json
import re
import sys


def losses_from_log(path: str):
  pat = re.compile(r"loss:\s*([0-9.eE+-]+)")
  with open(path) as f:
    return [float(m.group(1)) for line in f for m in [pat.search(line)] if m]


def main(argv=None):
  argv = argv or sys.argv[1:]
  ours = losses_from_log(argv[0])
  with open(argv[1]) as f:
    hf = [v for _, v in json.load(f)]
  import matplotlib
  matplotlib.use("Agg")
  import matplotlib.pyplot as plt
  plt.plot(range(1, len(ours) + 1), ours, label="torchprime_b200")
  plt.plot(range(1, len(hf) + 1), hf, label="HF Trainer + FSDP")
  plt.xlabel("step"); plt.ylabel("loss"); plt.legend(); plt.grid(alpha=0.3)
  out = argv[2] if len(argv) > 2 else "sft_loss_comparison.png"
  plt.savefig(out, dpi=120)
  print("wrote", out)


if __name__ == "__main__":
  main()
