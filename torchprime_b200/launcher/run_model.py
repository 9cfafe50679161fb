"""Times N forward passes of a registry model (reference: launcher/run_model.py, which offers
torch_xla and torchax back ends; here: eager CUDA, CUDA-graph replay, or CPU).

  python -m torchprime_b200.launcher.run_model --model resnet18 --batch-size 8 --runs 5 [--mode graph]
"""

from __future__ import annotations

import argparse
import time

import torch
from torch.utils import _pytree as pytree

from ..models import registry


def _sync(device):
  if device.type == "cuda":
    torch.cuda.synchronize()


def run_model_eager(model, batch_size: int, number_of_runs: int, device: torch.device) -> list[float]:
  model = model.to(device).eval()
  times = []
  with torch.no_grad():
    for _ in range(number_of_runs):
      args, kwargs = pytree.tree_map_only(torch.Tensor, lambda t: t.to(device), model.get_sample_inputs(batch_size))
      _sync(device)
      t0 = time.perf_counter()
      model(*args, **kwargs)
      _sync(device)
      times.append(time.perf_counter() - t0)
  return times


def run_model_graph(model, batch_size: int, number_of_runs: int, device: torch.device) -> list[float]:
  """Capture one forward in a CUDA graph and time replays (the compile-once analogue)."""
  from ..utils.cuda_graphs import GraphedForward
  assert device.type == "cuda", "graph mode needs a CUDA device"
  model = model.to(device).eval()
  args, kwargs = pytree.tree_map_only(torch.Tensor, lambda t: t.to(device), model.get_sample_inputs(batch_size))
  graphed = GraphedForward(model)
  graphed(*args, **kwargs)          # warm-up and capture
  times = []
  for _ in range(number_of_runs):
    _sync(device)
    t0 = time.perf_counter()
    graphed(*args, **kwargs)
    _sync(device)
    times.append(time.perf_counter() - t0)
  return times


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--model", required=True, choices=sorted(registry))
  ap.add_argument("--batch-size", type=int, default=1)
  ap.add_argument("--runs", type=int, default=5)
  ap.add_argument("--mode", default="eager", choices=["eager", "graph"])
  a = ap.parse_args(argv)
  device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
  model = registry[a.model]()
  fn = run_model_graph if a.mode == "graph" else run_model_eager
  times = fn(model, a.batch_size, a.runs, device)
  for i, t in enumerate(times):
    print(f"run {i}: {t * 1e3:.3f} ms")
  return times


if __name__ == "__main__":
  main()
