"""Per-kernel device-time shares of one training step (torch profiler, CUDA activity).

  python bench/step_breakdown.py [--model llama-3-8b] [--seq-len 8192] [--top 28] [hydra-style overrides ...]
  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/step_breakdown.py \\
      ici_mesh.fsdp=2 task.global_batch_size=2        # rank 0's step under FSDP

Runs two warm-up steps and profiles the third on one GPU.  The figures are for comparing
kernels with one another (shares of the step); step time itself is what ``bench.py`` measures
without a profiler attached.
"""

from __future__ import annotations

import argparse
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from torchprime_b200.config import compose  # noqa: E402
from torchprime_b200.data.synthetic import make_synthetic_dataset  # noqa: E402
from torchprime_b200.dist import runtime as rt  # noqa: E402
from torchprime_b200.models.model_utils import initialize_model_class  # noqa: E402
from torchprime_b200.trainer import Trainer  # noqa: E402


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--model", default="llama-3-8b")
  ap.add_argument("--seq-len", type=int, default=8192)
  ap.add_argument("--top", type=int, default=28)
  args, overrides = ap.parse_known_args()
  rt.init()
  cfg = compose("default", [f"model={args.model}", "dataset=synthetic", f"dataset.block_size={args.seq_len}",
                            "task.global_batch_size=1", "task.max_steps=10", "task.optimizer.type=adamw",
                            "ici_mesh.fsdp=1", "profile_start_step=-1", f"output_dir={tempfile.mkdtemp()}"] + overrides)
  model = initialize_model_class(cfg.model, device="meta")
  data = make_synthetic_dataset(vocab_size=cfg.model.vocab_size, block_size=args.seq_len, num_samples=16)
  tr = Trainer(model=model, config=cfg, train_dataset=data)
  loader = tr._get_train_dataloader()
  for _ in range(2):
    tr.train_step(tr._prepare_batch(loader.next_batch()))
  torch.cuda.synchronize()
  batch = tr._prepare_batch(loader.next_batch())
  acts = [torch.profiler.ProfilerActivity.CUDA, torch.profiler.ProfilerActivity.CPU]
  with torch.profiler.profile(activities=acts) as prof:
    tr.train_step(batch)
    torch.cuda.synchronize()
  rows = [(e.key, e.device_time_total / 1e3, e.count) for e in prof.key_averages()
          if e.device_time_total > 0 and getattr(e, "device_type", None) is not None]
  kernels = [(e.key, e.self_device_time_total / 1e3, e.count) for e in prof.key_averages() if e.self_device_time_total > 0]
  kernels.sort(key=lambda r: -r[1])
  total = sum(r[1] for r in kernels)
  if rt.rank() == 0:     # under torchrun (add ici_mesh.fsdp=N task.global_batch_size=N) rank 0 reports its own step
    print(f"total device time {total:.1f} ms over {sum(r[2] for r in kernels)} launches")
    for name, ms, count in kernels[: args.top]:
      print(f"{ms:9.2f} ms {100 * ms / total:5.1f}%  x{count:<5d} {name[:110]}")
  rt.barrier()
  tr.engine.close()
  rt.shutdown()


if __name__ == "__main__":
  main()
