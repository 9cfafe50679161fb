"""Writes a log of the runtime environment: arguments, platform, environment variables, package
versions, GPUs and a small device smoke computation.  Counterpart of the reference's
tools/system_check.py:1-167 (which smoke-tests torch_xla); output goes to
``<output_dir>/log-<timestamp>.log`` and to stdout."""

from __future__ import annotations

import argparse
import datetime
import importlib.metadata as md
import os
import platform
import sys


def gather(argv) -> list[str]:
  lines = ["== arguments ==", " ".join(argv), "== system =="]
  lines += [f"python {sys.version.split()[0]} on {platform.platform()}", f"cpu count {os.cpu_count()}"]
  lines.append("== environment ==")
  for k in sorted(os.environ):
    if k.startswith(("TORCHPRIME_", "NCCL_", "CUDA_", "RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_")):
      lines.append(f"{k}={os.environ[k]}")
  lines.append("== packages ==")
  for pkg in ("torch", "numpy", "transformers", "datasets", "safetensors", "tensorboard", "pyyaml"):
    try:
      lines.append(f"{pkg}=={md.version(pkg)}")
    except md.PackageNotFoundError:
      lines.append(f"{pkg}: not installed")
  lines.append("== devices ==")
  import torch
  lines.append(f"cuda available: {torch.cuda.is_available()}")
  if torch.cuda.is_available():
    for i in range(torch.cuda.device_count()):
      p = torch.cuda.get_device_properties(i)
      lines.append(f"cuda:{i} {p.name} {p.total_memory / 2**30:.0f} GiB sm_{p.major}{p.minor}")
    a = torch.ones(4, device="cuda") + torch.ones(4, device="cuda")
    lines.append(f"device smoke add: {a.tolist()}")
  else:
    lines.append(f"cpu smoke add: {(torch.ones(4) + torch.ones(4)).tolist()}")
  from torchprime_b200.ops import _lib
  lines.append(f"kernel library built: {_lib.available()} ({_lib.lib_path()})")
  return lines


def main(argv=None):
  argv = list(sys.argv[1:] if argv is None else argv)
  ap = argparse.ArgumentParser()
  ap.add_argument("--output_dir", "--output-dir", dest="output_dir", default=None)
  known, rest = ap.parse_known_args(argv)
  out_dir = known.output_dir
  for r in rest:
    if r.startswith("output_dir="):
      out_dir = r.split("=", 1)[1]
  out_dir = out_dir or "outputs"
  os.makedirs(out_dir, exist_ok=True)
  lines = gather(argv)
  path = os.path.join(out_dir, f"log-{datetime.datetime.now().strftime('%Y%m%d-%H%M%S')}.log")
  with open(path, "w") as f:
    f.write("\n".join(lines) + "\n")
  print("\n".join(lines))
  print(f"wrote {path}")
  return 0


if __name__ == "__main__":
  sys.exit(main())
