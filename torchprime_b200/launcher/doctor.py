"""Environment checks for a B200 box (reference: launcher/doctor.py checks docker / gcloud / kubectl
for its cluster workflow).  Read-only: it never changes a GPU setting."""

from __future__ import annotations

import os
import shutil
import subprocess
import sys


def _ok(msg):
  print(f"  [ok]   {msg}")
  return True


def _bad(msg):
  print(f"  [FAIL] {msg}")
  return False


def check_nvcc() -> bool:
  nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
  if not os.path.exists(nvcc):
    return _bad("nvcc not found (needed to build the sm_100a kernels)")
  out = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout
  rel = next((l for l in out.splitlines() if "release" in l), "").strip()
  return _ok(f"nvcc: {rel}")


def check_library() -> bool:
  from ..ops import _lib
  if _lib.available():
    return _ok(f"kernel library: {_lib.lib_path()}")
  return _bad("kernel library missing: run `tp build` (python -m torchprime_b200.build)")


def check_gpus() -> bool:
  import torch
  if not torch.cuda.is_available():
    return _bad("no CUDA device visible (CPU-only runs and tests still work)")
  ok = True
  n = torch.cuda.device_count()
  for i in range(n):
    p = torch.cuda.get_device_properties(i)
    line = f"GPU {i}: {p.name}, {p.total_memory / 2**30:.0f} GiB, sm_{p.major}{p.minor}, {p.multi_processor_count} SMs"
    ok &= _ok(line) if p.major >= 10 else _bad(line + " (kernels need sm_100a)")
  for i in range(n):
    for j in range(n):
      if i != j and not torch.cuda.can_device_access_peer(i, j):
        ok &= _bad(f"no P2P access {i} -> {j}: fused collective kernels need NVLink peer mapping")
  if n > 1 and ok:
    _ok(f"peer access between all {n} GPUs")
  return ok


def check_distributed() -> bool:
  import torch.distributed as dist
  return _ok(f"torch.distributed backends: nccl={dist.is_nccl_available()} gloo={dist.is_gloo_available()}")


def run_checks() -> int:
  print("torchprime_b200 doctor")
  results = [check_nvcc(), check_library(), check_gpus(), check_distributed()]
  return 0 if all(results[:2]) else 1


if __name__ == "__main__":
  sys.exit(run_checks())
