"""Builds ``libtpb200.so`` (all sm_100a kernels) in-tree with nvcc.

``python -m torchprime_b200.build`` compiles every ``csrc/*.cu`` with
``-gencode arch=compute_100a,code=sm_100a`` and links them into
``torchprime_b200/lib/libtpb200.so``.  nvcc cross-compiles, so this works on a
machine without a GPU; the shared object is loaded with ctypes (ops/_lib.py).
Objects are rebuilt only when a source or header is newer than the object.
"""

from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")
BUILD = os.path.join(ROOT, "build")
LIB_DIR = os.path.join(ROOT, "torchprime_b200", "lib")
LIB_PATH = os.path.join(LIB_DIR, "libtpb200.so")

NVCC_FLAGS = [
  "-gencode", "arch=compute_100a,code=sm_100a",
  "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
  "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
  for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
    if cand and os.path.exists(cand):
      return cand
  raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def _newest_header() -> float:
  hs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
  return max((os.path.getmtime(h) for h in hs), default=0.0)


def _compile(src: str, verbose: bool) -> str:
  obj = os.path.join(BUILD, os.path.basename(src)[:-3] + ".o")
  stamp = max(os.path.getmtime(src), _newest_header())
  if os.path.exists(obj) and os.path.getmtime(obj) >= stamp:
    return obj
  # TPB_NVCC_EXTRA: extra compiler flags for instrumented developer builds (e.g. -DTPB_ATTN_PROF)
  cmd = [_nvcc(), *NVCC_FLAGS, *os.environ.get("TPB_NVCC_EXTRA", "").split(), "-I", CSRC, "-c", src, "-o", obj]
  if verbose:
    cmd[1:1] = ["-Xptxas", "-v"]
  res = subprocess.run(cmd, capture_output=True, text=True)
  if res.returncode != 0:
    raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
  if verbose:
    sys.stderr.write(res.stderr)
  return obj


def build(force: bool = False, verbose: bool = False) -> str:
  os.makedirs(BUILD, exist_ok=True)
  os.makedirs(LIB_DIR, exist_ok=True)
  sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
  if force:
    for o in glob.glob(os.path.join(BUILD, "*.o")):
      os.remove(o)
  with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
    objs = list(ex.map(lambda s: _compile(s, verbose), sources))
  newest = max(os.path.getmtime(o) for o in objs)
  if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < newest:
    cmd = [_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
      raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
  return LIB_PATH


if __name__ == "__main__":
  print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
