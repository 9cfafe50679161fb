"""Microbenchmark of the tcgen05 GEMM in the three operand layouts a training step uses.

  python bench/gemm_bench.py [--shapes llama8b|square|small] [--iters 20] [--no-library]

For every (M, N, K) prints the achieved TFLOP/s of

  fwd    C = A[M,K] . B[N,K]^T      (both operands K-major; forward and recompute)
  dgrad  C = A[M,K] . B[K,N]        (B MN-major; input gradients)
  wgrad  C = A[K,M]^T . B[K,N]      (both MN-major, fp32 output; weight gradients)

next to torch.matmul (cuBLAS) on the same shape.  Timed with CUDA events after warm-up;
the operands of the listed shapes are larger than L2 except in ``small``, which exists for
profiler captures.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from torchprime_b200.ops import _lib  # noqa: E402
from torchprime_b200.ops import kernels as k  # noqa: E402

SHAPES = {
  # tokens x out x in of the Llama-3-8B projections at 8192 tokens
  "llama8b": [(8192, 6144, 4096), (8192, 4096, 4096), (8192, 28672, 4096), (8192, 4096, 14336)],
  "square": [(8192, 8192, 8192)],
  "small": [(4096, 4096, 4096)],
}


def timed(fn, iters):
  for _ in range(3):
    fn()
  torch.cuda.synchronize()
  s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  s.record()
  for _ in range(iters):
    fn()
  e.record()
  torch.cuda.synchronize()
  return s.elapsed_time(e) / iters


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--shapes", choices=sorted(SHAPES), default="llama8b")
  ap.add_argument("--iters", type=int, default=20)
  ap.add_argument("--no-library", action="store_true")
  args = ap.parse_args()
  for m, n, kk in SHAPES[args.shapes]:
    a = torch.randn(m, kk, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, kk, device="cuda", dtype=torch.bfloat16)
    at, bt = a.t().contiguous(), b.t().contiguous()
    flops = 2 * m * n * kk
    row = [f"M{m} N{n} K{kk}:"]
    for name, fn in (("fwd", lambda: k.gemm(a, b)),
                     ("dgrad", lambda: k.gemm(a, bt, b_mn=True)),
                     ("wgrad", lambda: k.gemm(at, bt, a_mn=True, b_mn=True, epi=k.EPI_F32))):
      t = timed(fn, args.iters)
      row.append(f"{name} {flops / t / 1e9:6.0f} TF ({t:.3f} ms)")
    if not args.no_library:
      t = timed(lambda: torch.nn.functional.linear(a, b), args.iters)
      row.append(f"| cuBLAS fwd {flops / t / 1e9:6.0f} TF")
    print("  ".join(row), flush=True)
  print("device status block:", _lib.status())


if __name__ == "__main__":
  main()
