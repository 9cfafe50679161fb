"""Microbenchmark of the mixture-of-experts kernels on one GPU.

  python bench/moe_bench.py [--config mixtral|deepseek|small] [--iters 10] [--no-library]

For one layer's routed experts (Mixtral 8x7B: 8 experts, top-2, D 4096, F 14336, 8192 tokens;
DeepSeek-V2-Lite: 64 experts, top-6, D 2048, F 1408, 8192 tokens) prints the time of every stage
(CUDA events after warm-up): router, dispatch plan, row gather, grouped gate/up GEMM with the SwiGLU
epilogue, grouped down GEMM, weighted combine, and the three weight-gradient grouped GEMMs; the
achieved TFLOP/s of the GEMMs counts only the routed rows (padding excluded) against the cuBLAS
peak measured on the box.  Unless ``--no-library`` is given the same work is also run as one
torch.matmul per expert (cuBLAS) for comparison.  ``small`` is a shape for profiler captures.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from torchprime_b200.metrics.mfu import measured_peak_tflops  # noqa: E402
from torchprime_b200.ops import _lib  # noqa: E402
from torchprime_b200.ops import moe  # noqa: E402

CONFIGS = {
  "mixtral": dict(T=8192, D=4096, F=14336, E=8, K=2, mode="softmax"),
  "deepseek": dict(T=8192, D=2048, F=1408, E=64, K=6, mode="sigmoid"),
  "small": dict(T=2048, D=2048, F=4096, E=8, K=2, mode="softmax"),
  "medium": dict(T=8192, D=2048, F=4096, E=8, K=2, mode="softmax"),    # Mixtral's rows per expert at a profiler-sized footprint
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
  ap.add_argument("--config", choices=sorted(CONFIGS), default="mixtral")
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--no-library", action="store_true")
  args = ap.parse_args()
  c = CONFIGS[args.config]
  T, D, F, E, K = c["T"], c["D"], c["F"], c["E"], c["K"]
  peaks = measured_peak_tflops() or {}
  peak, hbm = float(peaks.get("bf16_tflops", 1590.0)), float(peaks.get("hbm_gbs", 6650.0))
  dev, bf = "cuda", torch.bfloat16
  torch.manual_seed(0)
  x = torch.randn(T, D, device=dev, dtype=bf)
  logits = torch.randn(T, E, device=dev, dtype=torch.float32)
  wg = (torch.randn(E, D, F, device=dev) * 0.02).to(bf)
  wu = (torch.randn(E, D, F, device=dev) * 0.02).to(bf)
  wd = (torch.randn(E, F, D, device=dev) * 0.02).to(bf)

  def line(name, t, flops=None, nbytes=None):
    extra = ""
    if flops:
      extra = f"{flops / t / 1e9:7.0f} TFLOP/s  {flops / t / 1e9 / peak:5.2f} of measured cuBLAS peak"
    elif nbytes:
      extra = f"{nbytes / t / 1e6:7.0f} GB/s     {nbytes / t / 1e6 / hbm:5.2f} of measured copy bandwidth"
    print(f"{name:34s} {t * 1e3:9.1f} us  {extra}", flush=True)

  kw = dict(mode=c["mode"]) if c["mode"] == "softmax" else dict(mode="sigmoid", bias=torch.zeros(E, device=dev),
                                                                 n_group=8, topk_group=4)
  line("router top-k", timed(lambda: moe.router_topk(logits, K, **kw), args.iters), nbytes=T * E * 4 + T * K * 8)
  w, idx, _ = moe.router_topk(logits, K, **kw)
  line("dispatch plan (device sort)", timed(lambda: moe.build_dispatch_plan(idx, E), args.iters))
  plan = moe.build_dispatch_plan(idx, E)
  rows = T * K
  line("gather rows", timed(lambda: moe.gather_rows(x, plan.src_row), args.iters), nbytes=2 * rows * D * 2)
  xg = moe.gather_rows(x, plan.src_row)
  gu = torch.empty(plan.num_rows, 2 * F, dtype=bf, device=dev)
  f_up = 2.0 * rows * D * 2 * F
  line("grouped gate|up GEMM + SwiGLU", timed(lambda: moe.grouped_gemm_rows(
      xg, wg, plan, b_mn=True, b2=wu, epi=_lib.EPI_SWIGLU, c2=gu, n_total=2 * F), args.iters), flops=f_up)
  act = moe.grouped_gemm_rows(xg, wg, plan, b_mn=True, b2=wu, epi=_lib.EPI_SWIGLU, c2=gu, n_total=2 * F)
  f_dn = 2.0 * rows * F * D
  line("grouped down GEMM", timed(lambda: moe.grouped_gemm_rows(act, wd, plan, b_mn=True), args.iters), flops=f_dn)
  out_rows = moe.grouped_gemm_rows(act, wd, plan, b_mn=True)
  line("weighted combine", timed(lambda: moe.combine_rows(out_rows, plan.dest, w), args.iters),
       nbytes=(rows + T) * D * 2)
  line("grouped dgrad (down, transposed)", timed(lambda: moe.grouped_gemm_rows(out_rows, wd, plan, b_mn=False),
                                                   args.iters), flops=f_dn)
  gwd = torch.empty(E, F, D, dtype=torch.float32, device=dev)
  line("grouped wgrad (down, fp32 out)", timed(lambda: moe.grouped_gemm_wgrad(act, out_rows, plan, gwd, False),
                                                 args.iters), flops=f_dn)
  line("whole routed MLP forward", timed(lambda: moe.grouped_mlp(x, w, idx, wg, wu, wd), args.iters),
       flops=f_up + f_dn)
  if not args.no_library:
    counts = plan.counts.tolist()
    offs = plan.k_offsets.tolist()

    def per_expert():
      for e in range(E):
        if counts[e]:
          a = xg[offs[e]:offs[e] + counts[e]]
          h = torch.nn.functional.silu(a @ wg[e]) * (a @ wu[e])
          h @ wd[e]
    line("cuBLAS, one matmul per expert", timed(per_expert, args.iters), flops=f_up + f_dn)
  print("device status block:", _lib.status())


if __name__ == "__main__":
  main()
