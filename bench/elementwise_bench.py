"""Microbenchmark of the bandwidth-bound kernels at Llama-3-8B shapes (8192 tokens).

  python bench/elementwise_bench.py [--iters 20] [--small]

For every kernel: time per call (CUDA events after warm-up), the bytes it has to move, the achieved
GB/s and the fraction of the copy bandwidth measured on this box (MEASURED_PEAKS.json, else
6650 GB/s).  Working sets are larger than L2 except where the op itself is small (router, RoPE
tables).  ``--small`` shrinks the token count to 2048 for profiler captures.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from torchprime_b200.metrics.mfu import measured_peak_tflops  # noqa: E402
from torchprime_b200.ops import _lib  # noqa: E402
from torchprime_b200.ops import kernels as k  # noqa: E402
from torchprime_b200.ops import moe  # noqa: E402


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
  ap.add_argument("--iters", type=int, default=20)
  ap.add_argument("--small", action="store_true")
  args = ap.parse_args()
  peaks = measured_peak_tflops() or {}
  hbm = float(peaks.get("hbm_gbs", 6650.0))
  dev = "cuda"
  T = 2048 if args.small else 8192
  D, F, V, HQKV = 4096, 14336, 128256, 6144
  bf = torch.bfloat16
  rows = []

  def add(name, fn, nbytes):
    t = timed(fn, args.iters)
    rows.append((name, t, nbytes))
    print(f"{name:28s} {t * 1e3:9.1f} us  {nbytes / 1e6:9.1f} MB  {nbytes / t / 1e6:8.0f} GB/s  "
          f"{nbytes / t / 1e6 / hbm:5.2f} of measured copy bandwidth", flush=True)

  x = torch.randn(T, D, device=dev, dtype=bf)
  res = torch.randn(T, D, device=dev, dtype=bf)
  w = torch.randn(D, device=dev, dtype=bf)
  add("rmsnorm_fwd", lambda: k.rmsnorm_fwd(x, w, 1e-5), 2 * T * D * 2)
  add("add_rmsnorm_fwd", lambda: k.rmsnorm_fwd(x, w, 1e-5, res=res, want_h=True), 4 * T * D * 2)
  _, rstd, _ = k.rmsnorm_fwd(x, w, 1e-5)
  dwf = torch.zeros(D, device=dev, dtype=torch.float32)
  add("rmsnorm_bwd", lambda: k.rmsnorm_bwd(res, x, w, rstd, dw_f32=dwf), 3 * T * D * 2)
  add("rmsnorm_bwd + residual grad", lambda: k.rmsnorm_bwd(res, x, w, rstd, dres=res, dw_f32=dwf), 4 * T * D * 2)

  qkv = torch.randn(T, HQKV, device=dev, dtype=bf)
  inv = 1.0 / (500000.0 ** (torch.arange(0, 128, 2, device=dev, dtype=torch.float32) / 128))
  ang = torch.arange(T, device=dev, dtype=torch.float32)[:, None] * inv[None]
  cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
  add("rope (q and k heads)", lambda: k.rope_(qkv, 0, 40, 128, cos, sin, T), 2 * T * 40 * 128 * 2)

  gu = torch.randn(T, 2 * F, device=dev, dtype=bf)
  dact = torch.randn(T, F, device=dev, dtype=bf)
  add("swiglu_fwd", lambda: k.swiglu_fwd(gu), 3 * T * F * 2)
  add("swiglu_bwd", lambda: k.swiglu_bwd(dact, gu), 5 * T * F * 2)

  rows_ce = T // 4
  logits = torch.randn(rows_ce, V, device=dev, dtype=bf)
  tgt = torch.randint(0, V, (rows_ce,), device=dev)
  loss = torch.zeros(1, device=dev, dtype=torch.float32)
  add("cross-entropy fwd+grad", lambda: k.ce_fwd_bwd_(logits, tgt, loss), 2 * rows_ce * V * 2)

  table = torch.randn(V, D, device=dev, dtype=bf)
  ids = torch.randint(0, V, (T,), device=dev)
  add("embedding_fwd", lambda: k.embedding_fwd(table, ids), 2 * T * D * 2)
  dtable = torch.zeros(V, D, device=dev, dtype=torch.float32)
  add("embedding_bwd", lambda: k.embedding_bwd_(x, ids, dtable), T * D * 2 + 2 * T * D * 4)

  n = (64 if args.small else 256) * 1024 * 1024
  p32 = torch.randn(n, device=dev)
  m = torch.zeros(n, device=dev)
  v = torch.zeros(n, device=dev)
  g = torch.randn(n, device=dev)
  p16 = torch.empty(n, device=dev, dtype=bf)
  add("adamw (fp32 state, bf16 out)", lambda: k.adamw_(p32, m, v, g, p16, 1e-4, 0.9, 0.95, 1e-8, 0.1, 3), n * 30)
  acc = torch.zeros(1, device=dev, dtype=torch.float32)
  add("sum of squares", lambda: k.sumsq_(g, acc), n * 4)
  add("cast f32 -> bf16", lambda: k.cast_f32_to_bf16_(g, p16), n * 6)

  router_logits = torch.randn(T, 256, device=dev, dtype=torch.float32)
  bias = torch.zeros(256, device=dev, dtype=torch.float32)
  add("router top-8 of 256 (sigmoid)", lambda: moe.router_topk(router_logits, 8, mode="sigmoid", bias=bias, n_group=8,
                                                                 topk_group=4), T * 256 * 4 + T * 8 * 8)
  wts, idx, _ = moe.router_topk(router_logits[:, :8].contiguous(), 2, mode="softmax")
  plan = moe.build_dispatch_plan(idx, 8)
  add("moe gather (top-2 of 8)", lambda: moe.gather_rows(x, plan.src_row), (T + plan.src_row.numel()) * D * 2)
  gathered = moe.gather_rows(x, plan.src_row)
  add("moe combine", lambda: moe.combine_rows(gathered, plan.dest, wts.to(bf)), (2 * T + T) * D * 2)
  print("device status block:", _lib.status())


if __name__ == "__main__":
  main()
