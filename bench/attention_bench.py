"""Microbenchmark of the flash-attention forward and backward kernels.

  python bench/attention_bench.py [--seq 8192] [--batch 1] [--heads 32] [--kv-heads 8] [--iters 10]
                                  [--no-library] [--only fwd|bwd]

Prints one line per kernel: time per call (CUDA events, after warm-up; a buffer larger than
L2 is rewritten between timed calls) and the achieved tensor throughput counted with the
causal mask (half of the score matrix).  Unless ``--no-library`` is given the same shapes are also run through
torch's scaled_dot_product_attention for comparison.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from torchprime_b200.ops import _lib  # noqa: E402
from torchprime_b200.ops import attention_sm100 as A  # noqa: E402


def timed(fn, iters, flush):
  for _ in range(3):
    fn()
  torch.cuda.synchronize()
  total = 0.0
  for _ in range(iters):
    flush.add_(1)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    fn()
    e.record()
    torch.cuda.synchronize()
    total += s.elapsed_time(e)
  return total / iters


def _print_cycle_counters(launch):
  """A library built with ``TPB_NVCC_EXTRA=-DTPB_ATTN_PROF=<1|2|3> python -m torchprime_b200.build --force``
  exports the two-tile forward kernel's in-kernel cycle counters (``TPB_ATTN_FWD_V2=1``): print the sums of one
  launch (slots 0-7: a softmax thread at level 2 or the P V k-steps at level 3; slots 8-15: the MMA thread)."""
  import ctypes
  L = _lib.lib()
  if not hasattr(L, "tpb_attn_fwd_prof_read"):
    return
  host = (ctypes.c_ulonglong * 16)()
  L.tpb_attn_fwd_prof_read.argtypes = [ctypes.c_void_p]
  L.tpb_attn_fwd_prof_read.restype = ctypes.c_int
  torch.cuda.synchronize()
  L.tpb_attn_fwd_prof_read(host)      # clear what the timed launches accumulated
  launch()
  torch.cuda.synchronize()
  L.tpb_attn_fwd_prof_read(host)
  print("attn_fwd cycle counters of one launch:", list(host))


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--seq", type=int, default=8192)
  ap.add_argument("--batch", type=int, default=1)
  ap.add_argument("--heads", type=int, default=32)
  ap.add_argument("--kv-heads", type=int, default=8)
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--only", choices=["fwd", "bwd"], default=None)
  ap.add_argument("--no-library", action="store_true")
  args = ap.parse_args()
  b, s, hq, hkv, d = args.batch, args.seq, args.heads, args.kv_heads, 128
  torch.manual_seed(0)
  buf = torch.randn(b, s, (hq + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16)
  q = buf[..., : hq * d].view(b, s, hq, d)
  k = buf[..., hq * d : (hq + hkv) * d].view(b, s, hkv, d)
  v = buf[..., (hq + hkv) * d :].view(b, s, hkv, d)
  flush = torch.zeros(160 << 20, dtype=torch.uint8, device="cuda")   # > 126 MB of L2
  fwd_flops = 4 * b * s * s * hq * d / 2
  bwd_flops = 2.5 * fwd_flops
  if args.only in (None, "fwd"):
    t = timed(lambda: A.attn_fwd(q, k, v, causal=True), args.iters, flush)
    print(f"attn_fwd  {t:8.3f} ms  {fwd_flops / t / 1e9:7.0f} TFLOP/s")
    _print_cycle_counters(lambda: A.attn_fwd(q, k, v, causal=True))
  if args.only in (None, "bwd"):
    o, lse = A.attn_fwd(q, k, v, causal=True)
    do = torch.randn_like(o)
    dbuf = torch.empty_like(buf)
    dq = dbuf[..., : hq * d].view(b, s, hq, d)
    dk = dbuf[..., hq * d : (hq + hkv) * d].view(b, s, hkv, d)
    dv = dbuf[..., (hq + hkv) * d :].view(b, s, hkv, d)
    t = timed(lambda: A.attn_bwd(do, q, k, v, o, lse, causal=True, dq=dq, dk=dk, dv=dv), args.iters, flush)
    print(f"attn_bwd  {t:8.3f} ms  {bwd_flops / t / 1e9:7.0f} TFLOP/s")
  if not args.no_library:
    qt, kt, vt = (x.transpose(1, 2).detach().requires_grad_(True) for x in (q, k, v))
    sdpa = lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True)  # noqa: E731
    if args.only in (None, "fwd"):
      with torch.no_grad():
        t = timed(sdpa, args.iters, flush)
      print(f"sdpa_fwd  {t:8.3f} ms  {fwd_flops / t / 1e9:7.0f} TFLOP/s")
    if args.only in (None, "bwd"):
      oo = sdpa()
      dd = torch.randn_like(oo)
      t = timed(lambda: torch.autograd.grad(oo, (qt, kt, vt), dd, retain_graph=True), args.iters, flush)
      print(f"sdpa_bwd  {t:8.3f} ms  {bwd_flops / t / 1e9:7.0f} TFLOP/s")
  print("device status block:", _lib.status())


if __name__ == "__main__":
  main()
