"""Microbenchmark of the peer-memory FSDP collectives on one Llama-3-8B layer (218 M parameters).

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 bench/fsdp_comm_bench.py

Per rank count W, CUDA events on the launching stream, max over ranks, after warm-up:

  gather     copy-engine all-gather of the layer's bf16 shards (own shard + W-1 peer copies, one flag each,
             copies alternating between two streams; `gather_one_lane_ms`: all on one stream)
  wgrad      gate|up weight-gradient GEMM (28672 x 4096 x 8192 tokens) written locally (the GEMM alone)
  wgrad+rs   the same GEMM with the epilogue that stores every tile into the owners' staging slots
  reduce     fixed-order fp32 reduction of the W staging slots into the gradient shard

Rooflines: gather and the scatter side of wgrad+rs move (W-1)/W of the bytes over NVLink; the link
rate is 900 GB/s per direction (nominal) and 770 GB/s (measured peer copy); the GEMM's own bound is its
FLOPs at the measured cuBLAS bf16 rate.  Every fused path is reported as achieved / max(compute, link).
"""

from __future__ import annotations

import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LINK_NOMINAL, LINK_MEASURED = 900e9, 770e9


def timed(fn, iters=10, warmup=3):
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(iters):
    fn()
  e1.record()
  torch.cuda.synchronize()
  return e0.elapsed_time(e1) / iters * 1e-3


def main():
  import torch.distributed as dist
  from torchprime_b200.dist import runtime as rt
  from torchprime_b200.dist.symm import SymmetricBuffer
  from torchprime_b200.metrics.mfu import measured_peak_tflops
  from torchprime_b200.ops import _lib, kernels as k
  from torchprime_b200.ops._lib import check, lib, ptr, stream_ptr
  from torchprime_b200.parallel import fsdp_comm  # noqa: F401  (registers the C signatures)
  dev = rt.init()
  world, rank = rt.world_size(), rt.rank()
  peak = (measured_peak_tflops() or {}).get("bf16_tflops", 1590.0) * 1e12
  layer = 218_112_000 + 8192                       # parameters of one Llama-3-8B decoder layer
  shard = (layer + world * 8 - 1) // (world * 8) * 8
  L = lib()
  out = {"world": world}

  # ---- gather: copy engines, own shard first, peers in rotated order, one flag per shard
  params = SymmetricBuffer(shard, torch.bfloat16, dev)
  params.local.normal_()
  gathered = torch.empty(shard * world, dtype=torch.bfloat16, device=dev)
  flags = torch.zeros(world, dtype=torch.int32, device=dev)
  params.barrier()
  epoch = [0]

  lane2 = torch.cuda.Stream()

  def gather(lanes=2):
    epoch[0] += 1
    main = torch.cuda.current_stream()
    streams = (main, lane2) if lanes == 2 else (main,)
    if lanes == 2:
      lane2.wait_stream(main)
    fsdp_comm.gather_shards(gathered.data_ptr(), params.ptrs, 2 * shard, flags.data_ptr(), epoch[0], rank, streams)
    if lanes == 2:
      main.wait_stream(lane2)
  out["gather_one_lane_ms"] = round(rt.all_reduce_max_float(timed(lambda: gather(1))) * 1e3, 3)
  t = rt.all_reduce_max_float(timed(gather))
  recv = 2 * shard * (world - 1)
  out["gather_ms"] = round(t * 1e3, 3)
  out["gather_recv_GBps"] = round(recv / t / 1e9, 1)
  out["gather_of_900"] = round(recv / t / LINK_NOMINAL, 3)
  out["gather_of_770"] = round(recv / t / LINK_MEASURED, 3)
  gathered_nccl = torch.empty_like(gathered)
  t_nccl = rt.all_reduce_max_float(timed(lambda: dist.all_gather_into_tensor(gathered_nccl, params.local)))
  out["nccl_all_gather_ms"] = round(t_nccl * 1e3, 3)

  # ---- weight gradient of the fused gate|up projection: [28672, 4096] over 8192 tokens
  T, N, K = 8192, 28672, 4096
  dy = torch.randn(T, N, device=dev, dtype=torch.bfloat16)
  x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
  local = torch.empty(N, K, device=dev, dtype=torch.bfloat16)
  flops = 2.0 * T * N * K
  t_local = rt.all_reduce_max_float(timed(lambda: k.gemm(dy, x, a_mn=True, b_mn=True, out=local)))
  out["wgrad_ms"] = round(t_local * 1e3, 3)
  out["wgrad_TFLOPs"] = round(flops / t_local / 1e12, 1)
  wshard = (N * K + world * 8 - 1) // (world * 8) * 8
  stage = SymmetricBuffer(wshard * world, torch.bfloat16, dev)       # [source][shard] at every owner
  table = stage.ptr_table(rank * wshard)
  stage.barrier()

  def wgrad_rs():
    check(L.tpb_gemm_rs_store_bf16(ptr(dy), ptr(x), N, K, T, dy.stride(0), x.stride(0), K, 1, 1, 1.0, table, world,
                                   wshard, 0, rank, stream_ptr()), "gemm_rs_store")
  t_rs = rt.all_reduce_max_float(timed(wgrad_rs))
  sent = 2.0 * N * K * (world - 1) / world
  roof = max(flops / peak, sent / LINK_NOMINAL)
  out["wgrad_rs_ms"] = round(t_rs * 1e3, 3)
  out["wgrad_rs_of_roofline_900"] = round(roof / t_rs, 3)
  out["wgrad_rs_of_roofline_770"] = round(max(flops / peak, sent / LINK_MEASURED) / t_rs, 3)
  grad_full = torch.empty(wshard * world, dtype=torch.bfloat16, device=dev)
  gshard = torch.empty(wshard, dtype=torch.bfloat16, device=dev)

  def wgrad_then_nccl():
    k.gemm(dy, x, a_mn=True, b_mn=True, out=grad_full[:N * K].view(N, K))
    dist.reduce_scatter_tensor(gshard, grad_full, op=dist.ReduceOp.AVG)
  out["wgrad_then_nccl_rs_ms"] = round(rt.all_reduce_max_float(timed(wgrad_then_nccl)) * 1e3, 3)

  # ---- fixed-order reduction of the staging slots
  red = torch.empty(wshard, dtype=torch.bfloat16, device=dev)
  t_red = rt.all_reduce_max_float(timed(lambda: check(L.tpb_rs_reduce_bf16(
    stage.local.data_ptr(), world, wshard, wshard, red.data_ptr(), 0, 0, 1.0 / world, stream_ptr()), "reduce")))
  hbm = (measured_peak_tflops() or {}).get("hbm_gbs", 6650.0) * 1e9
  out["reduce_ms"] = round(t_red * 1e3, 3)
  out["reduce_of_hbm"] = round(2.0 * wshard * (world + 1) / t_red / hbm, 3)
  torch.cuda.synchronize()
  _lib.raise_on_device_timeout()
  if rank == 0:
    print(json.dumps(out), flush=True)
  rt.barrier()
  for sb in (stage, params):
    sb.close()
  rt.shutdown()


if __name__ == "__main__":
  main()
