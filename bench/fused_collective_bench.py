"""Micro-benchmark of the fused compute+collective kernels against NCCL + GEMM and their roofline.

  python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench/fused_collective_bench.py

Shapes are one Llama-3-8B decoder layer on one 8192-token sequence per GPU: the FSDP gather of the
layer's 218 M bf16 parameters fused into the QKV projection, and the gate/up weight-gradient GEMM
fused with its reduce-scatter, and a zig-zag context-parallel attention forward (8192 keys per
rank) with its K/V exchange inside the kernel.  Roofline = max(FLOPs / measured cuBLAS peak, bytes that cross NVLink /
770 GB/s per direction).  Times are CUDA-event times, max over ranks.
"""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from torchprime_b200.dist import runtime as rt
from torchprime_b200.dist.symm import SymmetricBuffer
from torchprime_b200.metrics.mfu import measured_peak_tflops
from torchprime_b200.ops import _lib, fused_collective as fc, kernels as k

NVLINK_GBS = 770.0


def timed(fn, pre=None, n=10, warm=3):
  ts = []
  for i in range(warm + n):
    if pre:
      pre()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    fn()
    e.record()
    torch.cuda.synchronize()
    if i >= warm:
      ts.append(s.elapsed_time(e))
  ts.sort()
  return rt.all_reduce_max_float(ts[len(ts) // 2])


def main():
  dev = rt.init()
  world, rank = rt.world_size(), rt.rank()
  peak = (measured_peak_tflops() or {}).get("bf16_tflops", 1590.0)
  T, D, F, HQKV = 8192, 4096, 14336, 6144
  unit = HQKV * D + D * D + 2 * F * D + F * D + 2 * D          # parameters of one decoder layer
  shard = (unit + world * 8 - 1) // (world * 8) * 8
  sb = SymmetricBuffer(shard, torch.bfloat16, dev)
  sb.local.normal_(0, 0.02)
  gathered = torch.empty(shard * world, dtype=torch.bfloat16, device=dev)
  x = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
  out = {}

  # ---- F1: all-gather fused into the QKV GEMM
  ag = fc.AllGatherGemm(sb, shard, copiers=int(os.environ.get("TPB_AG_COPIERS", "32")), push=False)
  t_fused = timed(lambda: ag(x, gathered, 0, HQKV, D), pre=sb.barrier)
  agp = fc.AllGatherGemm(sb, shard, copiers=int(os.environ.get("TPB_AG_COPIERS", "32")), push=True, multicast=False)
  t_push = timed(lambda: agp(x, None, 0, HQKV, D), pre=sb.barrier)
  # multicast push (one multimem store reaches every rank), swept over the number of copier CTAs
  mc = {}
  for cop in [int(c) for c in os.environ.get("TPB_AG_MC_COPIERS", "8,16,32").split(",")]:
    agm = fc.AllGatherGemm(sb, shard, copiers=cop, push=True, multicast=True)
    if not agm.multicast_ptr:
      mc = {"unavailable": "no multicast mapping on this platform"}
      break
    mc[str(cop)] = timed(lambda: agm(x, None, 0, HQKV, D), pre=sb.barrier)
  def nccl_then_gemm():
    dist.all_gather_into_tensor(gathered, sb.local)
    k.gemm(x, gathered[:HQKV * D].view(HQKV, D))
  t_nccl = timed(nccl_then_gemm)
  t_gemm = timed(lambda: k.gemm(x, gathered[:HQKV * D].view(HQKV, D)))
  flops = 2.0 * T * HQKV * D
  link_bytes = (world - 1) * shard * 2
  roof = max(flops / (peak * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
  best_mc = min([v for v in mc.values() if isinstance(v, float)], default=None)
  out["ag_gemm"] = {"fused_push_multicast_ms_by_copiers": mc,
                    "fraction_of_roofline_push_multicast": roof / best_mc if best_mc else None,
                    "fused_push_ms": t_push, "fraction_of_roofline_push": roof / t_push,
                    "fused_pull_ms": t_fused, "nccl_allgather_plus_gemm_ms": t_nccl, "gemm_only_ms": t_gemm,
                    "roofline_ms": roof, "fraction_of_roofline": roof / t_fused, "nvlink_bytes_in": link_bytes,
                    "copier_ctas": ag.copiers}

  # ---- F2: gate/up weight gradient fused with its reduce-scatter
  N2 = 2 * F
  gsz = (N2 * D + world * 8 - 1) // (world * 8) * 8
  gs = SymmetricBuffer(gsz, torch.bfloat16, dev)
  dy = torch.randn(T, N2, device=dev, dtype=torch.bfloat16)
  def pre_rs():
    gs.local.zero_()
    gs.barrier()
  t_rs = timed(lambda: fc.gemm_rs(dy, x, a_mn=True, b_mn=True, m=N2, n=D, ldc=D, grad_shards=gs, shard_elems=gsz,
                                  c_offset=0, alpha=1.0 / world), pre=pre_rs)
  full = torch.empty(gsz * world, dtype=torch.bfloat16, device=dev)
  shard_out = torch.empty(gsz, dtype=torch.bfloat16, device=dev)
  def nccl_rs():
    k.gemm(dy, x, a_mn=True, b_mn=True, out=full[:N2 * D].view(N2, D))
    dist.reduce_scatter_tensor(shard_out, full, op=dist.ReduceOp.AVG)
  t_nccl_rs = timed(nccl_rs)
  flops2 = 2.0 * T * N2 * D
  link2 = (world - 1) * gsz * 2
  roof2 = max(flops2 / (peak * 1e12), link2 / (NVLINK_GBS * 1e9)) * 1e3
  out["gemm_rs"] = {"fused_ms": t_rs, "gemm_plus_nccl_reduce_scatter_ms": t_nccl_rs, "roofline_ms": roof2,
                    "fraction_of_roofline": roof2 / t_rs, "nvlink_bytes_out": link2}
  # ---- F5: context-parallel attention forward with the K/V exchange inside the kernel
  from torchprime_b200.dist.mesh import Mesh
  from torchprime_b200.parallel.cp import ContextParallelAttention
  mesh = Mesh(shape={"data": 1, "fsdp": 1, "tensor": 1, "expert": 1, "context": world}, rank=rank, world_size=world)
  s_loc, hq, hkv, hd = 8192, 32, 8, 128
  qkv = torch.randn(1, s_loc, (hq + 2 * hkv) * hd, device=dev, dtype=torch.bfloat16)
  q = qkv[..., :hq * hd].view(1, s_loc, hq, hd)
  kk = qkv[..., hq * hd:(hq + hkv) * hd].view(1, s_loc, hkv, hd)
  vv = qkv[..., (hq + hkv) * hd:].view(1, s_loc, hkv, hd)
  nccl_cp = ContextParallelAttention(mesh, load_balanced=True, fused_exchange=False)
  fused_cp = ContextParallelAttention(mesh, load_balanced=True, fused_exchange=True, fused_multicast=False,
                                      fused_copiers=int(os.environ.get("TPB_CP_COPIERS", "16")))
  cp_mc = {}
  with torch.no_grad():
    t_cp_nccl = timed(lambda: nccl_cp.attention(q, kk, vv))
    t_cp_fused = timed(lambda: fused_cp.attention(q, kk, vv))
    for cop in [int(c) for c in os.environ.get("TPB_CP_MC_COPIERS", "4,8,16").split(",")]:
      cpm = ContextParallelAttention(mesh, load_balanced=True, fused_exchange=True, fused_multicast=True,
                                     fused_copiers=cop)
      t = timed(lambda: cpm.attention(q, kk, vv))
      if not next(iter(cpm._fused.values()))["k_all"].multicast_ptr:
        cp_mc = {"unavailable": "no multicast mapping on this platform"}
        break
      cp_mc[str(cop)] = t
  sk = s_loc * world
  flops5 = 4.0 * s_loc * sk * hq * hd / 2          # causal, zig-zag balanced: half of the score matrix
  link5 = (world - 1) * s_loc * hkv * hd * 2 * 2
  roof5 = max(flops5 / (peak * 1e12), link5 / (NVLINK_GBS * 1e9)) * 1e3
  best5 = min([v for v in cp_mc.values() if isinstance(v, float)], default=None)
  out["cp_attention_fwd"] = {"fused_multicast_ms_by_copiers": cp_mc,
                             "fraction_of_roofline_multicast": roof5 / best5 if best5 else None,
                             "fused_ms": t_cp_fused, "nccl_allgather_then_attention_ms": t_cp_nccl,
                             "roofline_ms": roof5, "fraction_of_roofline": roof5 / t_cp_fused,
                             "nvlink_bytes_in": link5, "keys_per_rank": s_loc}
  # ---- F4: expert-parallel MLP forward (Mixtral layer: 8 experts, top-2), dispatch/return by push kernel
  from torchprime_b200.parallel.ep import ExpertParallelMLP
  emesh = Mesh(shape={"data": 1, "fsdp": 1, "tensor": 1, "expert": world, "context": 1}, rank=rank, world_size=world)
  E, topk, Tm = 8, 2, 8192
  el = E // world
  wg = (torch.randn(el, D, F, device=dev) * 0.02).to(torch.bfloat16)
  wu = (torch.randn(el, D, F, device=dev) * 0.02).to(torch.bfloat16)
  wd = (torch.randn(el, F, D, device=dev) * 0.02).to(torch.bfloat16)
  xm = torch.randn(Tm, D, device=dev, dtype=torch.bfloat16)
  gidx = torch.stack([torch.randperm(E, device=dev)[:topk] for _ in range(Tm)]).to(torch.int32)
  gw = torch.rand(Tm, topk, device=dev)
  ep_nccl = ExpertParallelMLP(emesh, E, fused_exchange=False)
  ep_push = ExpertParallelMLP(emesh, E, fused_exchange=True)
  with torch.no_grad():
    t_ep_nccl = timed(lambda: ep_nccl.grouped_mlp(xm, gw, gidx, wg, wu, wd))
    t_ep_push = timed(lambda: ep_push.grouped_mlp(xm, gw, gidx, wg, wu, wd))
  flops4 = 2.0 * Tm * topk * 3 * D * F
  link4 = 2.0 * Tm * topk * D * 2 * (world - 1) / world        # rows out and back, remote fraction
  roof4 = max(flops4 / (peak * 1e12), link4 / (NVLINK_GBS * 1e9)) * 1e3
  out["ep_mlp_fwd"] = {"push_ms": t_ep_push, "nccl_all_to_all_ms": t_ep_nccl, "roofline_ms": roof4,
                       "fraction_of_roofline": roof4 / t_ep_push, "nvlink_bytes_each_way": link4 / 2}
  torch.cuda.synchronize()
  _lib.raise_on_device_timeout()
  if rank == 0:
    print(json.dumps({"world": world, "peak_tflops_used": peak, **out}))
  rt.barrier()
  rt.shutdown()


if __name__ == "__main__":
  main()
