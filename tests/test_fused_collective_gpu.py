"""GEMM fused with all-gather / reduce-scatter over NVLink peer memory (needs >= 2 GPUs)."""

import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
  os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                     "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0",
                     "TPB_SYMM_STRICT": "1"})      # the native symmetric-memory runtime, no silent fallback
  sys.path.insert(0, ROOT)
  import torch.distributed as dist
  from torchprime_b200.dist import runtime as rt
  from torchprime_b200.dist.symm import SymmetricBuffer
  from torchprime_b200.ops import _lib, fused_collective as fc, kernels as k
  dev = rt.init()
  try:
    # ---- symmetric-memory runtime: peers see each other's writes after the device barrier
    from torchprime_b200.dist import symm
    for backend in ("native", "torch"):
      t = SymmetricBuffer(1024, torch.float32, dev, backend=backend)
      assert t.backend == backend and t.local.numel() == 1024 and len(set(t.ptrs)) == world
      for it in range(3):
        t.local.fill_(float(10 * it + rank))
        t.barrier()
        peer = (rank + 1) % world
        got = torch.empty(1024, device=dev)
        t.copy_from_rank(got, peer)                # copy engine, through the mapped pointer
        torch.cuda.synchronize()
        assert torch.all(got == float(10 * it + peer)), f"{backend}: peer copy not visible after the barrier"
        t.barrier()                                # nobody overwrites before everyone has read
      if backend == "native":
        before = symm.live_native_segments()
        t.close()
        assert symm.live_native_segments() == before - world
    torch.manual_seed(0)
    N, K, M = 1536, 512, 640
    extra = 4096 + 8 * 13                       # other tensors of the "unit" after the weight
    total = N * K + extra
    shard = (total + world * 8 - 1) // (world * 8) * 8
    full = torch.zeros(shard * world, dtype=torch.bfloat16, device=dev)
    full[:total] = (torch.randn(total, device=dev) * 0.05).to(torch.bfloat16)   # same on every rank (seed)
    sb = SymmetricBuffer(shard, torch.bfloat16, dev)
    sb.local.copy_(full[rank * shard:(rank + 1) * shard])
    torch.manual_seed(100 + rank)
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    gathered = torch.empty(shard * world, dtype=torch.bfloat16, device=dev)
    ag = fc.AllGatherGemm(sb, shard, copiers=4, push=False)
    for it in range(2):                          # twice: epochs, reuse of flags
      gathered.zero_()
      sb.barrier()
      y = ag(x, gathered, 0, N, K)
      torch.cuda.synchronize()
      sb.barrier()
      want = x.float() @ full[:N * K].view(N, K).float().t()
      err = ((y.float() - want).norm() / want.norm()).item()
      assert err < 1e-2, f"ag_gemm rel err {err}"
      assert torch.equal(gathered, full), "gathered buffer differs from the concatenated shards"
    # ---- push mode: every rank sends its shard, flags are raised in the peers' memory; with per-peer
    # stores and, where the switch offers it, with one multicast store for all peers
    for mc in (False, True):
      agp = fc.AllGatherGemm(sb, shard, copiers=4, push=True, multicast=mc)
      assert mc or agp.multicast_ptr == 0
      results[f"multicast_{rank}"] = bool(agp.multicast_ptr)
      for it in range(2):
        agp.gathered.zero_()
        torch.cuda.synchronize()
        sb.barrier()
        y = agp(x, None, 0, N, K)
        torch.cuda.synchronize()
        sb.barrier()
        torch.cuda.synchronize()
        err = ((y.float() - want).norm() / want.norm()).item()
        assert err < 1e-2, f"ag_gemm (push, multicast={mc}) rel err {err}"
        assert torch.equal(agp.gathered, full), f"pushed gathered buffer differs (multicast={mc})"
    # ---- reduce-scatter fused into a wgrad-layout GEMM
    T, Nw, Kw = 768, 512, 256
    c_off = 8 * 5
    tot2 = c_off + Nw * Kw + 64
    shard2 = (tot2 + world * 8 - 1) // (world * 8) * 8
    gs = SymmetricBuffer(shard2, torch.bfloat16, dev)
    dy = torch.randn(T, Nw, device=dev, dtype=torch.bfloat16)
    xx = torch.randn(T, Kw, device=dev, dtype=torch.bfloat16)
    part = (dy.float().t() @ xx.float()) / world
    dist.all_reduce(part)
    for it in range(2):
      gs.local.zero_()
      gs.barrier()
      fc.gemm_rs(dy, xx, a_mn=True, b_mn=True, m=Nw, n=Kw, ldc=Kw, grad_shards=gs, shard_elems=shard2,
                 c_offset=c_off, alpha=1.0 / world)
      torch.cuda.synchronize()
      gs.barrier()
      torch.cuda.synchronize()
      flat = torch.zeros(shard2 * world, dtype=torch.float32, device=dev)
      flat[c_off:c_off + Nw * Kw] = part.reshape(-1)
      mine = flat[rank * shard2:(rank + 1) * shard2]
      err = ((gs.local.float() - mine).norm() / (mine.norm() + 1e-9)).item()
      assert err < 2e-2, f"gemm_rs rel err {err}"
    # ---- tensor-parallel all-reduce inside the GEMM epilogue (multimem.red through the multicast mapping)
    ar = fc.AllReduceGemm(dist.group.WORLD, dev)
    Ma, Na, Ka = 640, 256, 512
    torch.manual_seed(7)
    res_ar = torch.randn(Ma, Na, device=dev).to(torch.bfloat16)          # the same residual on every rank
    torch.manual_seed(700 + rank)
    a_ar = torch.randn(Ma, Ka, device=dev).to(torch.bfloat16)
    w_ar = (torch.randn(Na, Ka, device=dev) * 0.05).to(torch.bfloat16)
    wt_ar = (torch.randn(Ka, Na, device=dev) * 0.05).to(torch.bfloat16)   # [K, N] storage (input-gradient layout)
    results[f"tp_multicast_{rank}"] = bool(ar.usable(Ma, Na, Ka))
    if ar.usable(Ma, Na, Ka):
      for it in range(2):                          # the buffer is zeroed and reused
        y = ar.gemm_allreduce(a_ar, w_ar, res_ar)
        want = a_ar.float() @ w_ar.float().t()
        dist.all_reduce(want)
        want += res_ar.float()
        err = ((y.float() - want).norm() / want.norm()).item()
        assert err < 1e-2, f"gemm_allreduce rel err {err}"
        y2 = ar.gemm_allreduce(a_ar, wt_ar, None, b_mn=True)
        want2 = a_ar.float() @ wt_ar.float()
        dist.all_reduce(want2)
        err2 = ((y2.float() - want2).norm() / want2.norm()).item()
        assert err2 < 1e-2, f"gemm_allreduce (transposed weight) rel err {err2}"
    # ---- context-parallel attention with the K/V exchange fused into the forward kernel
    from torchprime_b200.dist.mesh import Mesh
    from torchprime_b200.parallel.cp import ContextParallelAttention
    mesh = Mesh(shape={"data": 1, "fsdp": 1, "tensor": 1, "expert": 1, "context": world}, rank=rank, world_size=world)
    for lb, mc in ((False, False), (True, True), (True, False)):
      ref_cp = ContextParallelAttention(mesh, load_balanced=lb, fused_exchange=False)
      fus_cp = ContextParallelAttention(mesh, load_balanced=lb, fused_exchange=True, fused_copiers=4,
                                        fused_multicast=mc)
      torch.manual_seed(500 + rank)
      b, s_loc, hq, hkv, d = 2, 512, 8, 2, 128
      qkv = (torch.randn(b, s_loc, (hq + 2 * hkv) * d, device=dev) * 0.5).to(torch.bfloat16)
      dout = (torch.randn(b, s_loc, hq, d, device=dev) * 0.1).to(torch.bfloat16)
      outs = []
      for cpa in (ref_cp, fus_cp):
        x = qkv.clone().requires_grad_(True)
        q = x[..., :hq * d].view(b, s_loc, hq, d)
        k = x[..., hq * d:(hq + hkv) * d].view(b, s_loc, hkv, d)
        v = x[..., (hq + hkv) * d:].view(b, s_loc, hkv, d)
        for _ in range(2):                       # twice: buffers and flags are reused with a new epoch
          x.grad = None
          o = cpa.attention(q, k, v)
          o.backward(dout)
        torch.cuda.synchronize()
        outs.append((o.detach().float(), x.grad.float()))
      (o_ref, g_ref), (o_fus, g_fus) = outs
      assert fus_cp._fused, "the fused exchange path was not taken"
      err_o = ((o_fus - o_ref).norm() / o_ref.norm()).item()
      err_g = ((g_fus - g_ref).norm() / g_ref.norm()).item()
      assert err_o < 1e-2 and err_g < 2e-2, f"fused cp attention (lb={lb}, multicast={mc}): out {err_o} grad {err_g}"
    # ---- expert-parallel MLP with dispatch / return by the push all-to-all kernel
    from torchprime_b200.parallel.ep import ExpertParallelMLP
    emesh = Mesh(shape={"data": 1, "fsdp": 1, "tensor": 1, "expert": world, "context": 1}, rank=rank, world_size=world)
    E, K_top, T, Dm, Fm = 4, 2, 384, 256, 512
    el = E // world
    torch.manual_seed(900)                        # the same experts everywhere, each rank keeps its slice
    wg_all = (torch.randn(E, Dm, Fm, device=dev) * 0.05).to(torch.bfloat16)
    wu_all = (torch.randn(E, Dm, Fm, device=dev) * 0.05).to(torch.bfloat16)
    wd_all = (torch.randn(E, Fm, Dm, device=dev) * 0.05).to(torch.bfloat16)
    torch.manual_seed(950 + rank)
    xt = torch.randn(T, Dm, device=dev).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device=dev)[:K_top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, K_top, device=dev)
    dy_ep = (torch.randn(T, Dm, device=dev) * 0.1).to(torch.bfloat16)
    res = []
    for fused in (False, True):
      epm = ExpertParallelMLP(emesh, E, fused_exchange=fused)
      xx2 = xt.clone().requires_grad_(True)
      ws = [w[rank * el:(rank + 1) * el].clone().requires_grad_(True) for w in (wg_all, wu_all, wd_all)]
      for _ in range(2):                          # buffers, flags and epochs are reused
        xx2.grad = None
        for w in ws:
          w.grad = None
        y = epm.grouped_mlp(xx2, wts, idx, ws[0], ws[1], ws[2])
        y.backward(dy_ep)
      torch.cuda.synchronize()
      res.append((y.detach().float(), xx2.grad.float(), ws[0].grad.float(), ws[2].grad.float()))
      if fused:
        assert epm._push, "the push all-to-all path was not taken"
    for a_, b_, name in zip(res[0], res[1], ("out", "dx", "dw_gate", "dw_down")):
      err = ((a_ - b_).norm() / (a_.norm() + 1e-9)).item()
      assert err < 2e-2, f"expert-parallel MLP with push all-to-all: {name} differs by {err}"
    _lib.raise_on_device_timeout()
    results[rank] = "ok"
  except Exception as e:  # noqa: BLE001
    import traceback
    results[rank] = "".join(traceback.format_exception(e))
  finally:
    rt.shutdown()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ag_gemm_and_gemm_rs_two_gpus(cuda_lib):
  import torch.multiprocessing as mp
  world = 2
  mgr = mp.Manager()
  results = mgr.dict()
  mp.spawn(_worker, args=(world, 29641, results), nprocs=world, join=True)
  assert all(results.get(r) == "ok" for r in range(world)), dict(results)
  print("multicast push used:", [results.get(f"multicast_{r}") for r in range(world)],
        "all-reduce in GEMM used:", [results.get(f"tp_multicast_{r}") for r in range(world)])
