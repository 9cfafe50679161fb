"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from torchprime_b200.ops import reference as ref


def _rel_err(got, want):
  got, want = got.float(), want.float()
  return ((got - want).norm() / (want.norm() + 1e-12)).item()


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (384, 768, 320), (130, 264, 72), (1024, 4096, 1024), (77, 40, 200)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(cuda_lib, M, N, K, a_mn, b_mn):
  from torchprime_b200.ops import kernels as k
  if (a_mn and M % 8) or (b_mn and N % 8) or K % 8:
    pytest.skip("leading dimension must be a multiple of 8 elements")
  torch.manual_seed(0)
  A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
  B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
  a_arg = A.t().contiguous() if a_mn else A
  b_arg = B.t().contiguous() if b_mn else B
  want = A.float() @ B.float().t()
  got = k.gemm(a_arg, b_arg, a_mn=a_mn, b_mn=b_mn, epi=k.EPI_F32)
  torch.cuda.synchronize()
  assert _rel_err(got, want) < 2e-3, _rel_err(got, want)
  got16 = k.gemm(a_arg, b_arg, a_mn=a_mn, b_mn=b_mn, epi=k.EPI_BF16)
  assert _rel_err(got16, want) < 1e-2


def test_gemm_epilogues(cuda_lib):
  from torchprime_b200.ops import kernels as k
  torch.manual_seed(1)
  M, N, K = 300, 520, 192
  A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
  B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
  want = A.float() @ B.float().t()
  acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
  got = k.gemm(A, B, out=acc.clone(), epi=k.EPI_F32_ACC, alpha=0.5)
  assert _rel_err(got, acc + 0.5 * want) < 2e-3
  acc16 = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
  got = k.gemm(A, B, out=acc16.clone(), epi=k.EPI_BF16_ACC)
  assert _rel_err(got, acc16.float() + want) < 1e-2
  res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
  got = k.gemm(A, B, epi=k.EPI_BF16_RES, aux=res)
  assert _rel_err(got, res.float() + want) < 1e-2


@pytest.mark.parametrize("M,F,K", [(256, 384, 128), (200, 136, 96)])
def test_gemm_swiglu(cuda_lib, M, F, K):
  from torchprime_b200.ops import kernels as k
  torch.manual_seed(2)
  A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
  W = (torch.randn(2 * F, K, device="cuda") / math.sqrt(K)).to(torch.bfloat16)
  gu = A.float() @ W.float().t()
  want = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
  c2 = torch.empty(M, 2 * F, device="cuda", dtype=torch.bfloat16)
  got = k.gemm(A, W, epi=k.EPI_SWIGLU, c2=c2)
  assert got.shape == (M, F)
  assert _rel_err(got, want) < 1.5e-2
  assert _rel_err(c2, gu) < 1e-2


# the larger row counts take the backward that streams its rows through shared memory by bulk copies
@pytest.mark.parametrize("rows,dim", [(64, 512), (1000, 4096), (33, 2048), (16, 8192), (4099, 4096), (3001, 2048),
                                      (2500, 8192), (5003, 520)])
def test_rmsnorm(cuda_lib, rows, dim):
  from torchprime_b200.ops import kernels as k
  torch.manual_seed(3)
  x = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
  r = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
  w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(torch.bfloat16)
  y, rstd, _ = k.rmsnorm_fwd(x, w, 1e-5)
  want = ref.rms_norm(x.float(), w.float(), 1e-5)
  assert _rel_err(y, want) < 1e-2
  y2, rstd2, h = k.rmsnorm_fwd(x, w, 1e-5, res=r, want_h=True)
  hw = (x + r)
  assert torch.equal(h, hw)
  assert _rel_err(y2, ref.rms_norm(hw.float(), w.float(), 1e-5)) < 1e-2
  # backward against autograd of the fp32 reference
  xf = x.float().requires_grad_(True)
  wf = w.float().requires_grad_(True)
  dy = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
  ref.rms_norm(xf, wf, 1e-5).backward(dy.float())
  dres = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
  dx, dw = k.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
  assert _rel_err(dx, xf.grad + dres.float()) < 1e-2
  assert _rel_err(dw, wf.grad) < 1e-2
  dx2, dw2 = k.rmsnorm_bwd(dy, x, w, rstd)
  assert _rel_err(dx2, xf.grad) < 1e-2
  assert _rel_err(dw2, wf.grad) < 1e-2
  from torchprime_b200.ops import _lib
  torch.cuda.synchronize()
  _lib.raise_on_device_timeout()


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope(cuda_lib, interleaved):
  from torchprime_b200.ops import kernels as k
  torch.manual_seed(4)
  B, S, H, D = 2, 48, 6, 128
  x = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16)
  inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
  ang = torch.arange(S, device="cuda").float()[:, None] * inv[None]
  cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
  cos_full, sin_full = torch.cat([cos, cos], -1), torch.cat([sin, sin], -1)
  buf = torch.zeros(B * S, 16 + H * D, device="cuda", dtype=torch.bfloat16)
  buf[:, 16:] = x.reshape(B * S, H * D)
  k.rope_(buf, 16, H, D, cos, sin, S, interleaved=interleaved)
  got = buf[:, 16:].reshape(B, S, H, D)
  if not interleaved:
    want = ref.rope_apply(x.float(), cos_full, sin_full)
  else:
    half = ref.rope_apply_interleaved(x.float(), cos_full, sin_full)
    want = torch.stack([half[..., : D // 2], half[..., D // 2:]], dim=-1).reshape(B, S, H, D)
  assert _rel_err(got, want) < 1e-2
  assert torch.equal(buf[:, :16], torch.zeros_like(buf[:, :16]))
  # inverse rotation restores the input
  k.rope_(buf, 16, H, D, cos, sin, S, inverse=True, interleaved=interleaved)
  assert _rel_err(buf[:, 16:].reshape(B, S, H, D), x) < 1.5e-2
  # explicit positions
  pos = torch.randint(0, S, (B * S,), device="cuda", dtype=torch.int32)
  buf2 = x.reshape(B * S, H * D).clone()
  k.rope_(buf2, 0, H, D, cos, sin, S, pos=pos)
  want = ref.rope_apply(x.float().reshape(1, B * S, H, D), cos_full[pos.long()], sin_full[pos.long()])
  assert _rel_err(buf2.reshape(1, B * S, H, D), want) < 1e-2


def test_swiglu(cuda_lib):
  from torchprime_b200.ops import kernels as k
  torch.manual_seed(5)
  gu = torch.randn(100, 2 * 264, device="cuda", dtype=torch.bfloat16)
  got = k.swiglu_fwd(gu)
  guf = gu.float().requires_grad_(True)
  want = ref.swiglu(guf)
  assert _rel_err(got, want) < 1e-2
  d = torch.randn_like(got)
  want.backward(d.float())
  assert _rel_err(k.swiglu_bwd(d, gu), guf.grad) < 1e-2


@pytest.mark.parametrize("rows,vocab", [(64, 1024), (37, 32000), (16, 128256)])
def test_cross_entropy(cuda_lib, rows, vocab):
  from torchprime_b200.ops import kernels as k
  torch.manual_seed(6)
  logits = (3 * torch.randn(rows, vocab, device="cuda")).to(torch.bfloat16)
  tgt = torch.randint(0, vocab, (rows,), device="cuda")
  tgt[::5] = -100
  lf = logits.float().requires_grad_(True)
  want = torch.nn.functional.cross_entropy(lf, tgt, ignore_index=-100, reduction="sum")
  want.backward()
  loss = torch.zeros(1, device="cuda")
  scale = torch.full((1,), 0.25, device="cuda")
  g = k.ce_fwd_bwd_(logits.clone(), tgt, loss, scale)
  assert abs(loss.item() - want.item()) / abs(want.item()) < 2e-3
  assert _rel_err(g, 0.25 * lf.grad) < 2e-2


def test_adamw_and_norm(cuda_lib):
  from torchprime_b200.ops import kernels as k
  torch.manual_seed(7)
  n = 1 << 20
  p = torch.randn(n, device="cuda")
  g = torch.randn(n, device="cuda").to(torch.bfloat16)
  m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
  p_ref = torch.nn.Parameter(p.clone())
  opt = torch.optim.AdamW([p_ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
  p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
  for step in (1, 2, 3):
    p_ref.grad = g.float() * 0.5
    opt.step()
    coef = torch.full((1,), 0.5, device="cuda")
    k.adamw_(p, m, v, g, p16, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, clip_coef=coef)
  assert _rel_err(p, p_ref.data) < 1e-5
  assert torch.equal(p16, p.to(torch.bfloat16))
  out = torch.zeros(1, device="cuda")
  k.sumsq_(g, out)
  assert abs(out.item() - g.float().pow(2).sum().item()) / out.item() < 1e-4
  out32 = torch.zeros(1, device="cuda")
  k.sumsq_(p[: n - 3], out32)
  assert abs(out32.item() - p[: n - 3].pow(2).sum().item()) / out32.item() < 1e-4
  coef, norm = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
  k.clip_coef_(out, 1.0, coef, norm)
  assert abs(norm.item() - math.sqrt(out.item())) < 1e-2 * norm.item()
  assert abs(coef.item() - 1.0 / norm.item()) < 1e-3


def test_embedding(cuda_lib):
  from torchprime_b200.ops import kernels as k
  torch.manual_seed(8)
  V, D = 1000, 256
  table = torch.randn(V, D, device="cuda", dtype=torch.bfloat16)
  ids = torch.randint(0, V, (4, 33), device="cuda")
  out = k.embedding_fwd(table, ids)
  assert torch.equal(out, table[ids])
  dout = torch.randn(4, 33, D, device="cuda", dtype=torch.bfloat16)
  dt = torch.zeros(V, D, device="cuda", dtype=torch.float32)
  k.embedding_bwd_(dout, ids, dt)
  want = torch.zeros(V, D, device="cuda").index_add_(0, ids.reshape(-1), dout.reshape(-1, D).float())
  assert _rel_err(dt, want) < 1e-5
  # sharded table: rows [250, 500)
  dts = torch.zeros(250, D, device="cuda", dtype=torch.float32)
  k.embedding_bwd_(dout, ids, dts, row0=250)
  assert _rel_err(dts, want[250:500]) < 1e-5


def test_tensor_kernels_are_bit_reproducible(cuda_lib):
  """Two runs of the GEMM and of the attention forward and backward give identical bits: no result
  depends on the order in which CTAs or atomics happen to run (a missing fence or a racy barrier
  protocol shows up here as a flaky mismatch)."""
  import torch
  from torchprime_b200.ops import attention_sm100 as A
  from torchprime_b200.ops import kernels as k
  torch.manual_seed(3)
  a = torch.randn(1024, 768, device="cuda", dtype=torch.bfloat16)
  b = torch.randn(1280, 768, device="cuda", dtype=torch.bfloat16)
  outs = [k.gemm(a, b).clone() for _ in range(3)]
  assert all(torch.equal(outs[0], o) for o in outs[1:])
  w = [k.gemm(a.t().contiguous(), b.t().contiguous()[:, :1024].contiguous(), a_mn=True, b_mn=True,
              epi=k.EPI_F32).clone() for _ in range(2)]
  assert torch.equal(w[0], w[1])
  qkv = torch.randn(2, 640, (8 + 2 * 2) * 128, device="cuda", dtype=torch.bfloat16)
  q = qkv[..., : 8 * 128].view(2, 640, 8, 128)
  kk = qkv[..., 8 * 128: 10 * 128].view(2, 640, 2, 128)
  v = qkv[..., 10 * 128:].view(2, 640, 2, 128)
  res = []
  for _ in range(2):
    o, lse = A.attn_fwd(q, kk, v, causal=True)
    do = torch.ones_like(o) * 0.01
    dq, dk, dv = A.attn_bwd(do, q, kk, v, o, lse, causal=True)
    res.append((o.clone(), lse.clone(), dq.clone(), dk.clone(), dv.clone()))
  for x, y in zip(res[0], res[1]):
    assert torch.equal(x, y)


def test_symmetric_runtime_single_rank(cuda_lib):
  """Allocation, the signal-pad barrier with one rank, the copy helper and release of the C++
  symmetric-memory runtime (the multi-rank mapping is covered by the two-GPU test)."""
  import ctypes
  import torch
  from torchprime_b200.dist import symm
  from torchprime_b200.ops import _lib
  L = symm._native_lib()
  assert L is not None
  before = L.tpb_symm_live_segments()
  payload, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
  assert L.tpb_symm_alloc(4096, ctypes.byref(payload), handle) == 0
  assert payload.value % 256 == 0 and handle.raw != b"\0" * 64
  assert L.tpb_symm_live_segments() == before + 1
  t = torch.as_tensor(symm._DeviceMemoryView(payload.value, 4096), device="cuda").view(torch.float32)
  assert float(t.abs().sum()) == 0.0                       # segments start zeroed
  t.copy_(torch.arange(1024, device="cuda", dtype=torch.float32))
  table = (ctypes.c_void_p * 1)(payload.value)
  for epoch in (1, 2, 3):
    assert L.tpb_symm_barrier(table, 0, 1, epoch, _lib.stream_ptr()) == 0
  out = torch.empty(1024, device="cuda")
  assert L.tpb_symm_copy(out.data_ptr(), payload.value, 4096, _lib.stream_ptr()) == 0
  torch.cuda.synchronize()
  assert torch.equal(out, torch.arange(1024, device="cuda", dtype=torch.float32))
  _lib.raise_on_device_timeout()
  del t
  assert L.tpb_symm_release(payload) == 0 and L.tpb_symm_live_segments() == before
  assert L.tpb_symm_release(payload) == -2                 # unknown segment
  assert L.tpb_symm_barrier(table, 1, 1, 1, _lib.stream_ptr()) == -2


def test_embedding_lookup_from_sharded_table(cuda_lib):
  """Rows read vector by vector from the shard that owns them (here three shards on one GPU; in training
  the shards are the fsdp ranks' peer-mapped parameter buffers).  Shard boundaries cut rows."""
  import ctypes
  from torchprime_b200.ops._lib import check, lib, ptr, stream_ptr
  from torchprime_b200.parallel import fsdp_comm  # noqa: F401  (registers the C signature)
  torch.manual_seed(3)
  vocab, dim, offset, world = 1000, 136, 48, 3
  table = torch.randn(vocab, dim, device="cuda", dtype=torch.bfloat16)
  total = offset + vocab * dim + 40
  shard = (total + world * 8 - 1) // (world * 8) * 8
  flat = torch.zeros(shard * world, device="cuda", dtype=torch.bfloat16)
  flat[offset:offset + vocab * dim] = table.reshape(-1)
  shards = [flat[r * shard:(r + 1) * shard].clone() for r in range(world)]
  assert (shard % dim) != 0                                  # rows straddle owners
  ids = torch.randint(0, vocab, (4, 77), device="cuda")
  ids[0, 0], ids[0, 1] = 0, vocab - 1
  out = torch.empty(ids.numel(), dim, device="cuda", dtype=torch.bfloat16)
  arr = (ctypes.c_void_p * world)(*[s.data_ptr() for s in shards])
  check(lib().tpb_embedding_fwd_peer(arr, world, shard, offset, ptr(ids.reshape(-1).contiguous()), ptr(out),
                                     ids.numel(), dim, vocab, stream_ptr()), "embedding_fwd_peer")
  torch.cuda.synchronize()
  assert torch.equal(out.view(4, 77, dim), table[ids])
