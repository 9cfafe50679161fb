"""sm_100a flash attention (forward and backward) against the eager fp32 reference."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from torchprime_b200.ops import reference as ref


def _rel(got, want):
  return ((got.float() - want.float()).norm() / (want.float().norm() + 1e-12)).item()


def _qkv(b, s, hq, hkv, d, dv=128, fused=True, seed=0):
  torch.manual_seed(seed)
  if fused and d == dv:
    buf = torch.randn(b, s, (hq + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16)
    q = buf[..., : hq * d].view(b, s, hq, d)
    k = buf[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
    v = buf[..., (hq + hkv) * d:].view(b, s, hkv, d)
    return q, k, v
  q = torch.randn(b, s, hq, d, device="cuda", dtype=torch.bfloat16)
  k = torch.randn(b, s, hkv, d, device="cuda", dtype=torch.bfloat16)
  v = torch.randn(b, s, hkv, dv, device="cuda", dtype=torch.bfloat16)
  return q, k, v


FWD_CASES = [
  # b, s, hq, hkv, d, causal, window
  (1, 128, 1, 1, 128, True, None),
  (1, 256, 2, 1, 128, True, None),
  (2, 384, 4, 2, 128, True, None),
  (1, 200, 2, 2, 128, True, None),
  (1, 320, 2, 1, 128, False, None),
  (1, 1024, 4, 1, 128, True, None),
  (1, 512, 2, 1, 128, True, 100),
  (1, 256, 2, 2, 192, True, None),
  (2, 2048, 4, 2, 128, True, None),     # several batch rows at a length with many key blocks
  (1, 8192, 4, 1, 128, True, None),     # the training sequence length
]


@pytest.mark.parametrize("b,s,hq,hkv,d,causal,window", FWD_CASES)
def test_attention_forward(cuda_lib, b, s, hq, hkv, d, causal, window):
  from torchprime_b200.ops import attention_sm100 as A
  q, k, v = _qkv(b, s, hq, hkv, d)
  o, lse = A.attn_fwd(q, k, v, causal=causal, window=window)
  want, want_lse = ref.attention(q, k, v, causal=causal, window=window, return_lse=True)
  torch.cuda.synchronize()
  assert _rel(o, want) < 2e-2, _rel(o, want)
  assert torch.allclose(lse, want_lse, atol=2e-2, rtol=1e-3), (lse - want_lse).abs().max()


def test_attention_forward_segments_and_positions(cuda_lib):
  from torchprime_b200.ops import attention_sm100 as A
  b, s, hq, hkv, d = 2, 256, 2, 1, 128
  q, k, v = _qkv(b, s, hq, hkv, d, seed=3)
  seg = torch.zeros(b, s, dtype=torch.int32, device="cuda")
  seg[0, 100:] = 1
  seg[1, 30:200] = 1
  seg[1, 200:] = 2
  o, _ = A.attn_fwd(q, k, v, causal=True, q_seg=seg.reshape(-1).contiguous(), kv_seg=seg.reshape(-1).contiguous())
  want = ref.attention(q, k, v, causal=True, q_segment_ids=seg)
  assert _rel(o, want) < 2e-2
  # rows of a zig-zag context-parallel shard: queries are chunks 0 and 3 of 4, keys are all 4 chunks
  pos = torch.cat([torch.arange(0, 64), torch.arange(192, 256)]).to(torch.int32).cuda()
  qs = q[:, pos.long()].contiguous()
  o2, _ = A.attn_fwd(qs, k, v, causal=True, q_pos=pos.repeat(b).contiguous())
  want2 = ref.attention(qs, k, v, causal=True, q_positions=pos.long())
  assert _rel(o2, want2) < 2e-2


BWD_CASES = [
  (1, 128, 1, 1, 128, True, None),
  (1, 256, 4, 1, 128, True, None),
  (2, 384, 4, 2, 128, True, None),
  (1, 200, 2, 2, 128, True, None),
  (1, 320, 2, 1, 128, False, None),
  (1, 512, 2, 1, 128, True, 100),
  (1, 256, 2, 2, 192, True, None),
  (2, 2048, 4, 2, 128, True, None),
  (1, 8192, 2, 1, 128, True, None),     # the training sequence length
]


@pytest.mark.parametrize("b,s,hq,hkv,d,causal,window", BWD_CASES)
def test_attention_backward(cuda_lib, b, s, hq, hkv, d, causal, window):
  from torchprime_b200.ops import attention_sm100 as A
  q, k, v = _qkv(b, s, hq, hkv, d, fused=False, seed=5)
  do = torch.randn(b, s, hq, 128, device="cuda", dtype=torch.bfloat16)
  o, lse = A.attn_fwd(q, k, v, causal=causal, window=window)
  dq, dk, dv = A.attn_bwd(do, q, k, v, o, lse, causal=causal, window=window)
  qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
  ref.attention(qf, kf, vf, causal=causal, window=window).backward(do.float())
  torch.cuda.synchronize()
  assert _rel(dv, vf.grad) < 3e-2, ("dv", _rel(dv, vf.grad))
  assert _rel(dk, kf.grad) < 3e-2, ("dk", _rel(dk, kf.grad))
  assert _rel(dq, qf.grad) < 3e-2, ("dq", _rel(dq, qf.grad))


def test_attention_autograd_fused_qkv(cuda_lib):
  from torchprime_b200.ops import functional as ops
  b, s, hq, hkv, d = 1, 256, 4, 2, 128
  torch.manual_seed(9)
  buf = torch.randn(b, s, (hq + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
  q = buf[..., : hq * d].view(b, s, hq, d)
  k = buf[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
  v = buf[..., (hq + hkv) * d:].view(b, s, hkv, d)
  o = ops.attention(q, k, v, causal=True)
  assert ops.attention_impl_in_use().startswith("sm100")
  do = torch.randn_like(o)
  o.backward(do)
  bf = buf.detach().float().requires_grad_(True)
  qf = bf[..., : hq * d].view(b, s, hq, d)
  kf = bf[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
  vf = bf[..., (hq + hkv) * d:].view(b, s, hkv, d)
  ref.attention(qf, kf, vf, causal=True).backward(do.float())
  assert _rel(buf.grad, bf.grad) < 3e-2


@pytest.mark.parametrize("b,s,hq,hkv,causal,window,cap", [(1, 384, 4, 2, True, None, 2.0), (2, 300, 2, 1, True, 100, 5.0),
                                                          (1, 256, 2, 2, False, None, 1.0), (1, 1024, 4, 1, True, None, 30.0)])
def test_attention_logit_soft_cap(cuda_lib, b, s, hq, hkv, causal, window, cap):
  """Scores capped as cap * tanh(s / cap) inside the kernels, forward and backward (the reference's
  splash-attention option attn_logits_soft_cap, torchprime/utils/kernel_utils.py:30-37)."""
  from torchprime_b200.ops import attention_sm100 as A
  from torchprime_b200.ops import functional as ops
  q, k, v = _qkv(b, s, hq, hkv, 128, fused=False, seed=11)
  q = (q * 2).contiguous()       # scores well into the curved part of the cap
  do = torch.randn(b, s, hq, 128, device="cuda", dtype=torch.bfloat16)
  o, lse = A.attn_fwd(q, k, v, causal=causal, window=window, softcap=cap)
  want, want_lse = ref.attention(q, k, v, causal=causal, window=window, softcap=cap, return_lse=True)
  assert _rel(o, want) < 2e-2, _rel(o, want)
  assert torch.allclose(lse, want_lse, atol=2e-2, rtol=1e-3), (lse - want_lse).abs().max()
  dq, dk, dv = A.attn_bwd(do, q, k, v, o, lse, causal=causal, window=window, softcap=cap)
  qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
  ref.attention(qf, kf, vf, causal=causal, window=window, softcap=cap).backward(do.float())
  torch.cuda.synchronize()
  assert _rel(dv, vf.grad) < 3e-2, ("dv", _rel(dv, vf.grad))
  assert _rel(dk, kf.grad) < 3e-2, ("dk", _rel(dk, kf.grad))
  assert _rel(dq, qf.grad) < 3e-2, ("dq", _rel(dq, qf.grad))
  # the public op takes the kernel path too
  qa = q.clone().requires_grad_(True)
  oa = ops.attention(qa, k, v, causal=causal, window=window, softcap=cap)
  assert ops.attention_impl_in_use().startswith("sm100")
  oa.backward(do)
  assert _rel(qa.grad, qf.grad) < 3e-2
