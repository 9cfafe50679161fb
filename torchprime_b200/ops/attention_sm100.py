"""Python side of the sm_100a flash-attention kernels (csrc/attention_fwd_sm100.cu,
csrc/attention_bwd_sm100.cu): argument checking, launch and the autograd Function.

Tensors are token-major ``[B, S, H, D]`` views (for example slices of a fused QKV
projection): unit stride over D, stride D over heads, one row pitch per token and
batches laid out back to back.  Supported: head dim 128 (and 192 for q/k with 128 for v:
the MLA shape), bf16, GQA, causal / full / sliding-window masks, segment ids, explicit
query positions (context-parallel shards).
"""

from __future__ import annotations

import math
from ctypes import c_uint, c_float, c_int, c_longlong, c_void_p

import torch

from . import _lib
from ._lib import check, lib, ptr, stream_ptr

P, I, LL, F = c_void_p, c_int, c_longlong, c_float
_lib.register_signature("tpb_attn_fwd", [P, P, P, P, P, I, I, I, I, I, I, I, LL, LL, LL, LL, F, I, I, P, P, P, P])
_lib.register_signature("tpb_attn_bwd", [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, LL, LL, LL, LL, LL,
                                         LL, LL, F, I, I, P, P, P, P])
# the same with a logit soft cap (a float before the stream)
_lib.register_signature("tpb_attn_fwd_softcap", [P, P, P, P, P, I, I, I, I, I, I, I, LL, LL, LL, LL, F, I, I, P, P, P, F,
                                                 P])
_lib.register_signature("tpb_attn_bwd_softcap", [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, LL, LL, LL, LL, LL,
                                                 LL, LL, F, I, I, P, P, P, F, P])


_lib.register_signature("tpb_attn_fwd_cp", [P, P, P, P, P, P, P, P, I, I, I, I, I, LL, LL, LL, LL, F, P, I, I, I, I,
                                            c_uint, P, P, P])


def attn_fwd_cp(q, k_local, v_local, k_all_sb, v_all_sb, flags_sb, q_pos, *, zigzag: bool, epoch: int,
                copiers: int = 16, scale=None, multicast: bool = True):
  """Causal attention forward with the context-parallel K/V exchange fused into the kernel.

  ``q`` [B,Sq,Hq,128] are this rank's query rows, ``k_local`` / ``v_local`` [B,S_local,Hkv,128] its
  keys and values; ``k_all_sb`` / ``v_all_sb`` / ``flags_sb`` are ``SymmetricBuffer`` objects that
  hold the gathered K, V ([B, world*S_local, Hkv, 128], natural key order) and one flag per 128
  keys.  Copier CTAs push the local rows into every rank's buffers while the other CTAs compute
  (with one ``multimem.st`` for all ranks when both buffers have a multicast mapping and
  ``multicast`` is on, else with one store per rank).
  Returns (o, lse); afterwards ``k_all_sb.local`` / ``v_all_sb.local`` hold the gathered tensors."""
  b, sq, hq, d = q.shape
  s_local, hkv = k_local.shape[1], k_local.shape[2]
  assert d == 128 and v_local.shape[-1] == 128 and _token_major(q) and _token_major(k_local) and _token_major(v_local)
  scale = scale if scale is not None else 1.0 / math.sqrt(d)
  o = torch.empty(b, sq, hq, 128, dtype=q.dtype, device=q.device)
  lse = torch.empty(b, hq, sq, dtype=torch.float32, device=q.device)
  rc = lib().tpb_attn_fwd_cp(ptr(q), ptr(k_local), ptr(v_local), k_all_sb.ptr_table(), v_all_sb.ptr_table(),
                             flags_sb.ptr_table(), ptr(o), ptr(lse), b, sq, s_local, hq, hkv, q.stride(1),
                             k_local.stride(1), v_local.stride(1), hq * 128, float(scale), ptr(q_pos),
                             k_all_sb.world, k_all_sb.rank, int(bool(zigzag)), int(copiers), int(epoch),
                             (k_all_sb.multicast_ptr or None) if multicast else None,
                             (v_all_sb.multicast_ptr or None) if multicast else None, stream_ptr())
  check(rc, f"attn_fwd_cp q{tuple(q.shape)} k{tuple(k_local.shape)} world={k_all_sb.world}")
  return o, lse


def _token_major(t: torch.Tensor) -> bool:
  b, s, h, d = t.shape
  return (t.stride(3) == 1 and t.stride(2) == d and t.stride(1) % 8 == 0 and (b == 1 or t.stride(0) == s * t.stride(1))
          and t.data_ptr() % 16 == 0)


def supported(q, k, v, causal, window, q_segment_ids, softcap, q_positions, kv_positions) -> bool:
  if kv_positions is not None:
    return False
  if softcap and (softcap <= 0 or q.shape[-1] != 128):   # the capped backward exists for head dim 128 only
    return False
  if q.dtype != torch.bfloat16 or not (q.is_cuda and k.is_cuda and v.is_cuda):
    return False
  dq, dv = q.shape[-1], v.shape[-1]
  if dv != 128 or dq not in (128, 192) or k.shape[-1] != dq:
    return False
  if q.shape[2] % k.shape[2] != 0 or k.shape[2] != v.shape[2]:
    return False
  return _token_major(q) and _token_major(k) and _token_major(v)


def _i32(t):
  return None if t is None else t.reshape(-1).to(torch.int32).contiguous()


def attn_fwd(q, k, v, causal=True, scale=None, window=None, q_pos=None, q_seg=None, kv_seg=None, softcap=None):
  """Returns (o [B,Sq,Hq,128] contiguous, lse [B,Hq,Sq] fp32 in natural-log units).  ``softcap``: the scores
  become ``softcap * tanh(q.k * scale / softcap)`` before the softmax."""
  b, sq, hq, dqk = q.shape
  sk, hkv, dv = k.shape[1], k.shape[2], v.shape[-1]
  scale = scale if scale is not None else 1.0 / math.sqrt(dqk)
  o = torch.empty(b, sq, hq, dv, dtype=q.dtype, device=q.device)
  lse = torch.empty(b, hq, sq, dtype=torch.float32, device=q.device)
  rc = lib().tpb_attn_fwd_softcap(ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), b, sq, sk, hq, hkv, dqk, dv, q.stride(1),
                                  k.stride(1), v.stride(1), hq * dv, float(scale), int(bool(causal)),
                                  int(window or 0), ptr(q_pos), ptr(q_seg), ptr(kv_seg), float(softcap or 0.0),
                                  stream_ptr())
  check(rc, f"attn_fwd q{tuple(q.shape)} k{tuple(k.shape)}")
  return o, lse


def attn_bwd(do, q, k, v, o, lse, causal=True, scale=None, window=None, q_pos=None, q_seg=None, kv_seg=None,
             dq=None, dk=None, dv=None, softcap=None):
  """Gradients of :func:`attn_fwd`.  dq/dk/dv may be preallocated token-major views (for
  example slices of one fused dQKV buffer); they are fully overwritten."""
  b, sq, hq, dqk = q.shape
  sk, hkv, dvd = k.shape[1], k.shape[2], v.shape[-1]
  scale = scale if scale is not None else 1.0 / math.sqrt(dqk)
  dq = torch.empty(b, sq, hq, dqk, dtype=q.dtype, device=q.device) if dq is None else dq
  dk = torch.empty(b, sk, hkv, dqk, dtype=q.dtype, device=q.device) if dk is None else dk
  dv = torch.empty(b, sk, hkv, dvd, dtype=q.dtype, device=q.device) if dv is None else dv
  do = do.contiguous()
  o = o.contiguous()
  if dqk != 128:
    assert not softcap, "the capped backward exists for head dim 128 only"
    return _eager_bwd(do, q, k, v, causal, scale, window, q_pos, q_seg, kv_seg, dq, dk, dv)
  scratch = torch.empty(2 * b * hq * ((sq + 127) // 128 * 128), dtype=torch.float32, device=q.device)
  rc = lib().tpb_attn_bwd_softcap(ptr(do), ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), ptr(scratch), ptr(dq),
                                  ptr(dk), ptr(dv), b, sq, sk, hq, hkv, dqk, dvd, q.stride(1), k.stride(1),
                                  v.stride(1), do.stride(1), dq.stride(1), dk.stride(1), dv.stride(1), float(scale),
                                  int(bool(causal)), int(window or 0), ptr(q_pos), ptr(q_seg), ptr(kv_seg),
                                  float(softcap or 0.0), stream_ptr())
  check(rc, f"attn_bwd q{tuple(q.shape)} k{tuple(k.shape)}")
  return dq, dk, dv


def _eager_bwd(do, q, k, v, causal, scale, window, q_pos, q_seg, kv_seg, dq, dk, dv):
  """Gradients for shapes the backward kernel does not cover yet (q/k head dim 192).  Plain causal
  or full attention goes through torch's scaled_dot_product_attention (a library call: forward is
  recomputed with autograd on); masks it cannot express fall back to the fp32 eager definition,
  one batch element at a time."""
  from . import reference as ref
  b, sq = q.shape[0], q.shape[1]
  sk = k.shape[1]
  if window is None and q_pos is None and q_seg is None and kv_seg is None and (not causal or sq == sk):
    try:
      with torch.enable_grad():
        qf, kf, vf = (t.detach().transpose(1, 2).requires_grad_(True) for t in (q, k, v))
        o = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=bool(causal), scale=scale,
                                                             enable_gqa=q.shape[2] != k.shape[2])
        gq, gk, gv = torch.autograd.grad(o, (qf, kf, vf), do.transpose(1, 2))
      dq.copy_(gq.transpose(1, 2)); dk.copy_(gk.transpose(1, 2)); dv.copy_(gv.transpose(1, 2))
      return dq, dk, dv
    except RuntimeError:
      pass   # no backend for this shape: use the eager definition below
  for i in range(b):
    with torch.enable_grad():
      qf, kf, vf = (t[i:i + 1].detach().float().requires_grad_(True) for t in (q, k, v))
      o = ref.attention(
        qf, kf, vf, causal=causal, scale=scale, window=window,
        q_segment_ids=None if q_seg is None else q_seg.view(b, sq)[i:i + 1],
        kv_segment_ids=None if kv_seg is None else kv_seg.view(b, sk)[i:i + 1],
        q_positions=None if q_pos is None else q_pos.view(b, sq)[i:i + 1].long())
      gq, gk, gv = torch.autograd.grad(o, (qf, kf, vf), do[i:i + 1].float())
    dq[i:i + 1].copy_(gq)
    dk[i:i + 1].copy_(gk)
    dv[i:i + 1].copy_(gv)
  return dq, dk, dv


class _AttentionFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, q, k, v, causal, scale, window, q_pos, q_seg, kv_seg, softcap=None):
    o, lse = attn_fwd(q, k, v, causal, scale, window, q_pos, q_seg, kv_seg, softcap)
    ctx.save_for_backward(q, k, v, o, lse, q_pos, q_seg, kv_seg)
    ctx.args = (causal, scale, window, softcap)
    return o

  @staticmethod
  def backward(ctx, do):
    q, k, v, o, lse, q_pos, q_seg, kv_seg = ctx.saved_tensors
    causal, scale, window, softcap = ctx.args
    dq = dk = dv = None
    fused = _fused_qkv_layout(q, k, v)
    if fused is not None:
      # q, k, v are column slices of one [B, S, (Hq + 2 Hkv) * D] projection: write the three
      # gradients into the matching slices of one buffer so autograd's slice-backward can
      # hand the GEMM a single contiguous dQKV.
      b, s, hq, d = q.shape
      hkv = k.shape[2]
      buf = torch.empty(b, s, (hq + 2 * hkv) * d, dtype=q.dtype, device=q.device)
      dq = buf[..., : hq * d].view(b, s, hq, d)
      dk = buf[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
      dv = buf[..., (hq + hkv) * d:].view(b, s, hkv, d)
    dq, dk, dv = attn_bwd(do, q, k, v, o, lse, causal, scale, window, q_pos, q_seg, kv_seg, dq, dk, dv, softcap)
    return dq, dk, dv, None, None, None, None, None, None, None


class _AttentionQKVFn(torch.autograd.Function):
  """Attention on one fused projection output ``qkv`` [B, S, (Hq + 2 Hkv) * D] (queries, keys, values
  back to back in every row).  A single autograd input means a single gradient: the backward
  kernels write dQ, dK and dV into the column ranges of one buffer, which goes straight to the
  projection's GEMMs.  With three sliced inputs autograd would materialise each slice's gradient as
  a zero-filled full-width tensor and add the three (three fills, three copies and two adds of
  100 MB per layer)."""

  @staticmethod
  def forward(ctx, qkv, hq, hkv, d, causal, scale, window, q_pos, q_seg, kv_seg):
    b, s, _ = qkv.shape
    q = qkv[..., : hq * d].view(b, s, hq, d)
    k = qkv[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
    v = qkv[..., (hq + hkv) * d:].view(b, s, hkv, d)
    o, lse = attn_fwd(q, k, v, causal, scale, window, q_pos, q_seg, kv_seg)
    ctx.save_for_backward(qkv, o, lse, q_pos, q_seg, kv_seg)
    ctx.args = (hq, hkv, d, causal, scale, window)
    return o

  @staticmethod
  def backward(ctx, do):
    qkv, o, lse, q_pos, q_seg, kv_seg = ctx.saved_tensors
    hq, hkv, d, causal, scale, window = ctx.args
    b, s, _ = qkv.shape
    q = qkv[..., : hq * d].view(b, s, hq, d)
    k = qkv[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
    v = qkv[..., (hq + hkv) * d:].view(b, s, hkv, d)
    buf = torch.empty_like(qkv)
    dq = buf[..., : hq * d].view(b, s, hq, d)
    dk = buf[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
    dv = buf[..., (hq + hkv) * d:].view(b, s, hkv, d)
    attn_bwd(do, q, k, v, o, lse, causal, scale, window, q_pos, q_seg, kv_seg, dq, dk, dv)
    return buf, None, None, None, None, None, None, None, None, None


def attention_qkv(qkv, hq, hkv, d, causal=True, scale=None, window=None, q_segment_ids=None, q_positions=None):
  """Self-attention on a fused [B, S, (Hq + 2 Hkv) * D] projection (head dim 128, contiguous)."""
  seg = _i32(q_segment_ids)
  return _AttentionQKVFn.apply(qkv, hq, hkv, d, causal, scale, window, _i32(q_positions), seg, seg)


def _fused_qkv_layout(q, k, v):
  if q.shape[-1] != v.shape[-1] or q.shape[1] != k.shape[1]:
    return None
  same = (q.untyped_storage().data_ptr() == k.untyped_storage().data_ptr() == v.untyped_storage().data_ptr())
  if not same or not (q.stride(1) == k.stride(1) == v.stride(1)):
    return None
  hq, hkv, d = q.shape[2], k.shape[2], q.shape[3]
  if q.stride(1) != (hq + 2 * hkv) * d:
    return None
  if k.storage_offset() - q.storage_offset() != hq * d or v.storage_offset() - k.storage_offset() != hkv * d:
    return None
  return True


def attention(q, k, v, causal=True, scale=None, window=None, q_segment_ids=None, kv_segment_ids=None, softcap=None,
              q_positions=None, kv_positions=None):
  q_seg = _i32(q_segment_ids)
  kv_seg = _i32(kv_segment_ids if kv_segment_ids is not None else q_segment_ids)
  return _AttentionFn.apply(q, k, v, causal, scale, window, _i32(q_positions), q_seg, kv_seg, softcap)
