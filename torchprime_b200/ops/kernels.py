"""Raw (no-autograd) Python entry points of the sm_100a kernels.

Each function validates shapes/dtypes, launches on the current CUDA stream and
returns torch tensors.  The autograd-aware operators live in ``functional.py``.
"""

from __future__ import annotations

import torch

from . import _debug, _lib
from ._lib import (EPI_BF16, EPI_BF16_ACC, EPI_BF16_RES, EPI_F32, EPI_F32_ACC, EPI_SWIGLU, check, lib, ptr,
                   stream_ptr)

__all__ = [
  "gemm", "rmsnorm_fwd", "rmsnorm_bwd", "rope_", "swiglu_fwd", "swiglu_bwd", "ce_fwd_bwd_", "adamw_",
  "sumsq_", "clip_coef_", "embedding_fwd", "embedding_bwd_", "cast_f32_to_bf16_",
  "EPI_BF16", "EPI_F32", "EPI_F32_ACC", "EPI_BF16_ACC", "EPI_BF16_RES", "EPI_SWIGLU",
]


def launch_count() -> int:
  return _lib.launch_count()


def _row_major_2d(t: torch.Tensor, name: str):
  assert t.dim() == 2 and t.stride(1) == 1, f"{name} must be 2-D with unit inner stride, got {t.shape} {t.stride()}"
  return t.shape[0], t.shape[1], t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def gemm(a, b, *, a_mn=False, b_mn=False, out=None, epi=EPI_BF16, alpha=1.0, aux=None, c2=None, max_ctas=0):
  """C = alpha * A @ B^T with logical A [M,K], B [N,K].

  ``a_mn``/``b_mn`` say that the tensor passed is the transposed storage ([K,M]
  resp. [K,N]).  ``epi`` selects the fused epilogue (see csrc/tpb.h).  For
  ``EPI_SWIGLU`` B holds [gate; up] rows and the result has N/2 columns.
  """
  assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
  r0, r1, lda = _row_major_2d(a, "a")
  M, K = (r1, r0) if a_mn else (r0, r1)
  r0, r1, ldb = _row_major_2d(b, "b")
  N, Kb = (r1, r0) if b_mn else (r0, r1)
  assert K == Kb, f"contraction mismatch {K} vs {Kb}"
  n_out = N // 2 if epi == EPI_SWIGLU else N
  if out is None:
    assert epi not in (EPI_F32_ACC, EPI_BF16_ACC), "accumulating epilogues need `out`"
    dt = torch.float32 if epi == EPI_F32 else torch.bfloat16
    out = torch.empty(M, n_out, dtype=dt, device=a.device)
  assert out.shape[0] == M and out.shape[1] == n_out and out.stride(1) == 1
  want = torch.float32 if epi in (EPI_F32, EPI_F32_ACC) else torch.bfloat16
  assert out.dtype == want, f"epilogue {epi} writes {want}, out is {out.dtype}"
  ldc = out.stride(0) if M > 1 else max(out.stride(0), n_out)
  ldaux = 0
  if epi == EPI_BF16_RES:
    assert aux is not None and aux.shape == out.shape and aux.stride(1) == 1 and aux.dtype == torch.bfloat16
    ldaux = aux.stride(0) if M > 1 else max(aux.stride(0), n_out)
  ldc2 = 0
  if c2 is not None:
    assert epi == EPI_SWIGLU and c2.shape == (M, N) and c2.stride(1) == 1 and c2.dtype == torch.bfloat16
    ldc2 = c2.stride(0)
  rc = lib().tpb_gemm_bf16(ptr(a), ptr(b), ptr(out), M, N, K, lda, ldb, ldc, int(a_mn), int(b_mn), epi, float(alpha),
                           ptr(aux), ldaux, ptr(c2), ldc2, int(max_ctas), stream_ptr())
  check(rc, f"gemm M={M} N={N} K={K} a_mn={a_mn} b_mn={b_mn} epi={epi}")
  return out


def rmsnorm_fwd(x, w, eps, res=None, want_h=False):
  """Returns (y, rstd, h) with h = x + res (None unless ``res`` given and ``want_h``)."""
  d = x.shape[-1]
  x2 = x.reshape(-1, d)
  assert x2.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
  rows = x2.shape[0]
  y = torch.empty_like(x2)
  rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
  h = torch.empty_like(x2) if (res is not None and want_h) else None
  r2 = None
  if res is not None:
    r2 = res.reshape(-1, d)
    assert r2.is_contiguous() and r2.dtype == torch.bfloat16
  check(lib().tpb_rmsnorm_fwd(ptr(x2), ptr(r2), ptr(w), ptr(y), ptr(h), ptr(rstd), rows, d, float(eps), stream_ptr()),
        "rmsnorm_fwd")
  return y.view(x.shape), rstd, (h.view(x.shape) if h is not None else None)


def rmsnorm_bwd(dy, x, w, rstd, dres=None, dw_f32=None):
  """dx (+ dres) and dw accumulated (atomics) into fp32 ``dw_f32`` [dim]."""
  d = x.shape[-1]
  dy2, x2 = dy.reshape(-1, d), x.reshape(-1, d)
  assert dy2.is_contiguous() and x2.is_contiguous()
  dx = torch.empty_like(x2)
  if dw_f32 is None:
    dw_f32 = torch.zeros(d, dtype=torch.float32, device=x.device)
  dr2 = dres.reshape(-1, d) if dres is not None else None
  check(lib().tpb_rmsnorm_bwd(ptr(dy2), ptr(x2), ptr(w), ptr(rstd), ptr(dr2), ptr(dx), ptr(dw_f32), x2.shape[0], d,
                              stream_ptr()), "rmsnorm_bwd")
  return dx.view(x.shape), dw_f32


def rope_(x2d, col0, heads, dim, cos, sin, seq_len, pos=None, inverse=False, interleaved=False, head_stride=None):
  """In-place RoPE on ``heads`` slices of width ``dim`` (``head_stride`` apart, default ``dim``)
  starting at column ``col0`` of a [tokens, ld] bf16 matrix."""
  assert x2d.dim() == 2 and x2d.stride(1) == 1 and x2d.dtype == torch.bfloat16
  assert cos.dtype == torch.float32 and cos.is_contiguous() and cos.shape[-1] == dim // 2
  if pos is not None:
    assert pos.dtype == torch.int32 and pos.numel() == x2d.shape[0]
    _debug.check_index("rope", "pos", pos, 0, cos.shape[0])
  check(lib().tpb_rope_strided(ptr(x2d), x2d.stride(0), col0, heads, dim, head_stride or dim, ptr(cos), ptr(sin),
                               ptr(pos), x2d.shape[0], seq_len, int(inverse), int(interleaved), stream_ptr()), "rope")
  return x2d


def swiglu_fwd(gu):
  f = gu.shape[-1] // 2
  g2 = gu.reshape(-1, 2 * f)
  assert g2.is_contiguous() and gu.dtype == torch.bfloat16
  act = torch.empty(g2.shape[0], f, dtype=gu.dtype, device=gu.device)
  check(lib().tpb_swiglu_fwd(ptr(g2), ptr(act), g2.shape[0], f, stream_ptr()), "swiglu_fwd")
  return act.view(*gu.shape[:-1], f)


def swiglu_bwd(dact, gu):
  f = gu.shape[-1] // 2
  g2, d2 = gu.reshape(-1, 2 * f), dact.reshape(-1, f)
  assert g2.is_contiguous() and d2.is_contiguous()
  dgu = torch.empty_like(g2)
  check(lib().tpb_swiglu_bwd(ptr(d2), ptr(g2), ptr(dgu), g2.shape[0], f, stream_ptr()), "swiglu_bwd")
  return dgu.view(gu.shape)


def ce_fwd_bwd_(logits2d, targets, loss_sum, grad_scale=None):
  """loss_sum += sum of row losses; logits2d becomes d(loss)/d(logits) * grad_scale."""
  assert logits2d.dim() == 2 and logits2d.stride(1) == 1 and logits2d.dtype == torch.bfloat16
  assert targets.dtype == torch.int64 and targets.is_contiguous() and targets.numel() == logits2d.shape[0]
  _debug.check_index("ce_fwd_bwd", "targets", targets, 0, logits2d.shape[1], also_allowed=-100)
  check(lib().tpb_ce_fwd_bwd(ptr(logits2d), logits2d.stride(0), ptr(targets), ptr(loss_sum), ptr(grad_scale),
                             logits2d.shape[0], logits2d.shape[1], stream_ptr()), "ce_fwd_bwd")
  return logits2d


def adamw_(p32, m, v, grad, p16, lr, beta1, beta2, eps, wd, step, clip_coef=None):
  n = p32.numel()
  assert p32.dtype == m.dtype == v.dtype == torch.float32 and grad.numel() == n
  assert grad.dtype in (torch.bfloat16, torch.float32)
  bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
  check(lib().tpb_adamw(ptr(p32), ptr(m), ptr(v), ptr(grad), ptr(p16), n, lr, beta1, beta2, eps, wd, bc1, bc2,
                        ptr(clip_coef), int(grad.dtype == torch.bfloat16), stream_ptr()), "adamw")


def sumsq_(g, out):
  check(lib().tpb_sumsq(ptr(g), g.numel(), int(g.dtype == torch.bfloat16), ptr(out), stream_ptr()), "sumsq")
  return out


def clip_coef_(sumsq, max_norm, coef, norm_out):
  check(lib().tpb_clip_coef(ptr(sumsq), float(max_norm or 0.0), ptr(coef), ptr(norm_out), stream_ptr()), "clip_coef")


def embedding_fwd(table, ids, row0=0):
  flat = ids.reshape(-1)
  assert flat.dtype == torch.int64 and flat.is_contiguous() and table.is_contiguous()
  out = torch.empty(flat.numel(), table.shape[1], dtype=table.dtype, device=table.device)
  check(lib().tpb_embedding_fwd(ptr(table), ptr(flat), ptr(out), flat.numel(), table.shape[1], table.shape[0], row0,
                                stream_ptr()), "embedding_fwd")
  return out.view(*ids.shape, table.shape[1])


def embedding_bwd_(dout, ids, dtable, row0=0):
  flat = ids.reshape(-1)
  d2 = dout.reshape(flat.numel(), -1)
  assert d2.is_contiguous() and dtable.is_contiguous() and d2.dtype == torch.bfloat16
  check(lib().tpb_embedding_bwd(ptr(d2), ptr(flat), ptr(dtable), flat.numel(), d2.shape[1], dtable.shape[0], row0,
                                int(dtable.dtype == torch.float32), stream_ptr()), "embedding_bwd")
  return dtable


def cast_f32_to_bf16_(src, dst, scale=1.0, accumulate=False):
  check(lib().tpb_cast_f32_to_bf16(ptr(src), ptr(dst), src.numel(), float(scale), int(accumulate), stream_ptr()),
        "cast_f32_to_bf16")
  return dst
