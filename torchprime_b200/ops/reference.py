"""Plain-PyTorch definitions of every operator (fp32 math where it matters).

These are the oracles the CUDA kernels are tested against and the code path that
runs on CPU (gloo ranks, unit tests) or when ``engine.kernels=torch``.  Tensor
layout for attention is token-major ``[B, S, H, D]`` throughout this package, so
projection outputs are consumed without a transpose.

Behavioural sources in the reference: eager attention
(torchprime/torch_xla_models/attention.py:151-170), RMSNorm
(torchprime/torch_xla_models/model/llama/model.py:38-52), rotate-half RoPE
(model/llama/model.py:91-122), SwiGLU MLP (model/llama/model.py:125-139),
shift-by-one cross entropy (torchprime/torch_xla_models/loss.py:5-20), grouped
matmul fallbacks (model/mixtral/model.py:303-334, model/deepseek_v3/model.py:274-291).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

IGNORE_INDEX = -100


def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
  xf = x.float()
  var = xf.pow(2).mean(-1, keepdim=True)
  y = (xf * torch.rsqrt(var + eps)).to(x.dtype)
  return y if weight is None else weight * y


def add_rms_norm(x, residual, weight, eps):
  """Returns (norm(x + residual), x + residual)."""
  h = x + residual
  return rms_norm(h, weight, eps), h


def rotate_half(x):
  d = x.shape[-1] // 2
  return torch.cat((-x[..., d:], x[..., :d]), dim=-1)


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
  """Rotate-half rotary embedding.  x: [B,S,H,D]; cos/sin: [S,D] or [B,S,D]."""
  if cos.dim() == 2:
    cos, sin = cos[None, :, None, :], sin[None, :, None, :]
  else:
    cos, sin = cos[:, :, None, :], sin[:, :, None, :]
  return (x * cos.to(x.dtype)) + (rotate_half(x) * sin.to(x.dtype))


def rope_apply_interleaved(x, cos, sin):
  """DeepSeek layout: pairs (x0,x1),(x2,x3).. are permuted to half layout first
  (model/deepseek_v3/model.py:84-103), then rotate-half is applied."""
  b, s, h, d = x.shape
  x = x.view(b, s, h, d // 2, 2).transpose(-1, -2).reshape(b, s, h, d)
  return rope_apply(x, cos, sin)


def rope_apply_complex(x, freqs_cis):
  """Llama-4 even/odd complex-pair form (model/llama4/model.py:364-409).
  x: [B,S,H,D]; freqs_cis: complex [S, D/2] or [B,S,D/2]."""
  xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
  f = freqs_cis[None, :, None, :] if freqs_cis.dim() == 2 else freqs_cis[:, :, None, :]
  return torch.view_as_real(xc * f).flatten(3).type_as(x)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
  """silu(gate) * up for a fused ``[..., 2F]`` tensor laid out as [gate | up]."""
  g, u = gate_up.chunk(2, dim=-1)
  return F.silu(g) * u


def linear(x, w, bias=None):
  return F.linear(x, w, bias)


def build_mask(
  sq: int,
  sk: int,
  device,
  causal: bool = True,
  window: int | None = None,
  q_segment_ids: torch.Tensor | None = None,
  kv_segment_ids: torch.Tensor | None = None,
  q_positions: torch.Tensor | None = None,
  kv_positions: torch.Tensor | None = None,
) -> torch.Tensor:
  """Boolean keep-mask ``[B or 1, 1, sq, sk]`` for the supported mask family:
  causal, sliding window, packed-sequence segment ids and explicit row/column
  positions (the load-balanced context-parallel layout permutes query rows)."""
  qpos = q_positions if q_positions is not None else torch.arange(sq, device=device) + (sk - sq)
  kpos = kv_positions if kv_positions is not None else torch.arange(sk, device=device)
  qpos = qpos.reshape(-1, sq) if qpos.dim() > 1 else qpos[None]
  kpos = kpos.reshape(-1, sk) if kpos.dim() > 1 else kpos[None]
  keep = torch.ones(1, sq, sk, dtype=torch.bool, device=device)
  if causal:
    keep = keep & (qpos[:, :, None] >= kpos[:, None, :])
  if window is not None and window > 0:
    keep = keep & (qpos[:, :, None] - kpos[:, None, :] < window)
  if q_segment_ids is not None:
    kv_segment_ids = kv_segment_ids if kv_segment_ids is not None else q_segment_ids
    keep = keep & (q_segment_ids[:, :, None] == kv_segment_ids[:, None, :])
  return keep[:, None]


def attention(
  q: torch.Tensor,
  k: torch.Tensor,
  v: torch.Tensor,
  causal: bool = True,
  scale: float | None = None,
  window: int | None = None,
  q_segment_ids=None,
  kv_segment_ids=None,
  softcap: float | None = None,
  q_positions=None,
  kv_positions=None,
  return_lse: bool = False,
):
  """Eager attention with fp32 softmax.  q: [B,Sq,Hq,D], k: [B,Sk,Hkv,D], v: [B,Sk,Hkv,Dv].
  GQA is native (Hq a multiple of Hkv)."""
  b, sq, hq, d = q.shape
  sk, hkv = k.shape[1], k.shape[2]
  scale = scale if scale is not None else 1.0 / math.sqrt(d)
  g = hq // hkv
  qf = q.float().permute(0, 2, 1, 3).reshape(b, hkv, g, sq, d)
  kf = k.float().permute(0, 2, 1, 3)
  vf = v.float().permute(0, 2, 1, 3)
  s = torch.einsum("bhgqd,bhkd->bhgqk", qf, kf) * scale
  if softcap:
    s = softcap * torch.tanh(s / softcap)
  keep = build_mask(sq, sk, q.device, causal, window, q_segment_ids, kv_segment_ids,
                    q_positions, kv_positions)
  s = s.masked_fill(~keep[:, :, None], float("-inf"))
  lse = torch.logsumexp(s, dim=-1)
  p = torch.exp(s - lse.unsqueeze(-1))
  p = torch.nan_to_num(p, nan=0.0)  # fully masked rows produce zeros
  o = torch.einsum("bhgqk,bhkd->bhgqd", p, vf)
  o = o.reshape(b, hq, sq, -1).permute(0, 2, 1, 3).to(q.dtype)
  if return_lse:
    return o, lse.reshape(b, hq, sq)
  return o


def cross_entropy_shifted(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
  """Next-token loss: logits[:, :-1] against labels[:, 1:], mean over labels != -100."""
  v = logits.shape[-1]
  lg = logits[..., :-1, :].reshape(-1, v).float()
  lb = labels[..., 1:].reshape(-1).to(lg.device)
  return F.cross_entropy(lg, lb, ignore_index=IGNORE_INDEX)


def shift_labels(labels: torch.Tensor) -> torch.Tensor:
  """labels[:, 1:] padded with -100 so position t holds the target of token t.
  Done on the host before any sequence sharding so context-parallel ranks need
  no halo exchange."""
  out = torch.full_like(labels, IGNORE_INDEX)
  out[..., :-1] = labels[..., 1:]
  return out


def linear_cross_entropy(h, w, targets):
  """mean CE of (h @ w.T) against already-shifted ``targets`` (ignore -100)."""
  logits = F.linear(h, w).float()
  return F.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1),
                         ignore_index=IGNORE_INDEX)


def grouped_gemm(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
  """out[rows of group e] = lhs[rows of group e] @ rhs[e].  lhs: [M,K], rhs: [E,K,N]."""
  out = lhs.new_zeros(lhs.shape[0], rhs.shape[-1])
  start = 0
  for e, n in enumerate(group_sizes.tolist()):
    if n:
      out[start:start + n] = lhs[start:start + n] @ rhs[e]
    start += n
  return out


def router_softmax_topk(logits: torch.Tensor, k: int, renormalize: bool = True):
  """Mixtral routing: softmax over experts, top-k, renormalise (model/mixtral/model.py:774-780)."""
  probs = torch.softmax(logits.float(), dim=-1)
  w, idx = torch.topk(probs, k, dim=-1)
  if renormalize:
    w = w / w.sum(-1, keepdim=True)
  return w, idx, probs


def router_sigmoid_group_topk(logits, bias, k, n_group, topk_group, norm_topk_prob, scale):
  """DeepSeek-V3 routing (model/deepseek_v3/model.py:155-188): sigmoid scores, add the
  correction bias for *selection only*, keep the best ``topk_group`` groups (group
  score = sum of its top-2), top-k inside them, weights from the unbiased scores."""
  scores = torch.sigmoid(logits.float())
  t, e = scores.shape
  sel = scores + (bias.float()[None] if bias is not None else 0.0)
  if n_group > 1:
    gs = sel.view(t, n_group, e // n_group).topk(2, dim=-1)[0].sum(-1)
    gidx = gs.topk(topk_group, dim=-1)[1]
    gmask = torch.zeros_like(gs).scatter_(1, gidx, 1.0)
    smask = gmask[:, :, None].expand(t, n_group, e // n_group).reshape(t, e)
    sel = sel.masked_fill(smask == 0, 0.0)
  idx = sel.topk(k, dim=-1, sorted=False)[1]
  w = scores.gather(1, idx)
  if norm_topk_prob:
    w = w / (w.sum(-1, keepdim=True) + 1e-20)
  return w * scale, idx, scores


def moe_permute(x: torch.Tensor, idx: torch.Tensor, num_experts: int):
  """Sort the T*k (token, slot) pairs by expert.  Returns (rows [T*k, D],
  group_sizes [E] int32, order [T*k] with order[j] = flat (token*k+slot) of row j)."""
  t, k = idx.shape
  flat = idx.reshape(-1)
  order = torch.argsort(flat, stable=True)
  rows = x[order // k]
  sizes = torch.bincount(flat, minlength=num_experts).to(torch.int32)
  return rows, sizes, order


def moe_unpermute(rows: torch.Tensor, order: torch.Tensor, weights: torch.Tensor):
  """Inverse of :func:`moe_permute` followed by the weighted sum over the k slots."""
  t, k = weights.shape
  out = torch.zeros(t * k, rows.shape[-1], dtype=rows.dtype, device=rows.device)
  out[order] = rows
  return (out.view(t, k, -1) * weights[..., None].to(rows.dtype)).sum(1)


def adamw_step(p32, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
  """One decoupled-weight-decay Adam step on fp32 tensors (torch.optim.AdamW math)."""
  g = g.float() * grad_scale
  m.mul_(beta1).add_(g, alpha=1 - beta1)
  v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
  bc1 = 1 - beta1 ** step
  bc2 = 1 - beta2 ** step
  p32.mul_(1 - lr * wd)
  denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
  p32.addcdiv_(m, denom, value=-lr / bc1)
  return p32
