"""Autograd-aware operators.  On CUDA bf16 tensors (and unless the backend is set to
``"torch"``) they run the hand-written sm_100a kernels; everywhere else they run
the plain-PyTorch definitions in ``reference.py``.

Weight gradients follow the "main_grad" convention: when a parameter carries a
``main_grad`` tensor (a view into the FSDP engine's flat gradient buffer) the
wgrad GEMM writes or accumulates straight into it (``param.grad_overwrite``
decides which) and autograd sees ``None``; otherwise the gradient is returned
normally.
"""

from __future__ import annotations

import math
from contextlib import contextmanager

import torch
import torch.nn.functional as F

from . import _lib, reference as ref

_STATE = {"backend": "auto", "attention": "auto"}


def set_backend(name: str):
  """``"sm100"`` (kernels required), ``"torch"`` (never use kernels) or ``"auto"``."""
  assert name in ("sm100", "torch", "auto")
  _STATE["backend"] = name


def get_backend() -> str:
  return _STATE["backend"]


@contextmanager
def backend(name: str):
  old = _STATE["backend"]
  set_backend(name)
  try:
    yield
  finally:
    _STATE["backend"] = old


def use_kernels(*tensors) -> bool:
  if _STATE["backend"] == "torch":
    return False
  for t in tensors:
    if t is None:
      continue
    if not t.is_cuda or t.dtype != torch.bfloat16:
      return False
  if _STATE["backend"] == "auto" and not _lib.available():
    # A CUDA box without the library is a build error, not a reason to fall back.
    raise _lib.KernelError("CUDA tensors but libtpb200.so is not built; run python -m torchprime_b200.build")
  return True


# --------------------------------------------------------------------------- helpers
def _adjacent(ts) -> bool:
  for a, b in zip(ts[:-1], ts[1:]):
    if not (a.is_contiguous() and b.is_contiguous()):
      return False
    if a.untyped_storage().data_ptr() != b.untyped_storage().data_ptr():
      return False
    if a.storage_offset() + a.numel() != b.storage_offset() or a.shape[1:] != b.shape[1:]:
      return False
  return ts[0].is_contiguous()


def _fused_view(ts):
  """One [sum(rows), K] view over row-adjacent 2-D tensors that share a storage."""
  if len(ts) == 1:
    return ts[0]
  rows = sum(t.shape[0] for t in ts)
  k = ts[0].shape[1]
  return ts[0].as_strided((rows, k), (k, 1))


def _grad_sink(weights):
  """Fused main_grad view if every weight has an adjacent main_grad, else None."""
  mgs = [getattr(w, "main_grad", None) for w in weights]
  if any(m is None for m in mgs):
    return None
  if len(mgs) > 1 and not _adjacent(mgs):
    return None
  return _fused_view(mgs)


def overwrites_grad(w) -> bool:
  """Whether the gradient about to be delivered replaces the content of ``w.main_grad`` (first
  gradient of the step) or adds to it.  A backward pass that is being captured into a CUDA graph is
  replayed once per step, so what it records is always the overwriting form."""
  if w.is_cuda and torch.cuda.is_current_stream_capturing():
    return True
  return bool(getattr(w, "grad_overwrite", False))


def _wgrad_into(sink, weights, dy2, x2):
  """dW = dy2^T @ x2 written into the main_grad sink (overwrite or accumulate).  Under the FSDP
  engine's peer-memory collectives the parameters carry ``rs_push``: the GEMM epilogue then stores
  the tiles straight into the staging slots of the ranks that own those rows of the flat gradient
  buffer (the reduce-scatter's send side) instead of into the local buffer."""
  from . import kernels as k
  overwrite = all(overwrites_grad(w) for w in weights)
  push = getattr(weights[0], "rs_push", None)
  if push is not None:
    if overwrite and all(getattr(w, "rs_push", None) is not None for w in weights) and push(sink, dy2, x2):
      for w in weights:
        w.grad_overwrite = False
      return
    if not overwrite:
      push.func.__self__.check_not_pushed(push.args[0], sink)
  if sink.dtype == torch.float32:
    k.gemm(dy2, x2, a_mn=True, b_mn=True, out=sink, epi=k.EPI_F32 if overwrite else k.EPI_F32_ACC)
  else:
    k.gemm(dy2, x2, a_mn=True, b_mn=True, out=sink, epi=k.EPI_BF16 if overwrite else k.EPI_BF16_ACC)
  for w in weights:
    w.grad_overwrite = False


# --------------------------------------------------------------------------- gathers in flight
# The FSDP engine's copy-engine all-gather of the unit whose forward is running (parallel/fsdp_comm.py):
# while it is set, GEMMs whose weight lies in that unit's gathered buffer wait for the weight's shards
# inside the kernel; any other reader of such a weight first orders the stream after the whole gather.
_AG_CTX = [None]


def set_gather_context(ctx):
  _AG_CTX[0] = ctx


def get_gather_context():
  return _AG_CTX[0]


def _inflight(w):
  """(context, element offset) when ``w`` belongs to a gather that is still in flight."""
  ctx = _AG_CTX[0]
  if ctx is None:
    return None, None
  off = ctx.offset_of(w)
  return (ctx, off) if off is not None else (None, None)


def _settle(*weights):
  """For readers that cannot wait in-kernel: the whole gather must have landed."""
  ctx = _AG_CTX[0]
  if ctx is not None and any(w is not None and ctx.offset_of(w) is not None for w in weights):
    ctx.wait_all()
    set_gather_context(None)


# --------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, residual, n_w, reducers, *weights):
    from . import kernels as k
    w = _fused_view(list(weights))
    x2 = x.reshape(-1, x.shape[-1])
    out_reduce, ctx.grad_reduce = reducers if reducers is not None else (None, None)
    ag, ag_off = _inflight(weights[0])
    if ag is not None and out_reduce is not None:
      _settle(weights[0])
      ag = None
    if out_reduce is not None:
      # row-parallel linear of tensor parallelism: the all-reduce over the tensor group happens in
      # the GEMM epilogue (rank 0 also adds the residual)
      res2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
      y = out_reduce.gemm_allreduce(x2, w, res2).view(*x.shape[:-1], w.shape[0])
      ctx.save_for_backward(x2, *weights)
      ctx.has_res = residual is not None
      ctx.x_shape = x.shape
      return y
    # the result is allocated in its final shape (not returned as a view) so that later
    # in-place operators such as RoPE may modify it
    y = torch.empty(*x.shape[:-1], w.shape[0], dtype=x.dtype, device=x.device)
    y2 = y.view(-1, w.shape[0])
    if ag is not None:
      from ..parallel.fsdp_comm import gemm_ag_wait
      res2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
      gemm_ag_wait(ag, x2, ag_off, w.shape[0], w.shape[1], y2, k.EPI_BF16_RES if res2 is not None else k.EPI_BF16,
                   aux=res2)
    elif residual is not None:
      k.gemm(x2, w, out=y2, epi=k.EPI_BF16_RES, aux=residual.reshape(-1, w.shape[0]))
    else:
      k.gemm(x2, w, out=y2)
    ctx.save_for_backward(x2, *weights)
    ctx.has_res = residual is not None
    ctx.x_shape = x.shape
    return y

  @staticmethod
  def backward(ctx, dy):
    from . import kernels as k
    x2, *weights = ctx.saved_tensors
    w = _fused_view(weights)
    dy2 = dy.reshape(-1, dy.shape[-1])
    if not dy2.is_contiguous():
      dy2 = dy2.contiguous()
    dx = None
    if ctx.needs_input_grad[0]:
      if ctx.grad_reduce is not None:      # column-parallel linear: the input gradient is summed over the group
        dx = ctx.grad_reduce.gemm_allreduce(dy2, w, None, b_mn=True).view(ctx.x_shape)
      else:
        dx = k.gemm(dy2, w, b_mn=True).view(ctx.x_shape)
    wgrads = [None] * len(weights)
    if any(ctx.needs_input_grad[4:]):
      sink = _grad_sink(weights)
      if sink is not None:
        _wgrad_into(sink, weights, dy2, x2)
      else:
        dw = k.gemm(dy2, x2, a_mn=True, b_mn=True)
        wgrads, r = [], 0
        for wt in weights:
          wgrads.append(dw[r:r + wt.shape[0]])
          r += wt.shape[0]
    dres = dy if ctx.has_res else None
    return (dx, dres, None, None, *wgrads)


def _gemm_friendly(x, ws) -> bool:
  """Shapes the TMA-fed GEMM accepts: 16-byte aligned rows for every operand."""
  n = sum(w.shape[0] for w in ws)
  k = ws[0].shape[1]
  return (n % 8 == 0 and k % 8 == 0 and all(w.dim() == 2 and w.is_contiguous() for w in ws)
          and x.shape[-1] == k and x.reshape(-1, k).stride(-1) == 1 and x.reshape(-1, k).stride(0) % 8 == 0)


def _reducer_ok(reducer, x, n_out, k_in) -> bool:
  return reducer is not None and reducer.usable(x.numel() // x.shape[-1], n_out, k_in)


def linear(x, weights, bias=None, residual=None, tp_reduce=None, tp_reduce_grad=None):
  """y = x @ cat(weights)^T (+ bias) (+ residual).  ``weights`` is one tensor or a list of
  row-adjacent tensors (q/k/v or gate/up laid out back to back) which then run as
  one GEMM.

  Tensor parallelism with the all-reduce inside the GEMM (``ops.fused_collective.AllReduceGemm``):
  ``tp_reduce`` sums the OUTPUT over the tensor group (row-parallel weight; the caller must not
  reduce again), ``tp_reduce_grad`` sums the INPUT GRADIENT (column-parallel weight).  Callers ask
  ``reducer.usable(rows, n, k)`` first; a request that cannot be honoured raises."""
  ws = list(weights) if isinstance(weights, (list, tuple)) else [weights]
  if (use_kernels(x, *ws) and bias is None and (len(ws) == 1 or _adjacent(ws)) and _gemm_friendly(x, ws)
      and (residual is None or residual.dtype == x.dtype)):
    n_out, k_in = sum(w.shape[0] for w in ws), ws[0].shape[1]
    reducers = None
    if tp_reduce is not None or tp_reduce_grad is not None:
      out_r = tp_reduce if _reducer_ok(tp_reduce, x, n_out, k_in) else None
      grad_r = tp_reduce_grad if _reducer_ok(tp_reduce_grad, x, k_in, n_out) else None
      if tp_reduce is not None and out_r is None:
        raise RuntimeError("fused tensor-parallel all-reduce requested but not available for this shape")
      if tp_reduce_grad is not None and grad_r is None:
        raise RuntimeError("fused tensor-parallel gradient all-reduce requested but not available for this shape")
      reducers = (out_r, grad_r)
    return _LinearFn.apply(x, residual, len(ws), reducers, *ws)
  if tp_reduce is not None or tp_reduce_grad is not None:
    raise RuntimeError("fused tensor-parallel all-reduce requested on a path without kernels")
  _settle(*ws)
  if len(ws) == 1:
    y = F.linear(x, ws[0], bias)
  else:
    y = torch.cat([F.linear(x, w) for w in ws], dim=-1)
    if bias is not None:
      y = y + bias
  return y if residual is None else y + residual


class _LinearSwigluFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, w_gate, w_up, grad_reduce=None):
    from . import kernels as k
    ctx.grad_reduce = grad_reduce
    w = _fused_view([w_gate, w_up])
    x2 = x.reshape(-1, x.shape[-1])
    need_grad = any(ctx.needs_input_grad)
    gu = torch.empty(x2.shape[0], w.shape[0], dtype=x.dtype, device=x.device) if need_grad else None
    act = torch.empty(*x.shape[:-1], w_gate.shape[0], dtype=x.dtype, device=x.device)
    ag, ag_off = _inflight(w_gate)
    if ag is not None:
      from ..parallel.fsdp_comm import gemm_ag_wait
      gemm_ag_wait(ag, x2, ag_off, w.shape[0], w.shape[1], act.view(-1, w_gate.shape[0]), k.EPI_SWIGLU, c2=gu)
    else:
      k.gemm(x2, w, out=act.view(-1, w_gate.shape[0]), epi=k.EPI_SWIGLU, c2=gu)
    if need_grad:
      ctx.save_for_backward(x2, gu, w_gate, w_up)
    ctx.x_shape = x.shape
    return act

  @staticmethod
  def backward(ctx, dact):
    from . import kernels as k
    x2, gu, w_gate, w_up = ctx.saved_tensors
    w = _fused_view([w_gate, w_up])
    dgu = k.swiglu_bwd(dact.reshape(-1, dact.shape[-1]).contiguous(), gu)
    dx = None
    if ctx.needs_input_grad[0]:
      if ctx.grad_reduce is not None:      # column-parallel gate/up: the input gradient is summed over the group
        dx = ctx.grad_reduce.gemm_allreduce(dgu, w, None, b_mn=True).view(ctx.x_shape)
      else:
        dx = k.gemm(dgu, w, b_mn=True).view(ctx.x_shape)
    grads = [None, None]
    if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
      sink = _grad_sink([w_gate, w_up])
      if sink is not None:
        _wgrad_into(sink, [w_gate, w_up], dgu, x2)
      else:
        dw = k.gemm(dgu, x2, a_mn=True, b_mn=True)
        grads = [dw[: w_gate.shape[0]], dw[w_gate.shape[0]:]]
    return (dx, *grads, None)


def linear_swiglu(x, w_gate, w_up, tp_reduce_grad=None):
  """silu(x @ w_gate^T) * (x @ w_up^T) as one GEMM with a fused epilogue."""
  if (use_kernels(x, w_gate, w_up) and _adjacent([w_gate, w_up]) and w_gate.shape[0] % 8 == 0
      and _gemm_friendly(x, [w_gate, w_up])):
    if tp_reduce_grad is not None and not _reducer_ok(tp_reduce_grad, x, x.shape[-1], 2 * w_gate.shape[0]):
      raise RuntimeError("fused tensor-parallel gradient all-reduce requested but not available for this shape")
    return _LinearSwigluFn.apply(x, w_gate, w_up, tp_reduce_grad)
  if tp_reduce_grad is not None:
    raise RuntimeError("fused tensor-parallel gradient all-reduce requested on a path without kernels")
  _settle(w_gate, w_up)
  return F.silu(F.linear(x, w_gate)) * F.linear(x, w_up)


# --------------------------------------------------------------------------- norm
def _norm_wgrad(w, dw_f32):
  """Deliver an fp32 norm-weight gradient: into main_grad if present, else return it."""
  from . import kernels as k
  mg = getattr(w, "main_grad", None)
  if mg is None:
    return dw_f32.to(w.dtype)
  overwrite = overwrites_grad(w)
  if mg.dtype == torch.float32:
    mg.copy_(dw_f32) if overwrite else mg.add_(dw_f32)
  elif mg.numel() % 4 == 0:
    k.cast_f32_to_bf16_(dw_f32, mg, 1.0, accumulate=not overwrite)
  else:
    mg.copy_(dw_f32 if overwrite else mg.float() + dw_f32)
  w.grad_overwrite = False
  return None


class _RMSNormFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, w, eps):
    from . import kernels as k
    xc = x.contiguous()
    y, rstd, _ = k.rmsnorm_fwd(xc, w, eps)
    ctx.save_for_backward(xc, w, rstd)
    return y

  @staticmethod
  def backward(ctx, dy):
    from . import kernels as k
    x, w, rstd = ctx.saved_tensors
    dx, dw = k.rmsnorm_bwd(dy.contiguous(), x, w, rstd)
    return dx, (_norm_wgrad(w, dw) if ctx.needs_input_grad[1] else None), None


class _AddRMSNormFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, res, w, eps):
    from . import kernels as k
    y, rstd, h = k.rmsnorm_fwd(x.contiguous(), w, eps, res=res.contiguous(), want_h=True)
    ctx.save_for_backward(h, w, rstd)
    ctx.mark_non_differentiable()
    return y, h

  @staticmethod
  def backward(ctx, dy, dh):
    from . import kernels as k
    h, w, rstd = ctx.saved_tensors
    dx, dw = k.rmsnorm_bwd(dy.contiguous(), h, w, rstd, dres=dh.contiguous() if dh is not None else None)
    return dx, dx, (_norm_wgrad(w, dw) if ctx.needs_input_grad[2] else None), None


def rms_norm(x, w, eps):
  if use_kernels(x, w) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
    return _RMSNormFn.apply(x, w, eps)
  return ref.rms_norm(x, w, eps)


class _RMSNormPassFn(torch.autograd.Function):
  """(rmsnorm(x) * w, x): the second output is ``x`` itself, handed on as the residual input of a
  later operator.  Its purpose is the backward: the gradient of the normalised branch and the
  gradient of the residual branch arrive together and are summed inside the norm-backward kernel,
  instead of by a separate elementwise add of two activation-sized tensors per norm."""

  @staticmethod
  def forward(ctx, x, w, eps):
    from . import kernels as k
    xc = x.contiguous()
    y, rstd, _ = k.rmsnorm_fwd(xc, w, eps)
    ctx.save_for_backward(xc, w, rstd)
    return y, x.view_as(x)

  @staticmethod
  def backward(ctx, dy, dres):
    from . import kernels as k
    x, w, rstd = ctx.saved_tensors
    if dy is None:
      return dres, None, None
    dx, dw = k.rmsnorm_bwd(dy.contiguous(), x, w, rstd, dres=dres.contiguous() if dres is not None else None)
    return dx, (_norm_wgrad(w, dw) if ctx.needs_input_grad[1] else None), None


def rms_norm_residual(x, w, eps):
  """Returns (rmsnorm(x) * w, x).  Use the second value wherever ``x`` is needed again (the
  residual connection): its gradient is then added inside the norm's backward kernel."""
  if use_kernels(x, w) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
    return _RMSNormPassFn.apply(x, w, eps)
  return ref.rms_norm(x, w, eps), x


def add_rms_norm(x, res, w, eps):
  """(rmsnorm(x + res) * w, x + res) with the add fused into the norm kernel."""
  if use_kernels(x, res, w) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
    return _AddRMSNormFn.apply(x, res, w, eps)
  return ref.add_rms_norm(x, res, w, eps)


# --------------------------------------------------------------------------- rope
class _RopeInplaceFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, qkv, cos, sin, heads, dim, seq_len, pos, interleaved, col0=0, head_stride=None):
    from . import kernels as k
    q2 = qkv.view(-1, qkv.shape[-1])
    k.rope_(q2, col0, heads, dim, cos, sin, seq_len, pos=pos, interleaved=interleaved, head_stride=head_stride)
    ctx.mark_dirty(qkv)
    ctx.save_for_backward(cos, sin, pos) if pos is not None else ctx.save_for_backward(cos, sin)
    ctx.args = (heads, dim, seq_len, interleaved, pos is not None, col0, head_stride)
    return qkv

  @staticmethod
  def backward(ctx, dqkv):
    from . import kernels as k
    heads, dim, seq_len, interleaved, has_pos, col0, head_stride = ctx.args
    saved = ctx.saved_tensors
    pos = saved[2] if has_pos else None
    # The incoming gradient is a buffer the attention backward produced for this node alone (RoPE is
    # applied in place on the projection output, so nothing else consumes that tensor's gradient):
    # rotate it in place instead of cloning 100 MB per layer.
    d = dqkv if dqkv.is_contiguous() else dqkv.contiguous()
    k.rope_(d.view(-1, d.shape[-1]), col0, heads, dim, saved[0], saved[1], seq_len, pos=pos, inverse=True,
            interleaved=interleaved, head_stride=head_stride)
    return d, None, None, None, None, None, None, None, None, None


def rope_slices(x, cos_half, sin_half, heads, dim, seq_len, col0, head_stride, pos=None, interleaved=False):
  """Rotate ``heads`` slices of width ``dim`` that start at column ``col0`` and lie ``head_stride``
  apart in the last dimension of ``x`` [B,S,C] (the rope part of MLA heads).  In place on CUDA."""
  if use_kernels(x):
    return _RopeInplaceFn.apply(x, cos_half, sin_half, heads, dim, seq_len, pos, interleaved, col0, head_stride)
  b, s, c = x.shape
  cols = (col0 + torch.arange(heads, device=x.device)[:, None] * head_stride
          + torch.arange(dim, device=x.device)[None, :]).reshape(-1)
  part = x[..., cols]
  rot = rope_inplace(part, cos_half, sin_half, heads, dim, seq_len, pos=pos, interleaved=interleaved)
  out = x.clone()
  out[..., cols] = rot
  return out


def rope_inplace(qkv, cos_half, sin_half, heads, dim, seq_len, pos=None, interleaved=False):
  """Rotate the first ``heads`` heads of a fused ``[B, S, (heads + rest) * dim]`` projection in
  place (q and k heads; v is left alone).  cos/sin: fp32 [max_pos, dim/2]."""
  if use_kernels(qkv):
    return _RopeInplaceFn.apply(qkv, cos_half, sin_half, heads, dim, seq_len, pos, interleaved)
  b, s, _ = qkv.shape
  head = qkv[..., : heads * dim].reshape(b, s, heads, dim)
  if pos is not None:
    p = pos.view(b, s).long()
    cos = torch.cat([cos_half[p], cos_half[p]], -1)
    sin = torch.cat([sin_half[p], sin_half[p]], -1)
  else:
    cos = torch.cat([cos_half[:s], cos_half[:s]], -1)
    sin = torch.cat([sin_half[:s], sin_half[:s]], -1)
  if interleaved:
    half = ref.rope_apply_interleaved(head.float(), cos, sin)
    rot = torch.stack([half[..., : dim // 2], half[..., dim // 2:]], dim=-1).reshape(b, s, heads, dim)
  else:
    rot = ref.rope_apply(head.float(), cos, sin)
  return torch.cat([rot.to(qkv.dtype).reshape(b, s, heads * dim), qkv[..., heads * dim:]], dim=-1)


# --------------------------------------------------------------------------- swiglu
class _SwigluFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, gu):
    from . import kernels as k
    guc = gu.contiguous()
    ctx.save_for_backward(guc)
    return k.swiglu_fwd(guc)

  @staticmethod
  def backward(ctx, dact):
    from . import kernels as k
    (gu,) = ctx.saved_tensors
    return k.swiglu_bwd(dact.contiguous(), gu)


def swiglu(gate_up):
  if use_kernels(gate_up) and (gate_up.shape[-1] // 2) % 8 == 0:
    return _SwigluFn.apply(gate_up)
  return ref.swiglu(gate_up)


# --------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, ids, table):
    from . import kernels as k
    ctx.save_for_backward(ids, table)
    return k.embedding_fwd(table, ids.contiguous())

  @staticmethod
  def backward(ctx, dout):
    from . import kernels as k
    ids, table = ctx.saved_tensors
    mg = getattr(table, "main_grad", None)
    if mg is not None:
      if getattr(table, "grad_overwrite", False):
        mg.zero_()
        table.grad_overwrite = False
      k.embedding_bwd_(dout.contiguous(), ids.contiguous(), mg)
      return None, None
    g = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
    k.embedding_bwd_(dout.contiguous(), ids.contiguous(), g)
    return None, g.to(table.dtype)


class _EmbeddingPeerFn(torch.autograd.Function):
  """Lookup in a table that stays sharded: rows are read straight from the owners' parameter shards
  over NVLink (``peer``: see parallel/fsdp_comm.PeerLookup).  ``table`` is the parameter, whose storage is
  empty on this path; it is an input only so that the backward runs and finds ``table.main_grad``."""

  @staticmethod
  def forward(ctx, ids, table, peer):
    flat = ids.reshape(-1).contiguous()
    out = torch.empty(flat.numel(), peer.dim, dtype=torch.bfloat16, device=ids.device)
    peer.lookup(flat, out)
    ctx.save_for_backward(ids)
    ctx.table = table
    return out.view(*ids.shape, peer.dim)

  @staticmethod
  def backward(ctx, dout):
    from . import kernels as k
    (ids,) = ctx.saved_tensors
    table = ctx.table
    mg = table.main_grad
    if overwrites_grad(table):
      mg.zero_()
      table.grad_overwrite = False
    k.embedding_bwd_(dout.contiguous(), ids.contiguous(), mg)
    return None, None, None


def embedding_peer(ids, table, peer):
  return _EmbeddingPeerFn.apply(ids, table, peer)


def embedding(ids, table):
  if use_kernels(table) and table.shape[1] % 8 == 0:
    return _EmbeddingFn.apply(ids, table)
  return F.embedding(ids, table)


# --------------------------------------------------------------------------- attention
def set_attention_impl(name: str):
  """``"auto"`` | ``"sm100"`` (own kernel) | ``"sdpa"`` (library baseline) | ``"eager"`` (oracle)."""
  assert name in ("auto", "sm100", "sdpa", "eager")
  _STATE["attention"] = name


_ATTN_USED = {"last": "none"}


def attention_impl_in_use() -> str:
  """Which implementation the last attention call ran (for benchmark records)."""
  return _ATTN_USED["last"]


def attention(q, k, v, causal=True, scale=None, window=None, q_segment_ids=None, kv_segment_ids=None,
              softcap=None, q_positions=None, kv_positions=None):
  """softmax(q k^T * scale + mask) v on ``[B, S, H, D]`` tensors, GQA-native."""
  impl = _STATE["attention"]
  plain = (window is None and q_segment_ids is None and softcap is None and q_positions is None
           and kv_positions is None)
  if impl in ("auto", "sm100") and q.is_cuda and q.dtype == torch.bfloat16 and _STATE["backend"] != "torch":
    from . import attention_sm100
    if attention_sm100.supported(q, k, v, causal, window, q_segment_ids, softcap, q_positions, kv_positions):
      _ATTN_USED["last"] = "sm100 tcgen05 kernel"
      return attention_sm100.attention(q, k, v, causal=causal, scale=scale, window=window,
                                       q_segment_ids=q_segment_ids, kv_segment_ids=kv_segment_ids,
                                       softcap=softcap, q_positions=q_positions, kv_positions=kv_positions)
    if impl == "sm100":
      raise _lib.KernelError(f"attention_sm100 does not support q{tuple(q.shape)} k{tuple(k.shape)} v{tuple(v.shape)}")
  if impl != "eager" and plain and q.is_cuda and q.shape[-1] == v.shape[-1]:
    _ATTN_USED["last"] = "torch SDPA (library)"
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal,
                                       scale=scale, enable_gqa=q.shape[2] != k.shape[2])
    return o.transpose(1, 2)
  _ATTN_USED["last"] = "eager fp32 reference"
  return ref.attention(q, k, v, causal=causal, scale=scale, window=window, q_segment_ids=q_segment_ids,
                       kv_segment_ids=kv_segment_ids, softcap=softcap, q_positions=q_positions,
                       kv_positions=kv_positions)


def attention_qkv(qkv, hq, hkv, d, causal=True, scale=None, window=None, q_segment_ids=None, q_positions=None):
  """Self-attention on a fused projection output ``qkv`` [B, S, (Hq + 2 Hkv) * d]: same result as
  slicing q, k, v out of it and calling :func:`attention`, but on the kernel path the tensor is a
  single autograd input, so its gradient is produced in one piece."""
  b, s, _ = qkv.shape
  if (_STATE["attention"] in ("auto", "sm100") and _STATE["backend"] != "torch" and qkv.is_cuda
      and qkv.dtype == torch.bfloat16 and d == 128 and qkv.is_contiguous()):
    from . import attention_sm100
    _ATTN_USED["last"] = "sm100 tcgen05 kernel"
    return attention_sm100.attention_qkv(qkv, hq, hkv, d, causal=causal, scale=scale, window=window,
                                         q_segment_ids=q_segment_ids, q_positions=q_positions)
  q = qkv[..., : hq * d].view(b, s, hq, d)
  k = qkv[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
  v = qkv[..., (hq + hkv) * d:].view(b, s, hkv, d)
  return attention(q, k, v, causal=causal, scale=scale, window=window, q_segment_ids=q_segment_ids,
                   q_positions=q_positions)


# --------------------------------------------------------------------------- lm head + CE
class _LinearCrossEntropyFn(torch.autograd.Function):
  """Chunked lm_head + softmax cross entropy.  The forward pass also produces the
  gradients (loss is the end of the graph), so fp32 logits for the full sequence
  are never materialised: per chunk of rows the bf16 logits tile is produced by
  the GEMM, turned into d(logits) in place by the CE kernel and consumed by the
  dgrad / wgrad GEMMs."""

  @staticmethod
  def forward(ctx, h, w, targets, chunk_rows, n_valid):
    from . import kernels as k
    h2 = h.reshape(-1, h.shape[-1])
    tg = targets.reshape(-1).contiguous()
    rows, vocab = h2.shape[0], w.shape[0]
    if n_valid is None:
      n_valid = (tg >= 0).sum().clamp(min=1).float()
    scale = (1.0 / n_valid.float()).reshape(1)
    loss_sum = torch.zeros(1, dtype=torch.float32, device=h.device)
    need_dh = ctx.needs_input_grad[0]
    need_dw = ctx.needs_input_grad[1]
    dh = torch.empty_like(h2) if need_dh else None
    sink = _grad_sink([w]) if need_dw else None
    dw_local = None
    if need_dw and sink is None:
      dw_local = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
    logits = torch.empty(min(chunk_rows, rows), vocab, dtype=torch.bfloat16, device=h.device)
    for r0 in range(0, rows, chunk_rows):
      r1 = min(rows, r0 + chunk_rows)
      lg = logits[: r1 - r0]
      k.gemm(h2[r0:r1], w, out=lg)
      k.ce_fwd_bwd_(lg, tg[r0:r1], loss_sum, scale)
      if need_dh:
        k.gemm(lg, w, b_mn=True, out=dh[r0:r1])
      if need_dw:
        if sink is not None:
          _wgrad_into(sink, [w], lg, h2[r0:r1])
        else:
          k.gemm(lg, h2[r0:r1], a_mn=True, b_mn=True, out=dw_local, epi=k.EPI_F32_ACC)
    ctx.save_for_backward(dh if need_dh else None, dw_local)
    ctx.h_shape = h.shape
    return (loss_sum * scale).reshape(())

  @staticmethod
  def backward(ctx, dloss):
    dh, dw_local = ctx.saved_tensors
    gh = (dh * dloss.to(dh.dtype)).view(ctx.h_shape) if dh is not None else None
    gw = (dw_local * dloss).to(torch.bfloat16) if dw_local is not None else None
    return gh, gw, None, None, None


def linear_cross_entropy(h, w, targets, chunk_rows: int = 2048, n_valid=None):
  """CE of ``h @ w^T`` against already shifted ``targets`` (-100 ignored), summed and divided by
  ``n_valid`` (default: the number of valid targets, i.e. the mean)."""
  if use_kernels(h, w) and w.shape[0] % 8 == 0 and h.shape[-1] % 8 == 0:
    return _LinearCrossEntropyFn.apply(h, w, targets, chunk_rows, n_valid)
  if n_valid is None:
    return ref.linear_cross_entropy(h, w, targets)
  logits = F.linear(h, w).float()
  return F.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1), ignore_index=ref.IGNORE_INDEX,
                         reduction="sum") / n_valid
