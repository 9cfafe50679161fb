"""Mixture-of-experts operators: routing, dropless (or capacity-limited) dispatch into an
expert-grouped row layout, grouped SwiGLU MLP, weighted combine.

What the reference does with argsort / one-hot / Pallas ``gmm`` calls
(torchprime/torch_xla_models/model/mixtral/model.py:302-626,
model/deepseek_v3/model.py:274-338) is organised here around one layout: the ``T*K``
(token, slot) pairs are sorted by expert and every expert's rows are padded to a multiple of
128, so a 128-row GEMM tile never straddles two experts and padded rows are zero.  All index
bookkeeping stays on the device (no host synchronisation): the padded row count is bounded
by ``T*K + 128*E`` and tiles past the real end are marked unused.

On CUDA/bf16 the heavy parts run as sm_100a kernels (router top-k, row gather, grouped
tcgen05 GEMMs with fused SwiGLU, combine); elsewhere the same math runs in plain PyTorch.
"""

from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _debug, _lib, reference as ref
from ._lib import check, lib, ptr, stream_ptr

P, I, LL, FL = c_void_p, c_int, c_longlong, c_float
_lib.register_signature("tpb_grouped_gemm_bf16", [P, P, P, P, I, I, I, I, LL, LL, LL, LL, I, I, I, FL, P, LL, I, P, P,
                                                  LL, I, P])
_lib.register_signature("tpb_router_topk", [P, I, P, P, P, P, I, I, I, I, I, I, I, FL, P])
_lib.register_signature("tpb_moe_plan", [P, I, I, I, I, I, P, P, P, P, P, P, P])
_lib.register_signature("tpb_moe_gather", [P, P, P, P, LL, I, P])
_lib.register_signature("tpb_moe_combine", [P, P, P, P, LL, I, I, P])
_lib.register_signature("tpb_moe_combine_dw", [P, P, P, P, LL, I, I, P])

ROW_ALIGN = 128


def _kernels_ok(*ts) -> bool:
  from .functional import use_kernels
  return use_kernels(*ts)


# ----------------------------------------------------------------------------- routing
class _RouterFn(torch.autograd.Function):
  """Kernel forward; the (tiny) backward re-derives the weights with PyTorch ops on the
  selected experts so gradients reach the gate."""

  @staticmethod
  def forward(ctx, logits, bias, k, mode, n_group, topk_group, norm_topk, scale):
    t, e = logits.shape
    lg = logits.contiguous()
    w = torch.empty(t, k, dtype=torch.float32, device=logits.device)
    idx = torch.empty(t, k, dtype=torch.int32, device=logits.device)
    scores = torch.empty(t, e, dtype=torch.float32, device=logits.device)
    b = bias.float().contiguous() if bias is not None else None
    check(lib().tpb_router_topk(ptr(lg), int(lg.dtype == torch.bfloat16), ptr(b), ptr(w), ptr(idx), ptr(scores), t, e,
                                k, mode, n_group, topk_group, int(norm_topk), float(scale), stream_ptr()),
          "router_topk")
    ctx.save_for_backward(logits, idx)
    ctx.args = (mode, norm_topk, scale)
    ctx.mark_non_differentiable(idx)
    return w, idx, scores

  @staticmethod
  def backward(ctx, dw, _didx, dscores):
    logits, idx = ctx.saved_tensors
    mode, norm_topk, scale = ctx.args
    with torch.enable_grad():
      lg = logits.detach().float().requires_grad_(True)
      s = torch.softmax(lg, dim=-1) if mode == 0 else torch.sigmoid(lg)
      w = s.gather(1, idx.long())
      if norm_topk:
        w = w / (w.sum(-1, keepdim=True) + (0.0 if mode == 0 else 1e-20))
      w = w * scale
      outs, grads = [w], [dw]
      if dscores is not None:
        outs.append(s)
        grads.append(dscores)
      (g,) = torch.autograd.grad(outs, lg, grads)
    return g.to(logits.dtype), None, None, None, None, None, None, None


def router_topk(logits, k, mode="softmax", bias=None, n_group=1, topk_group=1, norm_topk=True, scale=1.0):
  """Returns (weights [T,K] fp32, indices [T,K] int32, scores [T,E] fp32).

  ``mode="softmax"``: Mixtral (softmax, top-k, renormalise).  ``mode="sigmoid"``: DeepSeek-V3
  (sigmoid, optional selection bias, group-limited top-k, normalise, scale)."""
  m = 0 if mode == "softmax" else 1
  e = logits.shape[-1]
  if logits.is_cuda and _kernels_ok() and e <= 256 and logits.dtype in (torch.float32, torch.bfloat16):
    return _RouterFn.apply(logits, bias, k, m, n_group, topk_group, norm_topk, scale)
  if m == 0:
    w, idx, s = ref.router_softmax_topk(logits, k, renormalize=norm_topk)
    return w * scale, idx.to(torch.int32), s
  w, idx, s = ref.router_sigmoid_group_topk(logits, bias, k, n_group, topk_group, norm_topk, scale)
  return w, idx.to(torch.int32), s


# ----------------------------------------------------------------------------- dispatch plan
@dataclass
class DispatchPlan:
  src_row: torch.Tensor      # [M] int32: token feeding padded row r, -1 for padding
  src_pair: torch.Tensor     # [M] int64: flat (token*K+slot) feeding row r, -1 for padding
  dest: torch.Tensor         # [T,K] int32: padded row of each pair, -1 if dropped
  tile_expert: torch.Tensor  # [M/128] int32
  k_offsets: torch.Tensor    # [E+1] int32 (multiples of 128)
  counts: torch.Tensor       # [E] rows per expert (after dropping)
  num_rows: int              # M (static upper bound)
  num_experts: int
  top_k: int
  row_align: int = 128       # expert segments are padded to this many rows (256 lets the CTA-pair GEMM run)


def build_dispatch_plan(idx: torch.Tensor, num_experts: int, capacity: int | None = None,
                        rows_per_group: int | None = None, use_kernel: bool | None = None,
                        row_align: int | None = None) -> DispatchPlan:
  """Sort (token, slot) pairs by expert into 128-aligned segments, entirely on the device.

  ``capacity``: maximum rows per expert *per group of ``rows_per_group`` consecutive tokens*
  (the reference's "dropping" mode limits each expert per batch row); pairs beyond it are
  dropped (``dest = -1``)."""
  t, k = idx.shape
  e = num_experts
  dev = idx.device
  if row_align is None:
    # 256-row segments let the grouped GEMMs use 256x256 CTA-pair tiles; worth the extra padding
    # when an expert sees about a thousand rows or more
    row_align = 256 if (capacity is None and (t * k) // e >= 1024) else ROW_ALIGN
  assert row_align in (128, 256)
  if use_kernel is None:
    use_kernel = capacity is None and idx.is_cuda and _kernels_ok() and e <= 256
  if use_kernel:
    return _build_dispatch_plan_kernel(idx, e, row_align)
  align = row_align
  flat = idx.reshape(-1).long()
  n = flat.numel()
  if capacity is not None:
    grp = (torch.arange(n, device=dev) // k) // (rows_per_group or t)
    key = grp * e + flat
    order_g = torch.argsort(key, stable=True)
    sk = key[order_g]
    first = torch.ones(n, dtype=torch.bool, device=dev)
    first[1:] = sk[1:] != sk[:-1]
    start = torch.where(first, torch.arange(n, device=dev), torch.zeros((), dtype=torch.long, device=dev))
    start = torch.cummax(start, 0)[0]
    rank_g = torch.empty(n, dtype=torch.long, device=dev)
    rank_g[order_g] = torch.arange(n, device=dev) - start
    flat = torch.where(rank_g < capacity, flat, torch.full_like(flat, e))   # dropped pairs go to a sentinel
  order = torch.argsort(flat, stable=True)
  sorted_e = flat[order]
  # (torch.bincount reads the largest value back to the host; a scatter-add of ones does not)
  counts_all = torch.zeros(e + 1, dtype=torch.long, device=dev).scatter_add_(0, flat, torch.ones_like(flat))
  counts = counts_all[:e]
  padded = (counts + align - 1) // align * align
  ends_pad = torch.cumsum(padded, 0)
  off_pad = ends_pad - padded
  off = torch.cumsum(counts_all, 0) - counts_all
  rank = torch.arange(n, device=dev) - off[sorted_e]
  valid = sorted_e < e
  dest_sorted = torch.where(valid, torch.cat([off_pad, off_pad.new_zeros(1)])[sorted_e] + rank,
                            torch.full_like(rank, -1))
  m = (n + align - 1) // align * align + e * align
  dest = torch.empty(n, dtype=torch.long, device=dev)
  dest[order] = dest_sorted
  src_pair = torch.full((m + 1,), -1, dtype=torch.long, device=dev)
  src_pair[torch.where(valid, dest_sorted, torch.full_like(dest_sorted, m))] = order
  src_pair = src_pair[:m]
  src_row = torch.where(src_pair >= 0, src_pair // k, src_pair).to(torch.int32)
  tile_start = torch.arange(m // ROW_ALIGN, device=dev) * ROW_ALIGN
  te = torch.bucketize(tile_start, ends_pad, right=True)
  tile_expert = torch.where(te < e, te, torch.full_like(te, -1)).to(torch.int32)
  k_offsets = torch.cat([ends_pad.new_zeros(1), ends_pad]).to(torch.int32)
  return DispatchPlan(src_row=src_row.contiguous(), src_pair=src_pair, dest=dest.view(t, k).to(torch.int32).contiguous(),
                      tile_expert=tile_expert.contiguous(), k_offsets=k_offsets.contiguous(), counts=counts, num_rows=m,
                      num_experts=e, top_k=k, row_align=align)


def _build_dispatch_plan_kernel(idx: torch.Tensor, e: int, align: int = ROW_ALIGN) -> DispatchPlan:
  """The same plan from one kernel launch (a stable counting sort in a single CTA) instead of about
  twenty-five torch kernels; nothing is read back to the host."""
  t, k = idx.shape
  dev = idx.device
  n = t * k
  m = (n + align - 1) // align * align + e * align
  idx32 = idx.to(torch.int32).contiguous()
  ints = torch.empty(e + (e + 1) + n + m + m // ROW_ALIGN, dtype=torch.int32, device=dev)
  counts, k_offsets, dest, src_row, tile_expert = torch.split(ints, [e, e + 1, n, m, m // ROW_ALIGN])
  src_pair = torch.empty(m, dtype=torch.int64, device=dev)
  check(lib().tpb_moe_plan(ptr(idx32), t, k, e, m, align, ptr(counts), ptr(k_offsets), ptr(dest), ptr(src_row), ptr(src_pair),
                           ptr(tile_expert), stream_ptr()), "moe_plan")
  return DispatchPlan(src_row=src_row, src_pair=src_pair, dest=dest.view(t, k), tile_expert=tile_expert,
                      k_offsets=k_offsets, counts=counts, num_rows=m, num_experts=e, top_k=k, row_align=align)


# ----------------------------------------------------------------------------- raw kernels
def gather_rows(x, src_row, row_scale=None):
  m, d = src_row.numel(), x.shape[-1]
  out = torch.empty(m, d, dtype=x.dtype, device=x.device)
  _debug.check_index("moe_gather", "src_row", src_row, 0, x.reshape(-1, d).shape[0], also_allowed=-1)
  check(lib().tpb_moe_gather(ptr(x), ptr(src_row), ptr(row_scale), ptr(out), m, d, stream_ptr()), "moe_gather")
  return out


def combine_rows(rows, dest, w=None):
  t, k = dest.shape
  out = torch.empty(t, rows.shape[-1], dtype=rows.dtype, device=rows.device)
  _debug.check_index("moe_combine", "dest", dest, 0, rows.shape[0], also_allowed=-1)
  check(lib().tpb_moe_combine(ptr(rows), ptr(dest), ptr(w), ptr(out), t, k, rows.shape[-1], stream_ptr()),
        "moe_combine")
  return out


def combine_dw(rows, dest, dout):
  t, k = dest.shape
  dw = torch.empty(t, k, dtype=torch.float32, device=rows.device)
  _debug.check_index("moe_combine_dw", "dest", dest, 0, rows.shape[0], also_allowed=-1)
  check(lib().tpb_moe_combine_dw(ptr(rows), ptr(dest), ptr(dout), ptr(dw), t, k, rows.shape[-1], stream_ptr()),
        "moe_combine_dw")
  return dw


def grouped_gemm_rows(a, b, plan: DispatchPlan, *, b_mn: bool, b2=None, epi=_lib.EPI_BF16, out=None, c2=None,
                      n_total=None):
  """out[rows of e] = a[rows of e] @ B[e]^T.  ``b``: [E, N, K] (``b_mn=False``) or [E, K, N]
  (``b_mn=True``).  With ``epi=EPI_SWIGLU``: ``b`` = gate, ``b2`` = up (or ``b`` holds both
  halves along N when ``b2`` is None)."""
  m, k = a.shape
  e = b.shape[0]
  n_one = b.shape[2] if b_mn else b.shape[1]
  swiglu = epi == _lib.EPI_SWIGLU
  n = n_total if n_total is not None else (2 * n_one if (swiglu and b2 is not None) else n_one)
  n_out = n // 2 if swiglu else n
  if out is None:
    out = torch.empty(m, n_out, dtype=torch.bfloat16, device=a.device)
  assert a.stride(1) == 1 and b.is_contiguous() and (b2 is None or b2.is_contiguous())
  ldb = b.stride(1)
  rc = lib().tpb_grouped_gemm_bf16(ptr(a), ptr(b), ptr(b2), ptr(out), m, n, k, e, a.stride(0), ldb, b.stride(0),
                                   out.stride(0), 0, int(b_mn), epi, 1.0, ptr(c2), c2.stride(0) if c2 is not None else 0,
                                   1, ptr(plan.tile_expert), None, 0, int(getattr(plan, "row_align", ROW_ALIGN)),
                                   stream_ptr())
  check(rc, f"grouped_gemm rows M={m} N={n} K={k} E={e}")
  return out


def grouped_gemm_wgrad(a_rows, b_rows, plan: DispatchPlan, out, accumulate: bool):
  """out[e] (+)= a_rows[rows of e]^T @ b_rows[rows of e];  out: [E, Da, Db] bf16 or fp32."""
  e, da, db = out.shape
  assert a_rows.shape[1] == da and b_rows.shape[1] == db and out.is_contiguous()
  if out.dtype == torch.float32:
    epi = _lib.EPI_F32_ACC if accumulate else _lib.EPI_F32
  else:
    epi = _lib.EPI_BF16_ACC if accumulate else _lib.EPI_BF16
  rc = lib().tpb_grouped_gemm_bf16(ptr(a_rows), ptr(b_rows), None, ptr(out), da, db, a_rows.shape[0], e,
                                   a_rows.stride(0), b_rows.stride(0), 0, out.stride(1), 1, 1, epi, 1.0, None, 0, 2,
                                   None, ptr(plan.k_offsets), out.stride(0), 0, stream_ptr())
  check(rc, f"grouped_gemm wgrad E={e} {da}x{db}")
  return out


# ----------------------------------------------------------------------------- grouped SwiGLU MLP
def _deliver_wgrad(w, compute):
  """Run ``compute(out, accumulate)`` into ``w.main_grad`` when present, else return a fresh gradient."""
  mg = getattr(w, "main_grad", None)
  if mg is not None:
    from .functional import overwrites_grad
    compute(mg, not overwrites_grad(w))
    w.grad_overwrite = False
    return None
  g = torch.empty(w.shape, dtype=torch.bfloat16, device=w.device)
  compute(g, False)
  return g


class _GroupedMLPFn(torch.autograd.Function):
  """y[t] = sum_k w[t,k] * down_e( silu(x[t] Wg_e) * (x[t] Wu_e) ),  e = idx[t,k]."""

  @staticmethod
  def forward(ctx, x, weights, w_gate, w_up, w_down, plan, fused_gate_up):
    xg = gather_rows(x, plan.src_row)
    need_grad = any(ctx.needs_input_grad)
    n2 = w_gate.shape[2] if fused_gate_up else 2 * w_gate.shape[2]
    gu = torch.empty(plan.num_rows, n2, dtype=x.dtype, device=x.device) if need_grad else None
    act = grouped_gemm_rows(xg, w_gate, plan, b_mn=True, b2=None if fused_gate_up else w_up, epi=_lib.EPI_SWIGLU, c2=gu,
                            n_total=n2)
    rows = grouped_gemm_rows(act, w_down, plan, b_mn=True)
    y = combine_rows(rows, plan.dest, weights)
    ctx.plan, ctx.fused = plan, fused_gate_up
    if need_grad:
      ctx.save_for_backward(x, weights, w_gate, w_up, w_down, xg, gu, act, rows)
    return y

  @staticmethod
  def backward(ctx, dy):
    from . import kernels as kk
    x, weights, w_gate, w_up, w_down, xg, gu, act, rows = ctx.saved_tensors
    plan, fused = ctx.plan, ctx.fused
    dy = dy.contiguous()
    f = gu.shape[1] // 2
    dweights = combine_dw(rows, plan.dest, dy) if ctx.needs_input_grad[1] else None
    flat_w = torch.cat([weights.reshape(-1).float(), weights.new_zeros(1, dtype=torch.float32)])
    row_scale = flat_w[plan.src_pair].contiguous()          # -1 (padding) picks the appended zero
    d_rows = gather_rows(dy, plan.src_row, row_scale)
    # down projection: rows = act @ Wd[e]  (Wd [E, F, D])
    dact = grouped_gemm_rows(d_rows, w_down, plan, b_mn=False)
    g_down = _deliver_wgrad(w_down, lambda out, acc: grouped_gemm_wgrad(act, d_rows, plan, out, acc))
    dgu = kk.swiglu_bwd(dact, gu)
    if fused:
      d_xg = grouped_gemm_rows(dgu, w_gate, plan, b_mn=False)
      g_gate = _deliver_wgrad(w_gate, lambda out, acc: grouped_gemm_wgrad(xg, dgu, plan, out, acc))
      g_up = None
    else:
      dg, du = dgu[:, :f], dgu[:, f:]
      d_xg = grouped_gemm_rows(dg, w_gate, plan, b_mn=False)
      grouped_gemm_rows(du, w_up, plan, b_mn=False, epi=_lib.EPI_BF16_ACC, out=d_xg)
      g_gate = _deliver_wgrad(w_gate, lambda out, acc: grouped_gemm_wgrad(xg, dg, plan, out, acc))
      g_up = _deliver_wgrad(w_up, lambda out, acc: grouped_gemm_wgrad(xg, du, plan, out, acc))
    dx = combine_rows(d_xg, plan.dest, None) if ctx.needs_input_grad[0] else None
    return dx, dweights, g_gate, g_up, g_down, None, None


def grouped_mlp_reference(x, weights, idx, w_gate, w_up, w_down, fused_gate_up=False, dropped=None):
  """Plain PyTorch: loop over experts (the oracle and the CPU path)."""
  t, k = idx.shape
  y = torch.zeros_like(x, dtype=torch.float32)
  e = w_gate.shape[0]
  for ex in range(e):
    sel = idx == ex
    if dropped is not None:
      sel = sel & ~dropped
    tok, slot = torch.nonzero(sel, as_tuple=True)
    if tok.numel() == 0:
      continue
    xi = x[tok]
    if fused_gate_up:
      gu = xi @ w_gate[ex]
      f = gu.shape[-1] // 2
      h = F.silu(gu[:, :f]) * gu[:, f:]
    else:
      h = F.silu(xi @ w_gate[ex]) * (xi @ w_up[ex])
    out = (h @ w_down[ex]).float() * weights[tok, slot].float()[:, None]
    y.index_add_(0, tok, out)
  return y.to(x.dtype)


def grouped_mlp(x, weights, idx, w_gate, w_up, w_down, *, fused_gate_up=False, capacity=None, rows_per_group=None):
  """Routed SwiGLU experts.  x [T,D]; weights/idx [T,K]; w_gate/w_up [E,D,F]; w_down [E,F,D]
  (``fused_gate_up``: w_gate is [E,D,2F] = [gate | up] and w_up is ignored)."""
  e = w_gate.shape[0]
  f = w_down.shape[1]
  ok = (_kernels_ok(x, w_gate, w_down) and x.shape[-1] % 64 == 0 and f % 64 == 0 and x.is_cuda)
  if ok:
    plan = build_dispatch_plan(idx, e, capacity, rows_per_group)
    wu = w_gate if fused_gate_up else w_up
    return _GroupedMLPFn.apply(x.contiguous(), weights.float().contiguous(), w_gate, wu, w_down, plan, fused_gate_up)
  dropped = None
  if capacity is not None:
    dropped = build_dispatch_plan(idx, e, capacity, rows_per_group).dest < 0
  return grouped_mlp_reference(x, weights, idx, w_gate, w_up, w_down, fused_gate_up, dropped)
