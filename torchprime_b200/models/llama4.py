"""Llama-4 text decoder (Scout-style): interleaved RoPE / NoPE layers, optional weight-less QK
L2 norm, attention temperature tuning on NoPE layers, top-1 sigmoid-routed MoE with an
always-on shared expert.

Behavioural reference: torchprime/torch_xla_models/model/llama4/model.py:85-727.  State-dict
names match it (``feed_forward.experts.gate_up_proj [E,D,2F]``, ``experts.down_proj [E,F,D]``,
``feed_forward.router.weight``, ``feed_forward.shared_expert.*``).  MoE implementations:

* ``original``   every expert sees every token scaled by its (mostly zero) score — the dense oracle;
* ``sequential`` the same math one expert at a time;
* ``expert_parallel`` / ``gmm``  tokens are sorted by their selected expert and run through the
  grouped tcgen05 GEMMs (and through all-to-all dispatch when the expert axis is > 1).

In every variant the router score multiplies the expert *input* (as in the reference), and
unselected experts contribute exactly zero.  ``attention_chunk_size`` is parsed but, as in the
reference (model.py:544-548), chunked attention is not applied.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from ..ops import moe as moe_ops
from ..ops import reference as ref
from ..parallel.collectives import copy_to_tp, reduce_from_tp
from ..utils.profiling import trace_scope
from . import rope
from .base import BaseCausalLM
from .llama import CausalLMHead, LlamaEmbedding, LlamaRMSNorm


class Llama4TextRMSNorm(LlamaRMSNorm):
  pass


class Llama4TextL2Norm(nn.Module):
  def __init__(self, eps: float = 1e-6):
    super().__init__()
    self.eps = eps

  def forward(self, x):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x)

  def extra_repr(self):
    return f"eps={self.eps}"


class Llama4TextMLP(nn.Module):
  def __init__(self, config, intermediate_size=None):
    super().__init__()
    inter = intermediate_size or config.intermediate_size
    self.gate_proj = nn.Linear(config.hidden_size, inter, bias=False)
    self.up_proj = nn.Linear(config.hidden_size, inter, bias=False)
    self.down_proj = nn.Linear(inter, config.hidden_size, bias=False)
    self.tp_group = None

  def forward(self, x, partial=False):
    """Tensor parallel (``tp_group`` set by the engine): gate/up column-parallel, down row-parallel;
    ``partial`` returns this rank's partial sum for a caller that reduces it with other terms."""
    tp = getattr(self, "tp_group", None)
    if tp is not None and self.gate_proj.weight.shape[0] == self.gate_proj.out_features:
      tp = None        # this MLP's weights are not named by the sharding config: replicated, nothing to reduce
    if tp is None:
      act = ops.linear_swiglu(x, self.gate_proj.weight, self.up_proj.weight)
      return ops.linear(act, self.down_proj.weight)
    act = ops.linear_swiglu(copy_to_tp(x, tp), self.gate_proj.weight, self.up_proj.weight)
    y = ops.linear(act, self.down_proj.weight)
    return y if partial else reduce_from_tp(y, tp)


class Llama4TextExperts(nn.Module):
  def __init__(self, config):
    super().__init__()
    self.num_experts = config.num_local_experts
    self.intermediate_size = config.intermediate_size
    self.hidden_size = config.hidden_size
    self.expert_dim = self.intermediate_size
    self.gate_up_proj = nn.Parameter(torch.empty(self.num_experts, self.hidden_size, 2 * self.expert_dim))
    self.down_proj = nn.Parameter(torch.empty(self.num_experts, self.expert_dim, self.hidden_size))
    for w in (self.gate_up_proj, self.down_proj):
      if not w.is_meta:
        nn.init.normal_(w, mean=0.0, std=float(config.get("initializer_range", 0.02)))

  def forward(self, hidden_states):
    """hidden_states: [E * T, D] (expert-major) -> [E * T, D]."""
    x = hidden_states.view(self.num_experts, -1, self.hidden_size)
    gate, up = torch.bmm(x, self.gate_up_proj).chunk(2, dim=-1)
    return torch.bmm(up * F.silu(gate), self.down_proj).view(-1, self.hidden_size)


class Llama4TextMoe(nn.Module):
  """``original`` implementation (dense replication; memory-hungry, the correctness oracle)."""

  def __init__(self, config):
    super().__init__()
    self.top_k = config.num_experts_per_tok
    self.hidden_dim = config.hidden_size
    self.num_experts = config.num_local_experts
    self.experts = Llama4TextExperts(config)
    self.router = nn.Linear(config.hidden_size, config.num_local_experts, bias=False)
    self.shared_expert = Llama4TextMLP(config)
    self.ep = None
    self.tp_group = None   # set by the engine: experts and the shared expert split along the FFN dimension

  def _to_tp(self, t):
    """In front of a tensor-parallel GEMM: identity forward, gradient summed over the tensor group."""
    return t if self.tp_group is None else copy_to_tp(t, self.tp_group)

  def _finish(self, x, routed):
    """shared expert + routed experts; with tensor parallelism both are partial sums, reduced once."""
    if self.tp_group is None:
      return self.shared_expert(x) + routed
    return reduce_from_tp(self.shared_expert(x, partial=True) + routed, self.tp_group)

  def route(self, x):
    logits = F.linear(x, self.router.weight)
    top_v, top_i = torch.topk(logits, self.top_k, dim=1)
    return logits, top_v, top_i

  def forward(self, hidden_states):
    with trace_scope("Llama4TextMoe"):
      x = hidden_states.reshape(-1, self.hidden_dim)
      logits, top_v, top_i = self.route(x)
      scores = torch.full_like(logits, float("-inf")).scatter_(1, top_i, top_v).transpose(0, 1)
      scores = torch.sigmoid(scores.float()).to(x.dtype)
      routed_in = self._to_tp(x.repeat(self.num_experts, 1) * scores.reshape(-1, 1))
      routed_out = self.experts(routed_in)
      out = self._finish(x, routed_out.reshape(self.num_experts, -1, self.hidden_dim).sum(dim=0))
      return out, scores


class Llama4TextMoeSequential(Llama4TextMoe):
  def forward(self, hidden_states):
    with trace_scope("Llama4TextMoe"):
      x = hidden_states.reshape(-1, self.hidden_dim)
      logits, top_v, top_i = self.route(x)
      sparse = torch.sigmoid(torch.full_like(logits, float("-inf")).scatter_(1, top_i, top_v).float()).to(x.dtype)
      x_tp, sparse_tp = self._to_tp(x), self._to_tp(sparse)
      routed = 0
      for i in range(self.num_experts):
        gu = (x_tp @ self.experts.gate_up_proj[i]) * sparse_tp[:, i:i + 1]
        gate, up = gu.chunk(2, dim=-1)
        routed = routed + (up * F.silu(gate)) @ self.experts.down_proj[i]
      return self._finish(x, routed), sparse.transpose(0, 1)


class Llama4TextMoeExpertParallelism(Llama4TextMoe):
  """Sorted dispatch + grouped GEMMs (+ all-to-all when the expert axis is sharded)."""

  def forward(self, hidden_states):
    with trace_scope("Llama4TextMoe"):
      x = hidden_states.reshape(-1, self.hidden_dim)
      logits, top_v, top_i = self.route(x)
      score = torch.sigmoid(top_v.float()).to(x.dtype)                      # [T, K]
      out = 0
      ones = torch.ones(x.shape[0], 1, dtype=torch.float32, device=x.device)
      for k in range(self.top_k):                                           # Llama-4 uses top-1
        xin = self._to_tp(x * score[:, k:k + 1])
        idx = top_i[:, k:k + 1].to(torch.int32)
        if self.ep is not None:
          routed = self.ep.grouped_mlp(xin, ones, idx, self.experts.gate_up_proj, None, self.experts.down_proj,
                                       fused_gate_up=True)
        else:
          routed = moe_ops.grouped_mlp(xin, ones, idx, self.experts.gate_up_proj, None, self.experts.down_proj,
                                       fused_gate_up=True)
        out = out + routed
      scores = torch.sigmoid(torch.full_like(logits, float("-inf")).scatter_(1, top_i, top_v).float()).to(x.dtype)
      return self._finish(x, out), scores.transpose(0, 1)


_MOE_IMPLS = {"original": Llama4TextMoe, "sequential": Llama4TextMoeSequential,
              "expert_parallel": Llama4TextMoeExpertParallelism, "expert_parallelism": Llama4TextMoeExpertParallelism,
              "gmm": Llama4TextMoeExpertParallelism}


class Llama4TextAttention(nn.Module):
  def __init__(self, config, layer_idx=None):
    super().__init__()
    self.config = config
    self.layer_idx = layer_idx
    self.num_attention_heads = config.num_attention_heads
    self.num_key_value_heads = config.num_key_value_heads
    self.head_dim = config.hidden_size // config.num_attention_heads
    if self.head_dim * config.num_attention_heads != config.hidden_size:
      raise ValueError(f"hidden_size must be divisible by num_attention_heads (got `hidden_size`: "
                       f"{config.hidden_size} and `num_attention_heads`: {config.num_attention_heads}).")
    self.scaling = config.head_dim ** -0.5
    self.attn_scale = config.attn_scale
    self.floor_scale = config.floor_scale
    self.attn_temperature_tuning = config.attn_temperature_tuning
    nope = config.get("no_rope_layers", None)
    self.use_rope = bool(nope and layer_idx < len(nope) and nope[layer_idx])
    bias = bool(config.get("attention_bias", False))
    self.q_proj = nn.Linear(config.hidden_size, self.num_attention_heads * self.head_dim, bias=bias)
    self.k_proj = nn.Linear(config.hidden_size, self.num_key_value_heads * self.head_dim, bias=bias)
    self.v_proj = nn.Linear(config.hidden_size, self.num_key_value_heads * self.head_dim, bias=bias)
    self.o_proj = nn.Linear(config.hidden_size, config.hidden_size, bias=bias)
    if config.get("use_qk_norm", False) and self.use_rope:
      self.qk_norm = Llama4TextL2Norm(config.rms_norm_eps)
    self.attention_kernel = config.get("attention_kernel", None)
    self.tp_group = None   # set by the engine: q/k/v column-parallel (heads split), o row-parallel

  def forward(self, x, rope_cos, rope_sin, position_ids=None, segment_ids=None):
    with trace_scope("Llama4TextAttention"):
      b, s, _ = x.shape
      d = self.head_dim
      hq, hkv = self.q_proj.weight.shape[0] // d, self.k_proj.weight.shape[0] // d   # local heads
      if self.tp_group is not None:
        x = copy_to_tp(x, self.tp_group)
      bias = None
      if self.q_proj.bias is not None:
        bias = torch.cat([self.q_proj.bias, self.k_proj.bias, self.v_proj.bias])
      qkv = ops.linear(x, [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], bias=bias)
      if self.use_rope:
        qkv = ops.rope_inplace(qkv, rope_cos, rope_sin, hq + hkv, d, s, pos=position_ids, interleaved=True)
      q = qkv[..., : hq * d].view(b, s, hq, d)
      k = qkv[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
      v = qkv[..., (hq + hkv) * d:].view(b, s, hkv, d)
      if hasattr(self, "qk_norm"):
        q, k = self.qk_norm(q), self.qk_norm(k)
      if self.attn_temperature_tuning and not self.use_rope:
        pos = torch.arange(s, device=x.device).float() if position_ids is None else position_ids.view(b, s).float()
        scales = torch.log(torch.floor((pos + 1.0) / self.floor_scale) + 1.0) * self.attn_scale + 1.0
        q = (q * scales.view(-1, s, 1, 1)).to(q.dtype)
      if self.attention_kernel is None and not x.is_cuda:
        o = ref.attention(q, k, v, causal=True, scale=self.scaling, q_segment_ids=segment_ids)
      else:
        o = ops.attention(q, k, v, causal=True, scale=self.scaling, q_segment_ids=segment_ids)
      if self.tp_group is not None:
        out = reduce_from_tp(ops.linear(o.reshape(b, s, hq * d), self.o_proj.weight), self.tp_group)
        return out if self.o_proj.bias is None else out + self.o_proj.bias
      return ops.linear(o.reshape(b, s, hq * d), self.o_proj.weight, bias=self.o_proj.bias)


class Llama4TextDecoderLayer(nn.Module):
  def __init__(self, config, layer_idx):
    super().__init__()
    self.hidden_size = config.hidden_size
    self.layer_idx = layer_idx
    self.self_attn = Llama4TextAttention(config, layer_idx)
    nope = config.get("no_rope_layers", None)
    self.use_chunked_attention = config.get("attention_chunk_size", None) is not None and bool(
      nope and layer_idx < len(nope) and nope[layer_idx])
    self.is_moe_layer = layer_idx in list(config.moe_layers)
    if self.is_moe_layer:
      self.feed_forward = _MOE_IMPLS.get(str(config.get("moe_implementation", "original")), Llama4TextMoe)(config)
    else:
      self.feed_forward = Llama4TextMLP(config, intermediate_size=config.intermediate_size_mlp)
    self.input_layernorm = Llama4TextRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
    self.post_attention_layernorm = Llama4TextRMSNorm(config.hidden_size, eps=config.rms_norm_eps)

  def forward(self, hidden_states, rope_cos, rope_sin, position_ids=None, segment_ids=None, cp=None):
    with trace_scope("Llama4TextDecoderLayer"):
      h = hidden_states + self.self_attn(self.input_layernorm(hidden_states), rope_cos, rope_sin, position_ids,
                                         segment_ids)
      ff = self.feed_forward(self.post_attention_layernorm(h))
      if self.is_moe_layer:
        ff, _scores = ff
      return h + ff.view(h.shape)


class Llama4TextModel(nn.Module):
  def __init__(self, config):
    super().__init__()
    self.vocab_size = config.vocab_size
    self.embed_tokens = LlamaEmbedding(config.vocab_size, config.hidden_size)
    self.layers = nn.ModuleList([Llama4TextDecoderLayer(config, i) for i in range(config.num_hidden_layers)])
    self.norm = Llama4TextRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
    scaling = config.get("rope_scaling", None)
    if scaling is not None:
      scaling = rope.RopeScaling(**{k: scaling[k] for k in ("factor", "low_freq_factor", "high_freq_factor",
                                                           "original_context_len") if k in scaling})
    self.register_buffer("inv_freq", rope.llama3_rope_frequencies(config.head_dim, float(config.rope_theta), scaling),
                         persistent=False)
    self._rope_cache = None

  def rope_tables(self, seq_len, device, position_ids=None):
    need = seq_len if position_ids is None else max(seq_len, int(getattr(self, "max_rope_positions", 0)) or
                                                    int(position_ids.max().item()) + 1)
    c = self._rope_cache
    if c is None or c[0].shape[0] < need or c[0].device != device:
      self._rope_cache = rope.rope_tables(self.inv_freq.float(), max(need, 1), device)
    return self._rope_cache


class Llama4TextForCausalLM(BaseCausalLM):
  def __init__(self, config):
    super().__init__()
    self.config = config
    self.model = Llama4TextModel(config)
    self.vocab_size = config.vocab_size
    self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
    object.__setattr__(self, "_head", CausalLMHead(self.model.norm, self.lm_head, config.vocab_size))
    self.apply(self._init_weights)
    self.return_logits = True
    self.cp = None

  def param_init_kind(self, full_name, module, pname):
    if isinstance(module, Llama4TextExperts):
      return "normal"
    return None

  def tp_layout(self, name: str):
    """Dimension along which a tensor-parallel weight is split (None: replicated over the tensor axis);
    ``(dim, 2)`` for the fused ``gate_up_proj [E, D, 2F]``, whose gate and up halves are sliced one by
    one.  The reference's configs (llama4-fsdp-tp-ep.yaml:17-19) put ``tensor`` on the hidden dimension
    of the expert weights for its partitioning compiler; the explicit forward here splits the FFN
    dimension, which needs one reduction per block instead of one per GEMM."""
    if ".self_attn." in name and name.endswith("_proj.weight"):
      return 1 if ".o_proj." in name else 0
    if name.endswith("experts.gate_up_proj"):
      return (2, 2)
    if name.endswith("experts.down_proj"):
      return 1
    if name.endswith(("gate_proj.weight", "up_proj.weight")):
      return 0
    if name.endswith("down_proj.weight"):
      return 1
    return None

  def forward(self, input_ids, labels=None, attention_mask=None, position_ids=None, segment_ids=None,
              labels_are_shifted=False):
    with trace_scope("Llama4TextForCausalLM"):
      b, s = input_ids.shape
      h = self.model.embed_tokens(input_ids)
      cos, sin = self.model.rope_tables(s, h.device, position_ids)
      pos = position_ids.reshape(-1).to(torch.int32).contiguous() if position_ids is not None else None
      for layer in self.model.layers:
        h = layer(h, cos, sin, pos, segment_ids, self.cp)
      targets = None
      if labels is not None:
        targets = labels if labels_are_shifted else ref.shift_labels(labels)
      return self._head(h, targets, want_logits=self.return_logits or labels is None)
