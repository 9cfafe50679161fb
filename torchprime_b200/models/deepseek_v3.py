"""DeepSeek-V3 / V2-Lite style model: multi-head latent attention (MLA) + routed MoE.

Behavioural reference: torchprime/torch_xla_models/model/deepseek_v3/model.py:32-562 and
model_utils.py:4-119 (grouped <-> per-expert checkpoint key conversion).  State-dict names
match it: ``self_attn.{q_proj | q_a_proj, q_a_layernorm, q_b_proj}``,
``kv_a_proj_with_mqa``, ``kv_a_layernorm``, ``kv_b_proj``, ``o_proj``; dense layers
``mlp.{gate,up,down}_proj``; MoE layers ``mlp.gate.{weight,e_score_correction_bias}``,
``mlp.grouped.{W_gate,W_up,W_down}`` and ``mlp.shared_experts.*``.

Layout choices for the B200 kernels: activations stay token-major; RoPE rotates the 64-wide
slice at the end of each 192-wide query head (and the single shared key slice) in place; the
attention kernel is instantiated for (qk 192, v 128); routed experts run through the grouped
tcgen05 GEMMs (ops/moe.py).  The interleaved RoPE variant keeps the (even, odd) pair layout
instead of permuting to halves — q.k is invariant under a permutation applied to both.

Softmax scale: by default ``qk_head_dim^-0.5 * mscale^2`` (the published definition); the
reference applies ``1/sqrt(v_head_dim)`` because its attention wrapper derives the scale from
V (attention.py:58) — ``compat_reference_scale: true`` reproduces that.
"""

from __future__ import annotations

import math

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


class DeepseekV3RMSNorm(LlamaRMSNorm):
  pass


class DeepseekV3MLP(nn.Module):
  def __init__(self, config, hidden_size=None, intermediate_size=None):
    super().__init__()
    self.hidden_size = hidden_size or config.hidden_size
    self.intermediate_size = intermediate_size or config.intermediate_size
    self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
    self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
    self.down_proj = nn.Linear(self.intermediate_size, self.hidden_size, bias=False)
    self.tp_group = None   # set by the engine: gate/up column-parallel, down row-parallel

  def forward(self, x, residual=None, partial=False):
    """``partial`` (tensor parallel only): return this rank's partial sum, the caller reduces."""
    if self.tp_group is None:
      act = ops.linear_swiglu(x, self.gate_proj.weight, self.up_proj.weight)
      return ops.linear(act, self.down_proj.weight, residual=residual)
    act = ops.linear_swiglu(copy_to_tp(x, self.tp_group), self.gate_proj.weight, self.up_proj.weight)
    y = ops.linear(act, self.down_proj.weight)
    if partial:
      return y
    y = reduce_from_tp(y, self.tp_group)
    return y if residual is None else y + residual


class DeepseekV3TopkRouter(nn.Module):
  def __init__(self, config):
    super().__init__()
    self.top_k = config.num_experts_per_tok
    self.n_routed_experts = config.n_routed_experts
    self.routed_scaling_factor = float(config.routed_scaling_factor)
    self.n_group = int(config.n_group)
    self.topk_group = int(config.topk_group)
    self.norm_topk_prob = bool(config.norm_topk_prob)
    self.weight = nn.Parameter(torch.empty(self.n_routed_experts, config.hidden_size))
    if not self.weight.is_meta:
      nn.init.normal_(self.weight, std=float(config.get("initializer_range", 0.02)))
    self.register_buffer("e_score_correction_bias", torch.zeros(self.n_routed_experts, device="cpu"))

  def forward(self, x):
    logits = F.linear(x.reshape(-1, x.shape[-1]).float(), self.weight.float())
    bias = self.e_score_correction_bias
    if bias.device != logits.device:
      bias = bias.to(logits.device)
    w, idx, _ = moe_ops.router_topk(logits, self.top_k, mode="sigmoid", bias=bias, n_group=self.n_group,
                                    topk_group=self.topk_group, norm_topk=self.norm_topk_prob,
                                    scale=self.routed_scaling_factor)
    return idx, w


class GroupedMoEWeights(nn.Module):
  def __init__(self, E: int, D: int, I: int, dtype=None):
    super().__init__()
    self.W_gate = nn.Parameter(torch.empty(E, D, I))
    self.W_up = nn.Parameter(torch.empty(E, D, I))
    self.W_down = nn.Parameter(torch.empty(E, I, D))
    for w in (self.W_gate, self.W_up, self.W_down):
      if not w.is_meta:
        nn.init.kaiming_uniform_(w, a=math.sqrt(5))


class DeepseekV3MoE(nn.Module):
  def __init__(self, config):
    super().__init__()
    self.config = config
    self.gate = DeepseekV3TopkRouter(config)
    self.grouped = GroupedMoEWeights(config.n_routed_experts, config.hidden_size, config.moe_intermediate_size)
    self.shared_experts = DeepseekV3MLP(config, intermediate_size=config.moe_intermediate_size * config.n_shared_experts)
    self.use_gmm = bool(config.get("use_gmm_kernel_for_moe", True))
    self.num_experts = config.n_routed_experts
    self.ep = None
    self.tp_group = None   # set by the engine: routed and shared experts split along their FFN dimension

  def forward(self, hidden_states, residual=None):
    with trace_scope("DeepseekV3MoE"):
      b, s, d = hidden_states.shape
      x = hidden_states.reshape(-1, d)
      idx, w = self.gate(x)
      g = self.grouped
      tp = self.tp_group
      if tp is not None:
        # partial sums over the FFN slices: gradients into the tokens and the routing weights are
        # summed over the tensor group, routed + shared outputs are reduced once
        x, w = copy_to_tp(x, tp), copy_to_tp(w, tp)
      if self.ep is not None:
        routed = self.ep.grouped_mlp(x, w, idx, g.W_gate, g.W_up, g.W_down)
      elif self.use_gmm:
        routed = moe_ops.grouped_mlp(x, w, idx, g.W_gate, g.W_up, g.W_down)
      else:
        routed = moe_ops.grouped_mlp_reference(x, w, idx, g.W_gate, g.W_up, g.W_down)
      routed = routed.reshape(b, s, d)
      if tp is not None:
        out = reduce_from_tp(routed + self.shared_experts(hidden_states, partial=True), tp)
        return out if residual is None else out + residual
      if residual is not None:
        routed = routed + residual
      return self.shared_experts(hidden_states, residual=routed)


def _yarn_mscale(scale: float, m: float) -> float:
  return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0


class DeepseekV3Attention(nn.Module):
  """Multi-head latent attention."""

  def __init__(self, config, layer_idx=None):
    super().__init__()
    self.config = config
    self.layer_idx = layer_idx
    self.num_heads = config.num_attention_heads
    self.q_lora_rank = config.get("q_lora_rank", None)
    self.qk_rope_head_dim = config.qk_rope_head_dim
    self.kv_lora_rank = config.kv_lora_rank
    self.v_head_dim = config.v_head_dim
    self.qk_nope_head_dim = config.qk_nope_head_dim
    self.qk_head_dim = config.qk_head_dim
    bias = bool(config.get("attention_bias", False))
    if not self.q_lora_rank:
      self.q_proj = nn.Linear(config.hidden_size, self.num_heads * self.qk_head_dim, bias=False)
    else:
      self.q_a_proj = nn.Linear(config.hidden_size, self.q_lora_rank, bias=bias)
      self.q_a_layernorm = DeepseekV3RMSNorm(self.q_lora_rank)
      self.q_b_proj = nn.Linear(self.q_lora_rank, self.num_heads * self.qk_head_dim, bias=False)
    self.kv_a_proj_with_mqa = nn.Linear(config.hidden_size, self.kv_lora_rank + self.qk_rope_head_dim, bias=bias)
    self.kv_a_layernorm = DeepseekV3RMSNorm(self.kv_lora_rank)
    self.kv_b_proj = nn.Linear(self.kv_lora_rank, self.num_heads * (self.qk_nope_head_dim + self.v_head_dim),
                               bias=False)
    self.o_proj = nn.Linear(self.num_heads * self.v_head_dim, config.hidden_size, bias=bias)
    self.scaling = self.qk_head_dim ** (-0.5)
    rs = config.get("rope_scaling", None)
    if rs is not None and rs.get("mscale_all_dim", 0):
      m = _yarn_mscale(rs["factor"], rs["mscale_all_dim"])
      self.scaling = self.scaling * m * m
    if config.get("compat_reference_scale", False):
      self.scaling = 1.0 / math.sqrt(self.v_head_dim)
    self.rope_interleave = bool(config.get("rope_interleave", True))
    self.attention_kernel = config.get("attention_kernel", None)
    self.tp_group = None   # set by the engine: heads split (q_proj / q_b_proj / kv_b_proj rows, o_proj columns)

  def forward(self, x, rope_cos, rope_sin, residual=None, position_ids=None, segment_ids=None, cp=None):
    with trace_scope("DeepseekV3Attention"):
      b, s, _ = x.shape
      dn, dr, dv = self.qk_nope_head_dim, self.qk_rope_head_dim, self.v_head_dim
      tp = self.tp_group
      # Tensor parallel: the low-rank "a" projections and their norms are replicated; copy_to_tp sits
      # right in front of the head-split GEMMs, so that the replicated parameters see gradients that are
      # already summed over the ranks' heads.
      to_tp = (lambda t: copy_to_tp(t, tp)) if tp is not None else (lambda t: t)
      if not self.q_lora_rank:
        q = ops.linear(to_tp(x), self.q_proj.weight)
      else:
        q = ops.linear(to_tp(self.q_a_layernorm(ops.linear(x, self.q_a_proj.weight, bias=self.q_a_proj.bias))),
                       self.q_b_proj.weight)
      h = q.shape[-1] // (dn + dr)      # local heads (all of them without tensor parallelism)
      # rotate the last dr columns of every (dn + dr)-wide query head
      q = ops.rope_slices(q, rope_cos, rope_sin, h, dr, s, col0=dn, head_stride=dn + dr, pos=position_ids,
                          interleaved=self.rope_interleave)
      ckv = ops.linear(x, self.kv_a_proj_with_mqa.weight, bias=self.kv_a_proj_with_mqa.bias)
      ckv = ops.rope_slices(ckv, rope_cos, rope_sin, 1, dr, s, col0=self.kv_lora_rank, head_stride=dr,
                            pos=position_ids, interleaved=self.rope_interleave)
      k_lat, k_rot = ckv[..., : self.kv_lora_rank], to_tp(ckv[..., self.kv_lora_rank:])
      kv = ops.linear(to_tp(self.kv_a_layernorm(k_lat.contiguous())), self.kv_b_proj.weight).view(b, s, h, dn + dv)
      k_nope, v = kv[..., :dn], kv[..., dn:]
      k = torch.cat([k_nope, k_rot[:, :, None, :].expand(b, s, h, dr)], dim=-1)
      q4 = q.view(b, s, h, dn + dr)
      v = v.contiguous()
      if cp is not None:
        o = cp.attention(q4, k, v, segment_ids=segment_ids, scale=self.scaling)
      elif self.attention_kernel is None and not x.is_cuda:
        o = ref.attention(q4, k, v, causal=True, scale=self.scaling, q_segment_ids=segment_ids)
      else:
        o = ops.attention(q4, k, v, causal=True, scale=self.scaling, q_segment_ids=segment_ids)
      o = o.reshape(b, s, h * dv)
      if tp is not None:
        out = reduce_from_tp(ops.linear(o, self.o_proj.weight), tp)
        if self.o_proj.bias is not None:
          out = out + self.o_proj.bias
        return out if residual is None else out + residual
      if self.o_proj.bias is not None:
        out = ops.linear(o, self.o_proj.weight, bias=self.o_proj.bias)
        return out if residual is None else out + residual
      return ops.linear(o, self.o_proj.weight, residual=residual)


class DeepseekV3DecoderLayer(nn.Module):
  def __init__(self, config, layer_idx: int):
    super().__init__()
    self.hidden_size = config.hidden_size
    self.self_attn = DeepseekV3Attention(config, layer_idx)
    self.is_moe = layer_idx >= config.first_k_dense_replace
    self.mlp = DeepseekV3MoE(config) if self.is_moe else DeepseekV3MLP(config)
    self.input_layernorm = DeepseekV3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
    self.post_attention_layernorm = DeepseekV3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

  def forward(self, hidden_states, rope_cos, rope_sin, position_ids=None, segment_ids=None, cp=None):
    with trace_scope("DeepseekV3DecoderLayer"):
      x = self.input_layernorm(hidden_states)
      h = self.self_attn(x, rope_cos, rope_sin, residual=hidden_states, position_ids=position_ids,
                         segment_ids=segment_ids, cp=cp)
      x = self.post_attention_layernorm(h)
      return self.mlp(x, residual=h)


class DeepseekV3Model(nn.Module):
  def __init__(self, config):
    super().__init__()
    self.config = config
    self.vocab_size = config.vocab_size
    self.embed_tokens = LlamaEmbedding(config.vocab_size, config.hidden_size)
    self.layers = nn.ModuleList([DeepseekV3DecoderLayer(config, i) for i in range(config.num_hidden_layers)])
    self.norm = DeepseekV3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
    rope_cfg = type(config)(config)
    rope_cfg["head_dim"] = config.qk_rope_head_dim
    inv_freq, self.attention_factor = rope.yarn_rope_frequencies(rope_cfg)
    self.register_buffer("inv_freq", inv_freq, persistent=False)
    self._rope_cache = None

  def rope_tables(self, seq_len, device, position_ids=None):
    need = seq_len if position_ids is None else max(seq_len, int(getattr(self, "max_rope_positions", 0)) or
                                                    int(position_ids.max().item()) + 1)
    c = self._rope_cache
    if c is None or c[0].shape[0] < need or c[0].device != device:
      self._rope_cache = rope.rope_tables(self.inv_freq.float(), max(need, 1), device, self.attention_factor)
    return self._rope_cache


class DeepseekV3ForCausalLM(BaseCausalLM):
  def __init__(self, config):
    super().__init__()
    self.config = config
    self.model = DeepseekV3Model(config)
    self.vocab_size = config.vocab_size
    self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
    object.__setattr__(self, "_head", CausalLMHead(self.model.norm, self.lm_head, config.vocab_size))
    self.apply(self._init_weights)
    self.return_logits = True
    self.cp = None

  def param_init_kind(self, full_name, module, pname):
    if isinstance(module, (GroupedMoEWeights, DeepseekV3TopkRouter)):
      return "normal"
    return None

  def tp_layout(self, name: str):
    """Dimension along which a tensor-parallel weight is split (None: replicated over the tensor axis).
    The sharding configs of the reference describe hidden-dimension sharding for a partitioning
    compiler (torchprime/torch_xla_models/configs/model/sharding/deepseek-fsdp-tp-ep.yaml:4-17); the
    explicit forward here is column- / row-parallel: attention by heads (q_proj / q_b_proj / kv_b_proj
    rows, o_proj columns; the low-rank ``*_a`` projections and their norms stay replicated), dense and
    shared MLPs and the grouped experts along their FFN dimension."""
    if ".self_attn." in name:
      if name.endswith(("q_proj.weight", "q_b_proj.weight", "kv_b_proj.weight")):
        return 0
      return 1 if name.endswith("o_proj.weight") else None
    if name.endswith(("gate_proj.weight", "up_proj.weight")):
      return 0
    if name.endswith("down_proj.weight"):
      return 1
    if name.endswith(("grouped.W_gate", "grouped.W_up")):
      return 2
    if name.endswith("grouped.W_down"):
      return 1
    return None

  def convert_loaded_state_dict(self, state: dict) -> dict:
    """HF checkpoints store one Linear triple per expert; fold them into the grouped tensors."""
    if any(".mlp.experts." in k for k in state):
      return convert_hf_state_dict_for_grouped_moe(state, self.config)
    return state

  def forward(self, input_ids, labels=None, attention_mask=None, position_ids=None, segment_ids=None,
              labels_are_shifted=False):
    with trace_scope("DeepseekV3ForCausalLM"):
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


# ----------------------------------------------------------------------------------------
# Checkpoint key conversion between the HF per-expert layout and the grouped layout.
# ----------------------------------------------------------------------------------------
def convert_hf_state_dict_for_grouped_moe(hf_state: dict, config) -> dict:
  """``...mlp.experts.{i}.{gate,up,down}_proj.weight`` ([out,in] each) ->
  ``...mlp.grouped.{W_gate [E,D,I], W_up [E,D,I], W_down [E,I,D]}``; other keys unchanged."""
  out = dict(hf_state)
  e = config.n_routed_experts
  for layer in range(config.num_hidden_layers):
    if layer < config.first_k_dense_replace:
      continue
    base = f"model.layers.{layer}.mlp"
    if f"{base}.experts.0.gate_proj.weight" not in hf_state:
      continue
    for ours, theirs in (("W_gate", "gate_proj"), ("W_up", "up_proj"), ("W_down", "down_proj")):
      mats = []
      for i in range(e):
        key = f"{base}.experts.{i}.{theirs}.weight"
        mats.append(out.pop(key).t().contiguous())
      out[f"{base}.grouped.{ours}"] = torch.stack(mats, dim=0)
  return out


def revert_grouped_moe_to_hf_state_dict(state: dict, config) -> dict:
  """Inverse of :func:`convert_hf_state_dict_for_grouped_moe`."""
  out = dict(state)
  for layer in range(config.num_hidden_layers):
    base = f"model.layers.{layer}.mlp"
    if f"{base}.grouped.W_gate" not in state:
      continue
    for ours, theirs in (("W_gate", "gate_proj"), ("W_up", "up_proj"), ("W_down", "down_proj")):
      stacked = out.pop(f"{base}.grouped.{ours}")
      for i in range(stacked.shape[0]):
        out[f"{base}.experts.{i}.{theirs}.weight"] = stacked[i].t().contiguous()
  return out
