"""Mixtral 8x7B-style sparse mixture-of-experts decoder.

Public behaviour follows the reference (torchprime/torch_xla_models/model/mixtral/
model.py:640-1018): HF-compatible names, ``moe_implementation`` in {``static``,
``gmm_stack``} (per-expert ``w1/w2/w3`` Linear modules, HF key layout) or {``gmm``,
``dropping``} (stacked ``experts.w1 [E,D,F]``, ``w2 [E,F,D]``, ``w3 [E,D,F]``); router =
softmax -> top-k -> renormalise; the decoder layer threads a cumulative load-balance loss
through the stack; final loss = CE + ``router_aux_loss_coef`` * mean-over-layers aux loss.

Differences by design: ``dropping`` does not build ``[B,S,E,C]`` dispatch masks — the
capacity limit (``int(S*k/E*capacity_factor)`` rows per expert and batch row) is applied
while sorting tokens into the expert-grouped layout and dropped pairs simply contribute
nothing; routed experts run as grouped tcgen05 GEMMs.  The reference detaches the aux loss
(``torch.tensor(loss)``, model.py:858); ``aux_loss_grad=true`` lets its gradient flow.
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
from .llama import CausalLMHead, LlamaAttention, LlamaEmbedding, LlamaRMSNorm


class MixtralRMSNorm(LlamaRMSNorm):
  pass


class MixtralAttention(LlamaAttention):
  pass


class MixtralBlockSparseTop2MLP(nn.Module):
  """One expert with HF parameter names (w1 = gate, w3 = up, w2 = down)."""

  def __init__(self, config):
    super().__init__()
    self.w1 = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
    self.w2 = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)
    self.w3 = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)

  def forward(self, x):
    return self.w2(F.silu(self.w1(x)) * self.w3(x))


class MixtralStackedExperts(nn.Module):
  """Stacked expert weights (``gmm`` / ``dropping``)."""

  def __init__(self, config):
    super().__init__()
    e, d, f = config.num_local_experts, config.hidden_size, config.intermediate_size
    self.w1 = nn.Parameter(torch.empty(e, d, f))
    self.w3 = nn.Parameter(torch.empty(e, d, f))
    self.w2 = nn.Parameter(torch.empty(e, f, d))
    for w in (self.w1, self.w2, self.w3):
      if not w.is_meta:
        nn.init.kaiming_uniform_(w, a=math.sqrt(5))


class MixtralMoeBlock(nn.Module):
  def __init__(self, config):
    super().__init__()
    self.hidden_dim = config.hidden_size
    self.ffn_dim = config.intermediate_size
    self.num_experts = config.num_local_experts
    self.top_k = config.num_experts_per_tok
    self.moe_implementation = config.get("moe_implementation", "gmm")
    self.capacity_factor = float(config.get("capacity_factor", 1.25))
    self.gate = nn.Linear(self.hidden_dim, self.num_experts, bias=False)
    if self.moe_implementation in ("gmm", "dropping"):
      self.experts = MixtralStackedExperts(config)
    elif self.moe_implementation in ("static", "gmm_stack"):
      self.experts = nn.ModuleList([MixtralBlockSparseTop2MLP(config) for _ in range(self.num_experts)])
    else:
      raise NotImplementedError(f"Unsupported moe implementation {self.moe_implementation}")
    self.ep = None   # expert-parallel adaptor, set by the engine
    self.tp_group = None   # set by the engine: experts split along the FFN dimension (w1/w3 columns, w2 rows)

  def load_balance_loss(self, top_k_indices, probs):
    """Switch-Transformer auxiliary loss: mean(fraction routed * mean probability) * E^2.
    top_k_indices [B,S,K], probs [B,S,E]."""
    mask = F.one_hot(top_k_indices.long(), num_classes=self.num_experts).sum(dim=2).float()
    density = mask.mean(dim=1)
    density_prob = probs.float().mean(dim=1)
    return torch.mean(density * density_prob) * (self.num_experts ** 2)

  def forward(self, hidden_states):
    with trace_scope("MixtralMoeBlock"):
      b, s, d = hidden_states.shape
      x = hidden_states.reshape(-1, d)
      router_logits = ops.linear(x, self.gate.weight)
      weights, idx, probs = moe_ops.router_topk(router_logits, self.top_k, mode="softmax")
      weights = weights.to(x.dtype)
      if self.tp_group is not None:
        # every rank of the tensor group computes the experts on its slice of the FFN dimension: the
        # outputs are partial sums (reduced below), and so are the gradients that flow back into the
        # tokens and into the routing weights (summed by the backward of copy_to_tp)
        x, weights = copy_to_tp(x, self.tp_group), copy_to_tp(weights, self.tp_group)
      loss = hidden_states.new_zeros((), dtype=torch.float32)
      impl = self.moe_implementation
      if impl == "static":
        out = torch.zeros_like(x)
        for e, expert in enumerate(self.experts):
          w_e = weights.masked_fill(idx != e, 0.0).sum(dim=-1, keepdim=True)
          out = out + (expert(x) * w_e).to(x.dtype)
      else:
        if impl == "gmm_stack":
          w1 = torch.stack([ex.w1.weight.t() for ex in self.experts])
          w2 = torch.stack([ex.w2.weight.t() for ex in self.experts])
          w3 = torch.stack([ex.w3.weight.t() for ex in self.experts])
        else:
          w1, w2, w3 = self.experts.w1, self.experts.w2, self.experts.w3
        capacity = None
        if impl == "dropping":
          capacity = int((s * self.top_k / self.num_experts) * self.capacity_factor)
          loss = self.load_balance_loss(idx.view(b, s, self.top_k), probs.view(b, s, self.num_experts))
        if self.ep is not None:
          out = self.ep.grouped_mlp(x, weights, idx, w1, w3, w2, capacity=capacity, rows_per_group=s)
        else:
          out = moe_ops.grouped_mlp(x, weights, idx, w1, w3, w2, capacity=capacity, rows_per_group=s)
      if self.tp_group is not None:
        out = reduce_from_tp(out, self.tp_group)
      return out.reshape(b, s, d), router_logits, loss


class MixtralDecoderLayer(nn.Module):
  def __init__(self, config, layer_idx: int):
    super().__init__()
    self.hidden_size = config.hidden_size
    self.self_attn = MixtralAttention(config, layer_idx)
    self.block_sparse_moe = MixtralMoeBlock(config)
    self.input_layernorm = MixtralRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
    self.post_attention_layernorm = MixtralRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
    self.aux_loss_grad = bool(config.get("aux_loss_grad", False))

  def forward(self, hidden_states, cumulative_loss, rope_cos, rope_sin, position_ids=None, segment_ids=None, cp=None):
    with trace_scope("MixtralDecoderLayer"):
      x = self.input_layernorm(hidden_states)
      h = self.self_attn(x, rope_cos, rope_sin, residual=hidden_states, position_ids=position_ids,
                         segment_ids=segment_ids, cp=cp)
      x = self.post_attention_layernorm(h)
      moe_out, _router_logits, loss = self.block_sparse_moe(x)
      if not self.aux_loss_grad:
        loss = loss.detach()
      return h + moe_out, cumulative_loss + loss


class MixtralModel(nn.Module):
  def __init__(self, config):
    super().__init__()
    self.config = config
    self.vocab_size = config.vocab_size
    self.embed_tokens = LlamaEmbedding(config.vocab_size, config.hidden_size)
    self.layers = nn.ModuleList([MixtralDecoderLayer(config, i) for i in range(config.num_hidden_layers)])
    self.norm = MixtralRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
    head_dim = config.get("head_dim", None) or config.hidden_size // config.num_attention_heads
    self.register_buffer("inv_freq", rope.default_rope_frequencies(head_dim, float(config.rope_theta)),
                         persistent=False)
    self._rope_cache = None

  def rope_tables(self, seq_len, device, position_ids=None):
    need = seq_len if position_ids is None else max(seq_len, int(getattr(self, "max_rope_positions", 0)) or
                                                    int(position_ids.max().item()) + 1)
    c = self._rope_cache
    if c is None or c[0].shape[0] < need or c[0].device != device:
      self._rope_cache = rope.rope_tables(self.inv_freq.float(), max(need, 1), device)
    return self._rope_cache


class MixtralForCausalLM(BaseCausalLM):
  def __init__(self, config):
    super().__init__()
    self.config = config
    self.model = MixtralModel(config)
    self.vocab_size = config.vocab_size
    self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
    self.router_aux_loss_coef = config.router_aux_loss_coef
    self.num_experts = config.num_local_experts
    self.num_experts_per_tok = config.num_experts_per_tok
    object.__setattr__(self, "_head", CausalLMHead(self.model.norm, self.lm_head, config.vocab_size))
    self.apply(self._init_weights)
    self.return_logits = True
    self.cp = None

  def param_init_kind(self, full_name, module, pname):
    if isinstance(module, MixtralStackedExperts):
      return "normal"
    return None

  def tp_layout(self, name: str):
    """Dimension along which a tensor-parallel weight is split (None: replicated).  Attention: q/k/v
    by heads (rows), o_proj by its input columns; stacked experts [E, D, F] / [E, F, D] along F."""
    if ".self_attn." in name and name.endswith("_proj.weight"):
      return 1 if ".o_proj." in name else 0
    if name.endswith(("experts.w1", "experts.w3")):
      return 2
    if name.endswith("experts.w2"):
      return 1
    return None

  def forward(self, input_ids, labels=None, attention_mask=None, position_ids=None, segment_ids=None,
              labels_are_shifted=False):
    with trace_scope("MixtralForCausalLM"):
      b, s = input_ids.shape
      h = self.model.embed_tokens(input_ids)
      cos, sin = self.model.rope_tables(s, h.device, position_ids)
      pos = position_ids.reshape(-1).to(torch.int32).contiguous() if position_ids is not None else None
      aux = torch.zeros((), dtype=torch.float32, device=h.device)
      for layer in self.model.layers:
        h, aux = layer(h, aux, cos, sin, pos, segment_ids, self.cp)
      aux = aux / len(self.model.layers)
      targets = None
      if labels is not None:
        targets = labels if labels_are_shifted else ref.shift_labels(labels)
      logits, loss = self._head(h, targets, want_logits=self.return_logits or labels is None)
      if loss is not None:
        loss = loss + self.router_aux_loss_coef * aux
      return logits, loss
