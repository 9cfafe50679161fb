"""Llama 3 / 3.1 decoder-only transformer.

Module and parameter names follow the HuggingFace checkpoint layout
(``model.layers.N.self_attn.q_proj.weight`` ...), like the reference's
torchprime/torch_xla_models/model/llama/model.py:125-398, so exported and
pretrained safetensors load without renaming.  The computation is organised for
the B200 kernels instead of for a tracing compiler:

* activations stay token-major ``[B, S, H*D]``; q/k/v come out of one GEMM over the
  row-adjacent q/k/v weights and RoPE rotates the q and k heads of that buffer in
  place;
* residual adds ride in the epilogue of the o_proj / down_proj GEMMs, SiLU*mul in
  the epilogue of the fused gate/up GEMM;
* the head (final norm + lm_head + loss) runs as a chunked GEMM + cross-entropy that
  never materialises fp32 logits when only the loss is needed.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import functional as ops
from ..ops import reference as ref
from ..parallel.collectives import copy_to_tp, reduce_from_tp
from ..utils.profiling import trace_scope
from . import rope
from .base import BaseCausalLM


class LlamaRMSNorm(nn.Module):
  def __init__(self, hidden_size: int, eps: float = 1e-6):
    super().__init__()
    self.weight = nn.Parameter(torch.ones(hidden_size))
    self.variance_epsilon = eps

  def forward(self, x):
    return ops.rms_norm(x, self.weight, self.variance_epsilon)

  def with_residual(self, x):
    """(norm(x), x) where the returned ``x`` is the one to feed the residual connection with."""
    return ops.rms_norm_residual(x, self.weight, self.variance_epsilon)


class LlamaMLP(nn.Module):
  def __init__(self, config):
    super().__init__()
    self.hidden_size = config.hidden_size
    self.intermediate_size = config.intermediate_size
    self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
    self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
    self.down_proj = nn.Linear(self.intermediate_size, self.hidden_size, bias=False)
    assert config.get("hidden_act", "silu") == "silu", "only SiLU-gated MLPs are implemented"
    self.tp_group = None   # set by the engine when the tensor axis is > 1 (gate/up column-, down row-parallel)
    self.tp_reducer = None  # ops.fused_collective.AllReduceGemm, set by the engine with fused collectives on

  def forward(self, x, residual=None):
    with trace_scope("LlamaMLP"):
      if self.tp_group is not None:
        r = _fused_reducer(self, x, self.down_proj.weight.shape[0], self.down_proj.weight.shape[1],
                           2 * self.gate_proj.weight.shape[0])
        if r is not None:      # both all-reduces of the block happen inside GEMM epilogues
          act = ops.linear_swiglu(x, self.gate_proj.weight, self.up_proj.weight, tp_reduce_grad=r)
          return ops.linear(act, self.down_proj.weight, residual=residual, tp_reduce=r)
        x = copy_to_tp(x, self.tp_group)
        act = ops.linear_swiglu(x, self.gate_proj.weight, self.up_proj.weight)
        y = reduce_from_tp(ops.linear(act, self.down_proj.weight), self.tp_group)
        return y if residual is None else y + residual
      act = ops.linear_swiglu(x, self.gate_proj.weight, self.up_proj.weight)
      return ops.linear(act, self.down_proj.weight, residual=residual)


def _fused_reducer(module, x, n_out: int, k_in: int, n_col: int):
  """The module's all-reduce-in-GEMM object if it can take this block: hidden size ``n_out`` out of
  a row-parallel weight with ``k_in`` local inputs, and the input gradient of a column-parallel
  weight with ``n_col`` local outputs.  The answer is the same on every rank of the tensor group."""
  r = getattr(module, "tp_reducer", None)
  if r is None or not x.is_cuda or x.dtype != torch.bfloat16 or not ops.use_kernels(x):
    return None
  rows = x.numel() // x.shape[-1]
  if r.usable(rows, n_out, k_in) and r.usable(rows, x.shape[-1], n_col):
    return r
  return None


class LlamaAttention(nn.Module):
  def __init__(self, config, layer_idx: int | None = None):
    super().__init__()
    self.config = config
    self.layer_idx = layer_idx
    self.hidden_size = config.hidden_size
    self.num_heads = config.num_attention_heads
    self.head_dim = config.get("head_dim", None) or self.hidden_size // self.num_heads
    self.num_key_value_heads = config.num_key_value_heads
    bias = bool(config.get("attention_bias", False))
    self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=bias)
    self.k_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=bias)
    self.v_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=bias)
    self.o_proj = nn.Linear(self.num_heads * self.head_dim, self.hidden_size, bias=bias)
    self.attention_kernel = config.get("attention_kernel", None)
    self.tp_group = None   # set by the engine: q/k/v column-parallel (heads split), o row-parallel
    self.tp_reducer = None  # ops.fused_collective.AllReduceGemm, set by the engine with fused collectives on

  def forward(self, x, rope_cos, rope_sin, residual=None, position_ids=None, segment_ids=None, cp=None):
    with trace_scope("LlamaAttention"):
      b, s, _ = x.shape
      d = self.head_dim
      # local head counts follow the (possibly tensor-parallel sliced) weights
      hq, hkv = self.q_proj.weight.shape[0] // d, self.k_proj.weight.shape[0] // d
      bias = None
      if self.q_proj.bias is not None:
        bias = torch.cat([self.q_proj.bias, self.k_proj.bias, self.v_proj.bias])
      r = None
      if self.tp_group is not None:
        if bias is None and self.o_proj.bias is None:
          r = _fused_reducer(self, x, self.o_proj.weight.shape[0], self.o_proj.weight.shape[1], (hq + 2 * hkv) * d)
        if r is None:
          x = copy_to_tp(x, self.tp_group)
      qkv = ops.linear(x, [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], bias=bias,
                       tp_reduce_grad=r)
      qkv = ops.rope_inplace(qkv, rope_cos, rope_sin, hq + hkv, d, s, pos=position_ids)
      if cp is None and x.is_cuda:
        # one autograd input, one gradient (see ops.attention_qkv)
        o = ops.attention_qkv(qkv, hq, hkv, d, causal=True, q_segment_ids=segment_ids)
      else:
        q = qkv[..., : hq * d].view(b, s, hq, d)
        k = qkv[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
        v = qkv[..., (hq + hkv) * d:].view(b, s, hkv, d)
        if cp is not None:
          o = cp.attention(q, k, v, segment_ids=segment_ids)
        elif self.attention_kernel is None:
          o = ref.attention(q, k, v, causal=True, q_segment_ids=segment_ids)
        else:
          o = ops.attention(q, k, v, causal=True, q_segment_ids=segment_ids)
      o = o.reshape(b, s, hq * d)
      if r is not None:
        return ops.linear(o, self.o_proj.weight, residual=residual, tp_reduce=r)
      if self.tp_group is not None:
        out = reduce_from_tp(ops.linear(o, self.o_proj.weight), self.tp_group)
        if self.o_proj.bias is not None:
          out = out + self.o_proj.bias
        return out if residual is None else out + residual
      if self.o_proj.bias is not None:
        out = ops.linear(o, self.o_proj.weight, bias=self.o_proj.bias)
        return out if residual is None else out + residual
      return ops.linear(o, self.o_proj.weight, residual=residual)


class LlamaDecoderLayer(nn.Module):
  def __init__(self, config, layer_idx: int):
    super().__init__()
    self.self_attn = LlamaAttention(config, layer_idx)
    self.mlp = LlamaMLP(config)
    self.input_layernorm = LlamaRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
    self.post_attention_layernorm = LlamaRMSNorm(config.hidden_size, eps=config.rms_norm_eps)

  @property
  def fsdp_inkernel_gather(self) -> bool:
    """Tells the FSDP engine that every matrix of this layer is read in the forward pass only through
    ``ops.linear`` / ``ops.linear_swiglu``, which can wait for a weight that is still being gathered
    inside the GEMM (not so when the tensor-parallel adaptors or biases take other paths)."""
    a, m = self.self_attn, self.mlp
    return a.tp_group is None and m.tp_group is None and a.q_proj.bias is None and a.o_proj.bias is None

  def forward(self, hidden_states, rope_cos, rope_sin, position_ids=None, segment_ids=None, cp=None):
    with trace_scope("LlamaDecoderLayer"):
      x, hidden_states = self.input_layernorm.with_residual(hidden_states)
      h = self.self_attn(x, rope_cos, rope_sin, residual=hidden_states, position_ids=position_ids,
                         segment_ids=segment_ids, cp=cp)
      x, h = self.post_attention_layernorm.with_residual(h)
      return self.mlp(x, residual=h)


class LlamaEmbedding(nn.Embedding):
  """``peer_lookup``: set by the FSDP engine while the table stays sharded over the fsdp ranks; rows
  are then read from the owners' shards instead of from a gathered copy of the whole table."""
  supports_peer_lookup = True
  peer_lookup = None

  def forward(self, ids):
    if self.peer_lookup is not None:
      return ops.embedding_peer(ids, self.weight, self.peer_lookup)
    return ops.embedding(ids, self.weight)


class CausalLMHead(nn.Module):
  """Final norm + lm_head + next-token loss, the last FSDP unit of every model."""

  def __init__(self, norm: nn.Module, lm_head: nn.Linear, vocab_size: int):
    super().__init__()
    self.norm = norm
    self.lm_head = lm_head
    self.vocab_size = vocab_size
    self.loss_group = None   # context-parallel group: the token count is taken over the whole sequence

  def _valid_count(self, targets):
    """Tokens that count towards the loss.  Under context parallelism the per-rank average of
    this value over the group is used, so that the mean of the ranks' losses is the global mean."""
    if self.loss_group is None:
      return None
    import torch.distributed as dist
    n = (targets >= 0).sum().float()
    dist.all_reduce(n, group=self.loss_group)
    return (n / dist.get_world_size(self.loss_group)).clamp(min=1)

  def forward(self, hidden, targets=None, want_logits=True):
    """targets are already shifted (position t holds token t+1, -100 = ignore)."""
    with trace_scope("CausalLMHead"):
      h = self.norm(hidden)
      n_valid = self._valid_count(targets) if targets is not None else None
      if targets is not None and not want_logits:
        return None, ops.linear_cross_entropy(h, self.lm_head.weight, targets, n_valid=n_valid)
      logits = ops.linear(h, self.lm_head.weight).float()
      loss = None
      if targets is not None:
        flat = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]), targets.reshape(-1),
                                                 ignore_index=ref.IGNORE_INDEX,
                                                 reduction="mean" if n_valid is None else "sum")
        loss = flat if n_valid is None else flat / n_valid
      return logits, loss


class LlamaModel(nn.Module):
  def __init__(self, config):
    super().__init__()
    self.vocab_size = config.vocab_size
    self.embed_tokens = LlamaEmbedding(config.vocab_size, config.hidden_size)
    self.layers = nn.ModuleList([LlamaDecoderLayer(config, i) for i in range(config.num_hidden_layers)])
    self.norm = LlamaRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
    head_dim = config.get("head_dim", None) or config.hidden_size // config.num_attention_heads
    scaling = config.get("rope_scaling", None)
    if scaling is not None:
      scaling = rope.RopeScaling(**{k: scaling[k] for k in ("factor", "low_freq_factor", "high_freq_factor",
                                                           "original_context_len") if k in scaling})
    self.register_buffer("inv_freq", rope.llama3_rope_frequencies(head_dim, config.rope_theta, scaling),
                         persistent=False)
    self._rope_cache = None

  def rope_tables(self, seq_len: int, device, position_ids=None):
    # with explicit positions (context parallel) the table must cover the un-split sequence
    need = seq_len if position_ids is None else max(seq_len, int(getattr(self, "max_rope_positions", 0)) or
                                                    int(position_ids.max().item()) + 1)
    c = self._rope_cache
    if c is None or c[0].shape[0] < need or c[0].device != device:
      n = max(need, 1)
      self._rope_cache = rope.rope_tables(self.inv_freq.float(), n, device)
    return self._rope_cache


class LlamaForCausalLM(BaseCausalLM):
  def __init__(self, config):
    super().__init__()
    self.config = config
    self.model = LlamaModel(config)
    self.vocab_size = config.vocab_size
    self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
    object.__setattr__(self, "_head", CausalLMHead(self.model.norm, self.lm_head, config.vocab_size))
    self.apply(self._init_weights)
    self.return_logits = True   # trainers switch this off to use the chunked loss path
    self.cp = None              # context-parallel attention adaptor, set by the engine

  def forward(self, input_ids, labels=None, attention_mask=None, position_ids=None, segment_ids=None,
              labels_are_shifted=False):
    with trace_scope("LlamaForCausalLM"):
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
