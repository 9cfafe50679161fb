"""Model-FLOPs accounting for one training step (forward + backward = 3x forward matmuls).

The definitions are the MaxText-derived ones the reference uses
(torchprime/metrics/train_flops.py:12-289) so MFU numbers are comparable: causal
attention counts half of the dense S^2 work, the embedding lookup is free, the lm_head
counts once, recomputation (remat) is not counted.  Implemented as one table-driven
function over a :class:`StepShape` instead of one dataclass per family.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class StepShape:
  batch: int                 # sequences per step (global)
  seq: int
  layers: int
  hidden: int
  q_heads: int
  kv_heads: int
  head_dim: int
  ffn: int
  vocab: int
  gated_acts: int = 2        # SwiGLU: two input projections
  grad_accum: int = 1
  # MoE
  experts: int = 1
  top_k: int = 1
  moe_ffn: int = 0
  shared_experts: int = 0
  dense_layers: int | None = None     # DeepSeek: first k layers are dense
  moe_every: int = 1                  # Llama-4: every n-th layer is MoE
  # MLA
  mla: dict = field(default_factory=dict)
  # Llama-4 chunked attention
  chunk: int | None = None
  global_every: int = 1


def _ffn(s: StepShape, width: int) -> float:
  tok = s.batch * s.seq
  return 2.0 * tok * width * s.hidden * s.gated_acts + 2.0 * tok * width * s.hidden


def _moe_split(s: StepShape) -> tuple[int, int]:
  if s.dense_layers is not None:
    return s.dense_layers, s.layers - s.dense_layers
  n_moe = s.layers // s.moe_every
  return s.layers - n_moe, n_moe


def _all_ffn(s: StepShape) -> float:
  """FFN FLOPs summed over all layers."""
  if s.experts <= 1:
    return _ffn(s, s.ffn) * s.layers
  n_dense, n_moe = _moe_split(s)
  router = 2.0 * s.batch * s.seq * s.hidden * s.experts
  per_moe = router + _ffn(s, s.moe_ffn) * (s.shared_experts + s.top_k)
  return _ffn(s, s.ffn) * n_dense + per_moe * n_moe


def _projections(s: StepShape) -> tuple[float, float, float]:
  """(qkv, dense S^2 attention, output projection) FLOPs of one layer."""
  tok = s.batch * s.seq
  if s.mla:
    m = s.mla
    qk = m["qk_nope_head_dim"] + m["qk_rope_head_dim"]
    if not m.get("q_lora_rank"):
      q = 2.0 * tok * s.hidden * s.q_heads * qk
    else:
      q = 2.0 * tok * (s.hidden * m["q_lora_rank"] + m["q_lora_rank"] * s.q_heads * qk)
    kv = 2.0 * tok * (s.hidden * (m["kv_lora_rank"] + m["qk_rope_head_dim"])
                      + m["kv_lora_rank"] * s.q_heads * (m["qk_nope_head_dim"] + m["v_head_dim"]))
    attn = 2.0 * tok * s.seq * s.q_heads * (qk + m["v_head_dim"])
    proj = 2.0 * tok * s.hidden * s.q_heads * m["v_head_dim"]
    return q + kv, attn, proj
  qkv = 2.0 * tok * s.hidden * (s.q_heads + 2 * s.kv_heads) * s.head_dim
  attn = 4.0 * s.batch * s.seq ** 2 * s.q_heads * s.head_dim
  proj = 2.0 * tok * s.hidden * s.q_heads * s.head_dim
  return qkv, attn, proj


def _attention_all_layers(s: StepShape, dense_attn: float) -> float:
  """Causal attention FLOPs over all layers (handles Llama-4's chunked layers)."""
  if s.chunk is None:
    return dense_attn / 2.0 * s.layers
  n_global = s.layers // s.global_every
  n_chunked = s.layers - n_global
  full, rem = divmod(s.seq, s.chunk)
  chunked = 4.0 * s.batch * (full * s.chunk ** 2 + rem ** 2) * s.q_heads * s.head_dim
  return (n_global * dense_attn + n_chunked * chunked) / 2.0


def train_step_tflops(s: StepShape) -> tuple[float, float, float]:
  """(total, learnable-weight, attention) TFLOPs of one optimizer step."""
  qkv, dense_attn, proj = _projections(s)
  lm_head = 2.0 * s.batch * s.seq * s.hidden * s.vocab
  weights = (_all_ffn(s) + (qkv + proj) * s.layers + lm_head) * 3.0 / 1e12
  attn = _attention_all_layers(s, dense_attn) * 3.0 / 1e12
  weights *= s.grad_accum
  attn *= s.grad_accum
  return weights + attn, weights, attn


def shape_from_model_config(cfg: dict, batch_size: int, seq_len: int, grad_accum: int = 1) -> StepShape:
  """Pick the formula family the way the reference does (mfu.py:70-133): "deepseek" in the
  model id -> MLA + MoE; "llama-4" or more than one local expert -> MoE/chunked; else dense."""
  model_id = str(cfg.get("model_id", ""))
  hidden = int(cfg["hidden_size"])
  heads = int(cfg["num_attention_heads"])
  s = StepShape(batch=batch_size, seq=seq_len, layers=int(cfg["num_hidden_layers"]), hidden=hidden,
                q_heads=heads, kv_heads=int(cfg["num_key_value_heads"]), head_dim=hidden // heads,
                ffn=int(cfg["intermediate_size"]), vocab=int(cfg["vocab_size"]), grad_accum=grad_accum)
  if "deepseek" in model_id:
    s.experts = int(cfg["n_routed_experts"])
    s.top_k = int(cfg["num_experts_per_tok"])
    s.moe_ffn = int(cfg["moe_intermediate_size"])
    s.shared_experts = int(cfg["n_shared_experts"])
    s.dense_layers = int(cfg["first_k_dense_replace"])
    s.mla = {k: int(cfg.get(k) or 0) for k in ("qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim", "q_lora_rank",
                                               "kv_lora_rank")}
  elif "llama-4" in model_id or int(cfg.get("num_local_experts", 1)) > 1:
    s.experts = int(cfg.get("num_local_experts", 1))
    s.top_k = int(cfg.get("num_experts_per_tok", 1))
    s.moe_ffn = int(cfg.get("moe_intermediate_size", cfg["intermediate_size"]))
    s.shared_experts = int(cfg.get("n_shared_experts", cfg.get("shared_experts", 0)))
    s.moe_every = int(cfg.get("interleave_moe_layer_step", 1))
    s.chunk = int(cfg.get("chunk_attn_window_size", seq_len))
    s.global_every = int(cfg.get("nope_layer_interval", 1))
  return s
