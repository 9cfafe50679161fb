"""KV-cached inference for the DeepSeek-V3 family on top of the training model's weights.

Capability reference: torchprime/experimental/torchax_models/deepseek_v3/model.py:307-449 (MLA with
a ``naive`` cache of full keys/values or an ``absorb`` cache of the compressed latent) and
:718-773 (``Transformer.forward(tokens, start_pos)`` returning the logits of the last position).

The engine does not re-declare the network: it walks the layers of a
``DeepseekV3ForCausalLM`` and replaces only the attention core with a cached one, so a
checkpoint trained or converted for the training model serves as is.  Two cache layouts:

* ``naive``  - per layer K ``[B, S, H, dn+dr]`` and V ``[B, S, H, dv]``;
* ``absorb`` - per layer the normalised latent ``[B, S, kv_lora_rank]`` and the shared rotary
  key ``[B, S, dr]``.  The up-projection of keys is folded into the query and the
  up-projection of values is applied after the weighted sum, so a decode step reads
  ``kv_lora_rank + dr`` numbers per cached token instead of ``H * (dn + dr + dv)`` (576 against
  40960 for the 671B model) — on a bandwidth-bound decode that ratio is the speed-up.

Prefill at position 0 with the ``naive`` layout goes through the flash-attention kernel; decode
steps and the ``absorb`` layout use batched matrix products over the cache.
"""

from __future__ import annotations

import torch

from ...ops import functional as ops
from ...ops import reference as ref


class DeepseekInferenceEngine:
  def __init__(self, model, max_batch_size: int = 1, max_seq_len: int = 4096, attn_impl: str = "absorb",
               cache_dtype=None):
    assert attn_impl in ("naive", "absorb"), attn_impl
    self.model = model.eval()
    self.cfg = model.config
    self.attn_impl = attn_impl
    self.max_batch_size = max_batch_size
    self.max_seq_len = max_seq_len
    p = next(model.parameters())
    self.device, self.dtype = p.device, cache_dtype or p.dtype
    a0 = model.model.layers[0].self_attn
    h, dn, dr, dv, c = a0.num_heads, a0.qk_nope_head_dim, a0.qk_rope_head_dim, a0.v_head_dim, a0.kv_lora_rank
    n = len(model.model.layers)
    mk = lambda *shape: torch.zeros(*shape, device=self.device, dtype=self.dtype)  # noqa: E731
    if attn_impl == "naive":
      self.k_cache = [mk(max_batch_size, max_seq_len, h, dn + dr) for _ in range(n)]
      self.v_cache = [mk(max_batch_size, max_seq_len, h, dv) for _ in range(n)]
    else:
      self.kv_cache = [mk(max_batch_size, max_seq_len, c) for _ in range(n)]
      self.pe_cache = [mk(max_batch_size, max_seq_len, dr) for _ in range(n)]
    self.cos, self.sin = model.model.rope_tables(max_seq_len, self.device)

  def cache_bytes(self) -> int:
    bufs = (self.k_cache + self.v_cache) if self.attn_impl == "naive" else (self.kv_cache + self.pe_cache)
    return sum(t.numel() * t.element_size() for t in bufs)

  # -------------------------------------------------------------------------------------
  def _attention(self, li: int, attn, x, start: int, pos):
    b, s, _ = x.shape
    end = start + s
    h, dn, dr, dv, c = attn.num_heads, attn.qk_nope_head_dim, attn.qk_rope_head_dim, attn.v_head_dim, attn.kv_lora_rank
    if not attn.q_lora_rank:
      q = ops.linear(x, attn.q_proj.weight)
    else:
      q = ops.linear(attn.q_a_layernorm(ops.linear(x, attn.q_a_proj.weight, bias=attn.q_a_proj.bias)),
                     attn.q_b_proj.weight)
    q = ops.rope_slices(q, self.cos, self.sin, h, dr, s, col0=dn, head_stride=dn + dr, pos=pos,
                        interleaved=attn.rope_interleave)
    ckv = ops.linear(x, attn.kv_a_proj_with_mqa.weight, bias=attn.kv_a_proj_with_mqa.bias)
    ckv = ops.rope_slices(ckv, self.cos, self.sin, 1, dr, s, col0=c, head_stride=dr, pos=pos,
                          interleaved=attn.rope_interleave)
    latent = attn.kv_a_layernorm(ckv[..., :c].contiguous())
    k_rot = ckv[..., c:]
    q4 = q.view(b, s, h, dn + dr)
    causal = None
    if s > 1:
      t = torch.arange(end, device=x.device)
      causal = t[None, :] > (start + torch.arange(s, device=x.device))[:, None]          # [s, end]
    if self.attn_impl == "naive":
      kv = ops.linear(latent, attn.kv_b_proj.weight).view(b, s, h, dn + dv)
      k = torch.cat([kv[..., :dn], k_rot[:, :, None, :].expand(b, s, h, dr)], dim=-1)
      v = kv[..., dn:]
      self.k_cache[li][:b, start:end] = k
      self.v_cache[li][:b, start:end] = v
      if start == 0 and x.is_cuda and s >= 128:
        o = ops.attention(q4, k.contiguous(), v.contiguous(), causal=True, scale=attn.scaling)
      else:
        kc, vc = self.k_cache[li][:b, :end], self.v_cache[li][:b, :end]
        scores = torch.einsum("bshd,bthd->bsht", q4.float(), kc.float()) * attn.scaling
        if causal is not None:
          scores = scores.masked_fill(causal[None, :, None, :], float("-inf"))
        o = torch.einsum("bsht,bthd->bshd", scores.softmax(-1), vc.float()).to(x.dtype)
    else:
      w = attn.kv_b_proj.weight.view(h, dn + dv, c)
      self.kv_cache[li][:b, start:end] = latent
      self.pe_cache[li][:b, start:end] = k_rot
      q_abs = torch.einsum("bshd,hdc->bshc", q4[..., :dn].float(), w[:, :dn].float())
      lc, pc = self.kv_cache[li][:b, :end].float(), self.pe_cache[li][:b, :end].float()
      scores = (torch.einsum("bshc,btc->bsht", q_abs, lc)
                + torch.einsum("bshr,btr->bsht", q4[..., dn:].float(), pc)) * attn.scaling
      if causal is not None:
        scores = scores.masked_fill(causal[None, :, None, :], float("-inf"))
      o_lat = torch.einsum("bsht,btc->bshc", scores.softmax(-1), lc)
      o = torch.einsum("bshc,hdc->bshd", o_lat, w[:, dn:].float()).to(x.dtype)
    o = o.reshape(b, s, h * dv)
    return ops.linear(o, attn.o_proj.weight, bias=attn.o_proj.bias)

  @torch.no_grad()
  def forward(self, tokens: torch.Tensor, start_pos: int = 0) -> torch.Tensor:
    """tokens [B, S] at positions ``start_pos .. start_pos+S-1`` -> logits [B, vocab] of the last one."""
    b, s = tokens.shape
    assert b <= self.max_batch_size and start_pos + s <= self.max_seq_len, (b, start_pos, s)
    m = self.model.model
    h = m.embed_tokens(tokens.to(self.device))
    pos = (start_pos + torch.arange(s, device=self.device, dtype=torch.int32)).repeat(b).contiguous()
    for li, layer in enumerate(m.layers):
      a = self._attention(li, layer.self_attn, layer.input_layernorm(h), start_pos, pos)
      h = h + a
      h = layer.mlp(layer.post_attention_layernorm(h), residual=h)
    last = m.norm(h[:, -1:, :].contiguous())
    return torch.nn.functional.linear(last[:, 0].float(), self.model.lm_head.weight.float())

  __call__ = forward


def full_forward_last_logits(model, tokens: torch.Tensor) -> torch.Tensor:
  """Uncached oracle: the training model's own forward, last position (used by tests)."""
  with torch.no_grad():
    out = model(tokens)
  logits = out[0] if isinstance(out, (tuple, list)) else out
  return logits[:, -1].float()


__all__ = ["DeepseekInferenceEngine", "full_forward_last_logits", "ref"]
