"""TransAct: transformer over a user's recent actions for recommendation ranking (the
forward-only benchmark model of the reference, torchprime/models/transact/).  Inputs: action type
sequence, item-embedding sequence, action times, request time, candidate item embedding; output:
max-pooled projection concatenated with the latest ``latest_n_emb`` encoder outputs."""

from __future__ import annotations

import random
from dataclasses import dataclass, field

import torch
import torch.nn as nn


@dataclass
class TransActConfig:
  seq_len: int = 100
  time_window_ms: int = 1000 * 60 * 60
  latest_n_emb: int = 10
  concat_candidate_emb: bool = True
  concat_max_pool: bool = True
  action_vocab: list = field(default_factory=lambda: list(range(20)))
  action_emb_dim: int = 32
  item_emb_dim: int = 32
  num_layer: int = 2
  nhead: int = 2
  dim_feedforward: int = 32


class TransAct(nn.Module):
  def __init__(self, cfg: TransActConfig):
    super().__init__()
    self.cfg = cfg
    self.seq_len, self.latest_n_emb, self.item_emb_dim = cfg.seq_len, cfg.latest_n_emb, cfg.item_emb_dim
    vocab = sorted(cfg.action_vocab)
    lookup = torch.zeros(100, dtype=torch.long)
    for i, a in enumerate(vocab):
      lookup[a + 1] = i
    self.register_buffer("action_type_lookup", lookup)
    self.action_emb = nn.Embedding(len(vocab), cfg.action_emb_dim, padding_idx=0)
    d_model = cfg.action_emb_dim + cfg.item_emb_dim * (2 if cfg.concat_candidate_emb else 1)
    layer = nn.TransformerEncoderLayer(d_model=d_model, nhead=cfg.nhead, dim_feedforward=cfg.dim_feedforward,
                                       batch_first=True)
    self.encoder = nn.TransformerEncoder(layer, num_layers=cfg.num_layer)
    if cfg.concat_max_pool:
      self.out_linear = nn.Linear(d_model, d_model)

  def _mask(self, pad, recent):
    m = pad | recent
    m[:, 0] = False   # never mask every position
    return torch.zeros_like(m, dtype=torch.float).masked_fill_(m, float("-inf"))

  def forward(self, action_type_seq, item_embedding_seq, action_time_seq, request_time, item_embedding):
    n = self.seq_len
    a = self.action_type_lookup[action_type_seq[:, :n] + 1]
    items, times = item_embedding_seq[:, :n], action_time_seq[:, :n]
    emb = self.action_emb(a)
    delta = request_time.unsqueeze(-1).expand(-1, n) - times
    window = random.randint(0, self.cfg.time_window_ms) if self.training else 0
    mask = self._mask(a <= 0, delta < window)
    x = torch.cat((emb, items), dim=2)
    if self.cfg.concat_candidate_emb:
      x = torch.cat((x, item_embedding.unsqueeze(1).expand(-1, n, -1)), dim=-1)
    y = self.encoder(src=x, src_key_padding_mask=mask)
    outs = []
    if self.cfg.concat_max_pool:
      outs.append(self.out_linear(y.max(dim=1).values))
    if self.latest_n_emb > 0:
      y = y[:, : self.latest_n_emb]
    outs.append(y.flatten(1))
    return torch.cat(outs, dim=1)

  def get_sample_inputs(self, batch_size: int):
    n = 100
    return ((torch.randint(0, 20, (batch_size, n)), torch.rand(batch_size, n, self.item_emb_dim),
             torch.randint(0, 20, (batch_size, n)), torch.randint(500, 1000, (batch_size,)),
             torch.rand(batch_size, self.item_emb_dim)), {})


def get_model():
  return TransAct(TransActConfig())
