"""Batch / interactive text generation with the cached DeepSeek-V3 engine.

  python -m torchprime_b200.experimental.deepseek_inference.generate --ckpt-path <export dir> \
      --model deepseek-v2-lite [--input-file prompts.txt | --interactive] [--max-new-tokens 100] \
      [--temperature 1.0] [--attn-impl absorb]

Capability reference: torchprime/experimental/torchax_models/deepseek_v3/generate.py:11-234
(``sample`` = Gumbel-max over temperature-scaled logits, ``generate`` = prompt-aware incremental
decode that stops at EOS, a CLI with an interactive loop and a prompts file).
"""

from __future__ import annotations

import argparse

import torch

from .engine import DeepseekInferenceEngine


def sample(logits: torch.Tensor, temperature: float = 1.0, generator=None) -> torch.Tensor:
  """Draw one token per row: argmax(p / Exp(1)) is a sample from p (the exponential race)."""
  probs = torch.softmax(logits.float() / max(temperature, 1e-5), dim=-1)
  noise = torch.empty_like(probs).exponential_(1, generator=generator)
  return (probs / noise).argmax(dim=-1)


@torch.no_grad()
def generate(engine: DeepseekInferenceEngine, prompt_tokens: list[list[int]], max_new_tokens: int, eos_id: int,
             temperature: float = 1.0, generator=None) -> list[list[int]]:
  """Complete every prompt by up to ``max_new_tokens`` tokens.  Prompts of different lengths
  share the batch: positions still inside a prompt keep the prompt's token."""
  lens = [len(t) for t in prompt_tokens]
  assert prompt_tokens and min(lens) > 0 and max(lens) <= engine.max_seq_len
  total = min(engine.max_seq_len, max_new_tokens + max(lens))
  dev = engine.device
  tokens = torch.full((len(prompt_tokens), total), -1, dtype=torch.long, device=dev)
  for i, t in enumerate(prompt_tokens):
    tokens[i, : len(t)] = torch.tensor(t, dtype=torch.long, device=dev)
  prompt_mask = tokens != -1
  finished = torch.zeros(len(prompt_tokens), dtype=torch.bool, device=dev)
  prev = 0
  for cur in range(min(lens), total):
    logits = engine.forward(tokens[:, prev:cur].clamp_min(0), prev)
    nxt = sample(logits, temperature, generator) if temperature > 0 else logits.argmax(dim=-1)
    nxt = torch.where(prompt_mask[:, cur], tokens[:, cur], nxt)
    tokens[:, cur] = nxt
    finished |= (~prompt_mask[:, cur]) & (nxt == eos_id)
    prev = cur
    if bool(finished.all()):
      break
  out = []
  for i, row in enumerate(tokens.tolist()):
    row = [t for t in row[lens[i]: lens[i] + max_new_tokens] if t >= 0]
    if eos_id in row:
      row = row[: row.index(eos_id)]
    out.append(row)
  return out


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--ckpt-path", required=True, help="directory written by model.export() or convert.py")
  ap.add_argument("--model", default="deepseek-v2-lite", help="name of a configs/model/*.yaml")
  ap.add_argument("--tokenizer", default=None, help="defaults to the checkpoint directory")
  ap.add_argument("--input-file", default="")
  ap.add_argument("--interactive", action="store_true")
  ap.add_argument("--max-new-tokens", type=int, default=100)
  ap.add_argument("--max-seq-len", type=int, default=4096)
  ap.add_argument("--temperature", type=float, default=1.0)
  ap.add_argument("--attn-impl", choices=["naive", "absorb"], default="absorb")
  args = ap.parse_args(argv)
  from transformers import AutoTokenizer

  from ...config import compose
  from ...models.model_utils import initialize_model_class
  cfg = compose("default", [f"model={args.model}"]).model
  dev = "cuda" if torch.cuda.is_available() else "cpu"
  model = initialize_model_class(cfg, device=dev, dtype=torch.bfloat16)
  model.from_pretrained(args.ckpt_path)
  tok = AutoTokenizer.from_pretrained(args.tokenizer or args.ckpt_path)
  prompts = []
  if args.input_file:
    with open(args.input_file) as f:
      prompts = [line.strip() for line in f if line.strip()]
  engine = DeepseekInferenceEngine(model, max_batch_size=max(1, len(prompts)), max_seq_len=args.max_seq_len,
                                   attn_impl=args.attn_impl)

  def encode(text):
    if getattr(tok, "chat_template", None):
      return tok.apply_chat_template([{"role": "user", "content": text}], add_generation_prompt=True)
    return tok.encode(text)

  if prompts:
    outs = generate(engine, [encode(p) for p in prompts], args.max_new_tokens, tok.eos_token_id, args.temperature)
    for p, o in zip(prompts, outs):
      print("Prompt:", p)
      print("Completion:", tok.decode(o, skip_special_tokens=True))
      print()
  if args.interactive or not prompts:
    while True:
      try:
        text = input(">>> ")
      except EOFError:
        break
      if text in ("/exit", "/quit"):
        break
      out = generate(engine, [encode(text)], args.max_new_tokens, tok.eos_token_id, args.temperature)[0]
      print(tok.decode(out, skip_special_tokens=True))


if __name__ == "__main__":
  main()
