"""SFT / pre-training dataset construction with a toy word-level tokenizer (no network)."""

import json

import pytest

from torchprime_b200.data import sft_dataset as S
from torchprime_b200.data.dataset import group_texts, make_train_dataset


class ToyTokenizer:
  """Whitespace tokenizer with a growing vocabulary and a trivial chat template."""

  def __init__(self, eos=True, pad=None):
    self.vocab = {"<eos>": 0}
    self.eos_token_id = 0 if eos else None
    self.pad_token_id = pad

  def _id(self, w):
    return self.vocab.setdefault(w, len(self.vocab))

  def encode(self, text, add_special_tokens=False):
    return [self._id(w) for w in text.split()]

  def __call__(self, text):
    return {"input_ids": self.encode(text)}

  def convert_tokens_to_ids(self, tok):
    return self._id(tok)

  def apply_chat_template(self, messages, tokenize=False):
    return " ".join(f"<{m['role']}> {m['content']}" for m in messages)


def test_prompt_completion_masks_prompt_and_appends_eos():
  t = ToyTokenizer()
  out = S._tokenize_prompt_completion({"prompt": "a b", "completion": "c d e"}, t, compute_loss_on="completion",
                                      max_length=16, truncation="right")
  assert out["input_ids"][-1] == 0 and len(out["input_ids"]) == 6
  assert out["labels"][:2] == [-100, -100] and out["labels"][2:] == out["input_ids"][2:]
  full = S._tokenize_prompt_completion({"prompt": "a b", "completion": "c"}, t, compute_loss_on="all", max_length=16,
                                       truncation="right")
  assert full["labels"] == full["input_ids"]


def test_question_answer_template_and_text_alias():
  t = ToyTokenizer()
  qa = S._tokenize_prompt_completion({"question": "q1 q2", "answer": "a1"}, t, compute_loss_on="completion",
                                     max_length=32, truncation="right")
  words = {v: k for k, v in t.vocab.items()}
  assert [words[i] for i in qa["input_ids"]][:1] == ["Question:"] and "Answer:" in [words[i] for i in qa["input_ids"]]
  assert qa["labels"].count(-100) == 4
  txt = S._tokenize_prompt_completion({"text": "x y"}, t, compute_loss_on="completion", max_length=8, truncation="right")
  assert -100 not in txt["labels"]
  with pytest.raises(ValueError, match="Invalid input format"):
    S._tokenize_prompt_completion({"foo": 1}, t, compute_loss_on="all", max_length=8, truncation="right")


@pytest.mark.parametrize("trunc,want", [("right", [1, 2, 3]), ("left", [4, 5, 0]), ("drop", None)])
def test_truncation(trunc, want):
  t = ToyTokenizer()
  out = S._tokenize_prompt_completion({"text": "a b c d e"}, t, compute_loss_on="all", max_length=3, truncation=trunc)
  assert (out is None) if want is None else out["input_ids"] == want


@pytest.mark.parametrize("mode,expected_unmasked", [("all", 4), ("assistant", 2), ("last_assistant", 1), ("completion", 1)])
def test_chat_loss_masks(mode, expected_unmasked):
  t = ToyTokenizer(eos=False)
  msgs = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"},
          {"role": "user", "content": "more"}, {"role": "assistant", "content": "ok"}]
  out = S._tokenize_chat({"messages": msgs}, t, compute_loss_on=mode, max_length=64, truncation="right")
  per_msg = 2  # "<role> content"
  assert sum(1 for l in out["labels"] if l != -100) == expected_unmasked * per_msg


def test_padding_and_packing():
  t = ToyTokenizer()
  ex = {"input_ids": [[1, 2, 3], [4, 5], [6, 7, 8, 9]], "labels": [[1, 2, 3], [-100, 5], [6, 7, 8, 9]]}
  pad = S._pad_and_maybe_pack_samples(ex, t, 4, pack=False)
  assert pad["input_ids"][1] == [4, 5, 0, 0] and pad["labels"][1] == [-100, 5, -100, -100]
  assert pad["attention_mask"][0] == [1, 1, 1, 0]
  packed = S._pad_and_maybe_pack_samples(ex, t, 6, pack=True)
  assert packed["input_ids"] == [[1, 2, 3, 4, 5, 0], [6, 7, 8, 9, 0, 0]]
  assert packed["segment_ids"][0] == [1, 1, 1, 2, 2, 0]
  assert packed["attention_mask"][1] == [1, 1, 1, 1, 0, 0]
  exact = S._pad_and_maybe_pack_samples({"input_ids": [[1, 2], [3, 4]], "labels": [[1, 2], [3, 4]]}, t, 4, pack=True)
  assert exact["input_ids"] == [[1, 2, 3, 4]] and exact["attention_mask"] == [[1, 1, 1, 1]]


def test_make_datasets_from_jsonl(tmp_path):
  t = ToyTokenizer()
  p = tmp_path / "d.jsonl"
  p.write_text("\n".join(json.dumps({"prompt": f"p{i} q", "completion": f"c{i} d e"}) for i in range(5)))
  ds = S.make_sft_dataset(file_dataset_path=str(p), tokenizer=t, block_size=8, truncation="drop")
  assert len(ds) == 5 and set(ds[0]) == {"input_ids", "labels", "attention_mask"} and ds[0]["input_ids"].shape == (8,)
  packed = S.make_sft_dataset(file_dataset_path=str(p), tokenizer=t, block_size=12, pack_samples=True,
                              emit_segment_ids=True)
  assert len(packed) == 3 and "segment_ids" in packed[0]
  q = tmp_path / "t.jsonl"
  q.write_text("\n".join(json.dumps({"text": "a b c d e f g"}) for _ in range(4)))
  pre = make_train_dataset(file_dataset_path=str(q), tokenizer=t, block_size=5)
  assert len(pre) == 5 and pre[0]["labels"].tolist() == pre[0]["input_ids"].tolist()
  assert group_texts([[1, 2, 3], [4, 5]], 2) == [[1, 2], [3, 4]]
  with pytest.raises(ValueError, match="Either"):
    make_train_dataset(tokenizer=t, block_size=4)
