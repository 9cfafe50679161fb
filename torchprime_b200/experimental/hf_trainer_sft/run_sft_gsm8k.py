"""The same SFT recipe through the Hugging Face ``Trainer`` with PyTorch FSDP, for loss-curve comparison.

  python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 \
      torchprime_b200/experimental/hf_trainer_sft/run_sft_gsm8k.py --model /path/to/Meta-Llama-3-8B

Counterpart of the reference's experimental/torchrun_gpu_sft/run_sft_gsm8k.py:1-95: identical data
pipeline (``data/sft_dataset.py``: question/answer template, loss on the completion only, block
size 256, no packing), global batch 64, AdamW 4e-5 / 100 steps, so that the per-step losses can be
laid over those of ``python -m torchprime_b200.train task=sft ...`` (``draw_figure.py``).
Needs the model weights and the gsm8k dataset on local disk or network access.
"""

from __future__ import annotations

import argparse
import json
import os


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--model", required=True)
  ap.add_argument("--dataset", default="openai/gsm8k")
  ap.add_argument("--dataset-config", default="main")
  ap.add_argument("--block-size", type=int, default=256)
  ap.add_argument("--global-batch", type=int, default=64)
  ap.add_argument("--max-steps", type=int, default=100)
  ap.add_argument("--lr", type=float, default=4e-5)
  ap.add_argument("--out", default="outputs/hf_trainer_sft")
  a = ap.parse_args(argv)

  import torch
  from transformers import AutoModelForCausalLM, AutoTokenizer, Trainer, TrainerCallback, TrainingArguments

  from torchprime_b200.data.sft_dataset import make_sft_dataset

  world = int(os.environ.get("WORLD_SIZE", "1"))
  tok = AutoTokenizer.from_pretrained(a.model)
  if tok.pad_token is None:
    tok.pad_token = tok.eos_token
  data = make_sft_dataset(a.dataset, a.dataset_config, split="train", format="prompt_completion", pack_samples=False,
                          tokenizer=tok, block_size=a.block_size)
  model = AutoModelForCausalLM.from_pretrained(a.model, torch_dtype=torch.bfloat16)

  losses = []

  class Record(TrainerCallback):
    def on_log(self, args, state, control, logs=None, **kw):
      if logs and "loss" in logs:
        losses.append((state.global_step, float(logs["loss"])))

  args = TrainingArguments(
    output_dir=a.out, per_device_train_batch_size=max(1, a.global_batch // world), max_steps=a.max_steps,
    learning_rate=a.lr, lr_scheduler_type="linear", warmup_steps=0, weight_decay=0.0, bf16=True, logging_steps=1,
    save_strategy="no", report_to=[], fsdp="full_shard auto_wrap" if world > 1 else "",
    fsdp_config={"transformer_layer_cls_to_wrap": ["LlamaDecoderLayer"]} if world > 1 else None)
  Trainer(model=model, args=args, train_dataset=data, callbacks=[Record()]).train()
  if int(os.environ.get("RANK", "0")) == 0:
    os.makedirs(a.out, exist_ok=True)
    with open(os.path.join(a.out, "losses.json"), "w") as f:
      json.dump(losses, f)


if __name__ == "__main__":
  main()
