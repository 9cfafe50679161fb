"""Training entry point.

  python -m torchprime_b200.train model=llama-3-8b dataset=synthetic ici_mesh.fsdp=8 task.max_steps=20
  torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m torchprime_b200.train ici_mesh.fsdp=8 ...
  python -m torchprime_b200.train --config-name llama-3-8b-sft-w-gsm8k

Same flow as the reference's hydra main (torchprime/torch_xla_models/train.py:29-106):
validate config -> start the metrics clock -> seed -> tokenizer (only when the dataset
needs one) -> build the model in bf16 -> parameter report -> dataset -> trainer by
``task.name`` -> train_loop -> finalize_training.  One process drives one GPU; launch N
processes (torchrun or ``python -m torchprime_b200.dist.launcher``) for N GPUs.
"""

from __future__ import annotations

import logging
import random
import sys

import numpy as np
import torch

from .config import compose, parse_cli
from .data import DATASET_BUILDERS, make_synthetic_dataset
from .dist import runtime as rt
from .metrics.metrics import MetricsLogger
from .models.model_utils import initialize_model_class, log_parameter_breakdown
from .trainer import TRAINERS
from .utils.config_utils import config_validator
from .utils.retry import retry

logger = logging.getLogger(__name__)
_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def set_seed(seed: int):
  random.seed(seed)
  np.random.seed(seed % (2 ** 32))
  torch.manual_seed(seed)
  if torch.cuda.is_available():
    torch.cuda.manual_seed_all(seed)


def build_dataset(config, tokenizer_fn):
  ds_cfg = config.dataset
  if ds_cfg.get("synthetic", False) or (ds_cfg.get("hf_dataset_name", None) is None
                                         and ds_cfg.get("file_dataset_path", None) is None):
    return make_synthetic_dataset(vocab_size=config.model.vocab_size, block_size=ds_cfg.block_size,
                                  num_samples=int(ds_cfg.get("num_samples", 4096)), seed=int(config.seed))
  builder = DATASET_BUILDERS[config.task.name]
  kwargs = {k: v for k, v in ds_cfg.items() if k not in ("synthetic", "num_samples")}
  return retry(lambda: builder(**kwargs, tokenizer=tokenizer_fn()))


def main(config):
  config_validator(config)
  metrics_logger = MetricsLogger()
  device = rt.init()
  logging.basicConfig(
    level=logging.INFO if rt.is_main() else logging.WARNING,
    format="%(asctime)s %(levelname)s %(name)s: %(message)s", force=True)
  set_seed(int(config.seed))
  assert config.torch_dtype in _DTYPES, f"Unsupported torch_dtype {config.torch_dtype}"
  assert config.torch_dtype == "bfloat16" or device.type == "cpu", "Currently only bfloat16 is supported on GPU"

  def tokenizer_fn():
    from transformers import AutoTokenizer
    from .checkpoint.safetensors_io import local_path_from_gcs
    name = config.model.tokenizer_name
    with local_path_from_gcs(name) as local:
      return retry(lambda: AutoTokenizer.from_pretrained(local))

  # skeleton on the meta device: each rank only ever allocates its own shard
  model = initialize_model_class(config.model, device="meta")
  log_parameter_breakdown(model, logger)
  data = build_dataset(config, tokenizer_fn)
  trainer_cls = TRAINERS[config.task.name]
  if device.type == "cpu" and "engine" in config and config.engine.get("cpu_dtype", None) is None:
    config.engine.cpu_dtype = "float32"
  trainer = trainer_cls(model=model, config=config, train_dataset=data)
  trainer.train_loop()
  trainer.finalize_training(metrics_logger)
  rt.shutdown()
  return 0


def cli(argv=None):
  argv = list(sys.argv[1:] if argv is None else argv)
  config_name, overrides = parse_cli(argv)
  config = compose(config_name or "default", overrides)
  return main(config)


if __name__ == "__main__":
  sys.exit(cli())
