"""Supervised fine-tuning trainer: load pretrained weights before the engine shards them,
export the model after the loop.  Same hooks as the reference's ``SFTTrainer``
(torchprime/torch_xla_models/trainer/sft_trainer.py:20-61)."""

from __future__ import annotations

import logging
import time

from .base_trainer import Trainer

logger = logging.getLogger(__name__)


class SFTTrainer(Trainer):
  def __init__(self, model, config, train_dataset):
    pretrained = config.model.get("pretrained_model", None)
    state = None
    if pretrained:
      from ..checkpoint import safetensors_io
      logger.info("Loading pretrained weights from %s", pretrained)
      with safetensors_io.model_dir(pretrained) as model_dir:
        state = model.convert_loaded_state_dict(safetensors_io.load_safetensors_to_state_dict(model_dir))
    else:
      logger.warning("No pretrained checkpoint specified; training from scratch")
    super().__init__(model, config, train_dataset)
    if state is not None:
      self.engine.load_full_state_dict(state, strict=True)

  def train_loop(self) -> None:
    super().train_loop()
    t0 = time.perf_counter()
    self.model._maybe_save_checkpoint(self.config, engine=self.engine)
    logger.info("Finished saving model weights in %.2f s", time.perf_counter() - t0)
