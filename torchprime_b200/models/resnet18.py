"""ResNet-18 classifier (CelebA identity study of the reference, torchprime/models/resnet18/
model.py).  Same interface: ``Resnet18ForClassification(num_classes, num_channels, seed)``,
``freeze_backbone`` / ``unfreeze_all`` and ``get_sample_inputs``.  ImageNet weights are used
when they can be loaded (no network here: falls back to random init and says so)."""

from __future__ import annotations

import hashlib
import io
import logging

import torch
import torch.nn as nn

logger = logging.getLogger(__name__)


def state_dict_hash(model: nn.Module) -> str:
  buf = io.BytesIO()
  torch.save(model.state_dict(), buf)
  return hashlib.sha256(buf.getvalue()).hexdigest()


class Resnet18ForClassification(nn.Module):
  def __init__(self, num_classes: int, num_channels: int = 3, seed: int = 42, pretrained: bool = True):
    super().__init__()
    import torchvision
    self.num_channels = num_channels
    torch.manual_seed(seed)
    weights = None
    if pretrained:
      try:
        weights = torchvision.models.ResNet18_Weights.IMAGENET1K_V1
        self.model = torchvision.models.resnet18(weights=weights)
      except Exception as e:  # noqa: BLE001 - offline
        logger.warning("ImageNet weights unavailable (%s); using random initialisation", type(e).__name__)
        weights = None
    if weights is None:
      self.model = torchvision.models.resnet18(weights=None)
    self.model.fc = nn.Linear(self.model.fc.in_features, num_classes)
    self.model.conv1 = nn.Conv2d(num_channels, 64, kernel_size=7, stride=2, padding=3, bias=False)
    self.model.bn1 = nn.BatchNorm2d(64)
    self.model_hash = state_dict_hash(self.model)
    logger.info("Initialized model with seed %d and hash %s", seed, self.model_hash)

  def forward(self, x):
    return self.model(x)

  def _trainable_head(self):
    return [self.model.fc, self.model.conv1, self.model.bn1]

  def freeze_backbone(self):
    for p in self.model.parameters():
      p.requires_grad = False
    for layer in self._trainable_head():
      for p in layer.parameters():
        p.requires_grad = True
    logger.info("Backbone of the model has been frozen.")

  def unfreeze_all(self):
    for p in self.model.parameters():
      p.requires_grad = True
    logger.info("Backbone of the model has been unfrozen.")

  def get_sample_inputs(self, batch_size: int):
    return (torch.rand(batch_size, self.num_channels, 224, 224, dtype=torch.float32),), {}


def get_model(num_classes: int = 1000, **kw):
  return Resnet18ForClassification(num_classes=num_classes, pretrained=False, **kw)
