"""Image-classification fine-tuning loop (ResNet-18; the reference's torch_xla_vision_models/train.py
trains CelebA identity classification on ``cuda`` or ``xla``).  AdamW, cosine schedule with linear
warm-up, frozen backbone for the first epochs, per-epoch CSV metrics.  Data: an image-folder style
dataset when a path is given, otherwise synthetic images so the loop runs anywhere."""

from __future__ import annotations

import argparse
import csv
import math
import os
import time

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, Dataset

from ..models.resnet18 import Resnet18ForClassification


class SyntheticImages(Dataset):
  def __init__(self, n: int, num_classes: int, channels: int = 3, size: int = 64, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    self.y = torch.randint(0, num_classes, (n,), generator=g)
    self.protos = torch.randn(num_classes, channels, size, size, generator=g)
    self.n, self.seed = n, seed

  def __len__(self):
    return self.n

  def __getitem__(self, i):
    g = torch.Generator().manual_seed(self.seed * 7919 + i)
    return self.protos[self.y[i]] + 0.5 * torch.randn(self.protos.shape[1:], generator=g), self.y[i]


def cosine_with_warmup(step: int, warmup: int, total: int) -> float:
  if step < warmup:
    return step / max(1, warmup)
  return 0.5 * (1 + math.cos(math.pi * (step - warmup) / max(1, total - warmup)))


def accuracy(model, loader, device) -> float:
  model.eval()
  hit = n = 0
  with torch.no_grad():
    for x, y in loader:
      pred = model(x.to(device)).argmax(-1).cpu()
      hit += (pred == y).sum().item()
      n += y.numel()
  return hit / max(1, n)


def train(num_classes=10, epochs=3, freeze_epochs=1, batch_size=32, lr=1e-3, weight_decay=1e-2, data_dir=None,
          out_csv=None, train_samples=256, device=None, seed=42):
  device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
  torch.manual_seed(seed)
  if data_dir:
    import torchvision
    tf = torchvision.transforms.Compose([torchvision.transforms.Resize((224, 224)), torchvision.transforms.ToTensor()])
    train_ds = torchvision.datasets.ImageFolder(os.path.join(data_dir, "train"), tf)
    val_ds = torchvision.datasets.ImageFolder(os.path.join(data_dir, "val"), tf)
    num_classes = len(train_ds.classes)
  else:
    train_ds = SyntheticImages(train_samples, num_classes, seed=seed)
    val_ds = SyntheticImages(max(32, train_samples // 4), num_classes, seed=seed)   # same prototypes
  model = Resnet18ForClassification(num_classes=num_classes, seed=seed, pretrained=bool(data_dir)).to(device)
  loader = DataLoader(train_ds, batch_size=batch_size, shuffle=True, drop_last=True)
  val_loader = DataLoader(val_ds, batch_size=batch_size)
  opt = torch.optim.AdamW([p for p in model.parameters()], lr=lr, weight_decay=weight_decay)
  total = epochs * len(loader)
  sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: cosine_with_warmup(s, max(1, total // 10), total))
  loss_fn = nn.CrossEntropyLoss()
  rows = []
  for epoch in range(epochs):
    model.freeze_backbone() if epoch < freeze_epochs else model.unfreeze_all()
    model.train()
    t0, run_loss = time.perf_counter(), 0.0
    for x, y in loader:
      opt.zero_grad(set_to_none=True)
      loss = loss_fn(model(x.to(device)), y.to(device))
      loss.backward()
      opt.step()
      sched.step()
      run_loss += loss.item()
    rows.append({"epoch": epoch, "train_loss": run_loss / len(loader), "val_accuracy": accuracy(model, val_loader, device),
                 "epoch_seconds": time.perf_counter() - t0, "device": str(device), "model_hash": model.model_hash})
    print(rows[-1])
  if out_csv:
    os.makedirs(os.path.dirname(os.path.abspath(out_csv)), exist_ok=True)
    with open(out_csv, "w", newline="") as f:
      w = csv.DictWriter(f, fieldnames=list(rows[0]))
      w.writeheader()
      w.writerows(rows)
  return rows


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--data-dir")
  ap.add_argument("--epochs", type=int, default=3)
  ap.add_argument("--batch-size", type=int, default=32)
  ap.add_argument("--lr", type=float, default=1e-3)
  ap.add_argument("--out-csv", default="outputs/vision_metrics.csv")
  a = ap.parse_args(argv)
  train(epochs=a.epochs, batch_size=a.batch_size, lr=a.lr, data_dir=a.data_dir, out_csv=a.out_csv)


if __name__ == "__main__":
  main()
