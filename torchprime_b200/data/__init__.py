"""Dataset builders, keyed by ``task.name`` like the reference's ``DATASET_BUILDERS``
(torchprime/data/__init__.py:1-17)."""

from .synthetic import SyntheticTokenDataset, make_synthetic_dataset


def _make_train_dataset(**kw):
  from .dataset import make_train_dataset
  return make_train_dataset(**kw)


def _make_sft_dataset(**kw):
  from .sft_dataset import make_sft_dataset
  return make_sft_dataset(**kw)


DATASET_BUILDERS = {"train": _make_train_dataset, "sft": _make_sft_dataset}

__all__ = ["DATASET_BUILDERS", "SyntheticTokenDataset", "make_synthetic_dataset"]
