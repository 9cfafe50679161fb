"""Model families.  ``registry`` maps benchmark model names to factories that return a module
exposing ``get_sample_inputs(batch_size)`` (reference: torchprime/models/__init__.py)."""


def _transact():
  from . import transact
  return transact.get_model()


def _resnet18():
  from . import resnet18
  return resnet18.get_model()


registry = {"pinterest/transformer_user_action": _transact, "resnet18": _resnet18}
