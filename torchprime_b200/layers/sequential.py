"""A stack of identical layers that forwards keyword arguments unchanged to every layer.

Same contract as the reference's layers/sequential.py:8-41 (``HomogeneousSequential``): every
child has the same type; ``forward(*inputs, **broadcast)`` feeds the outputs of layer i to layer
i + 1 positionally and hands ``broadcast`` (rotary tables, position ids, masks) to all of them.
The reference compiles the body once with ``scan``; here the loop is a Python loop in training and
can be replayed from one CUDA graph in inference (``utils/cuda_graphs.GraphedForward``).
"""

from __future__ import annotations

import torch.nn as nn


class HomogeneousSequential(nn.Sequential):
  def __init__(self, *layers: nn.Module):
    kinds = {type(m) for m in layers}
    assert len(kinds) <= 1, f"all layers must have the same type, got {sorted(k.__name__ for k in kinds)}"
    super().__init__(*layers)

  def forward(self, *inputs, **broadcast):
    for layer in self:
      out = layer(*inputs, **broadcast)
      inputs = out if isinstance(out, tuple) else (out,)
    return inputs if len(inputs) > 1 else inputs[0]
