"""Replay a forward pass from a CUDA graph.

A forward over many small kernels (short sequences, small batches, the 30-odd launches of every
decoder layer) is bound by launch overhead, not by the GPU.  ``GraphedForward`` captures one call
of a module (or any callable of tensors) into a CUDA graph with static input and output buffers
and replays it: one launch per call whatever the number of layers.  This is what stands in for the
reference's compile-once layer loop (``scan_layers``, torch_xla scan) where it matters, i.e. in
inference and evaluation; training steps are GPU-bound and run the layers as a Python loop.

Requirements: CUDA, no gradient recording, shapes fixed after the first call, and a callable that
neither synchronises with the host nor allocates outside PyTorch's allocator (the framework's
kernels are launched on the current stream and fulfil this).
"""

from __future__ import annotations

import torch
from torch.utils import _pytree as pytree


class GraphedForward:
  def __init__(self, fn, warmup: int = 3):
    self.fn = fn
    self.warmup = warmup
    self._graph = None
    self._static_in = None
    self._static_out = None
    self._spec = None

  def _signature(self, flat):
    return tuple((tuple(t.shape), t.dtype, t.device) if isinstance(t, torch.Tensor) else t for t in flat)

  def _capture(self, args, kwargs):
    flat, spec = pytree.tree_flatten((args, kwargs))
    self._static_in = [t.clone() if isinstance(t, torch.Tensor) else t for t in flat]
    sargs, skwargs = pytree.tree_unflatten(self._static_in, spec)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.no_grad():
      for _ in range(self.warmup):
        self.fn(*sargs, **skwargs)
    torch.cuda.current_stream().wait_stream(side)
    self._graph = torch.cuda.CUDAGraph()
    with torch.no_grad(), torch.cuda.graph(self._graph):
      self._static_out = self.fn(*sargs, **skwargs)
    self._spec = self._signature(flat)

  def __call__(self, *args, **kwargs):
    flat, _ = pytree.tree_flatten((args, kwargs))
    if self._graph is None:
      self._capture(args, kwargs)
    elif self._signature(flat) != self._spec:
      raise ValueError("GraphedForward was captured for other shapes/dtypes; create a new one")
    for dst, src in zip(self._static_in, flat):
      if isinstance(dst, torch.Tensor) and dst.data_ptr() != src.data_ptr():
        dst.copy_(src)
    self._graph.replay()
    return self._static_out
