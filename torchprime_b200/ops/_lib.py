"""ctypes binding to ``libtpb200.so`` (the hand-written sm_100a kernels).

The library is built in-tree by :mod:`torchprime_b200.build`.  On a machine with a
GPU a missing library is an error, never a silent fallback: :func:`lib` raises
and the operator layer propagates it.  Every call checks the return code and the
status block that bounded device-side waits report into.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libtpb200.so")
_lib = None

EPI_BF16, EPI_F32, EPI_F32_ACC, EPI_BF16_ACC, EPI_BF16_RES, EPI_SWIGLU = range(6)
EPI_RS_BF16, EPI_AR_BF16 = 6, 7     # reduce-scatter / all-reduce epilogues of the fused collective GEMMs

_STATUS_NAMES = {
  1: "consumer timed out waiting for a TMA stage",
  2: "producer timed out waiting for a free stage",
  3: "epilogue timed out waiting for an accumulator",
  4: "MMA timed out waiting for the epilogue",
  5: "timed out waiting for a flag written by a peer GPU",
  6: "softmax pipeline wait timed out",
  7: "bad argument detected on device",
}


class KernelError(RuntimeError):
  pass


def lib_path() -> str:
  return _LIB_PATH


def available() -> bool:
  return os.path.exists(_LIB_PATH)


def lib():
  global _lib
  if _lib is None:
    if not os.path.exists(_LIB_PATH):
      raise KernelError(
        f"{_LIB_PATH} is missing: run `python -m torchprime_b200.build` (nvcc, sm_100a) first"
      )
    _lib = ctypes.CDLL(_LIB_PATH)
    _declare(_lib)
  return _lib


def _declare(L):
  P, I, LL, F = c_void_p, c_int, c_longlong, c_float
  sigs = {
    "tpb_status": [P],
    "tpb_sm_count": [],
    "tpb_gemm_bf16": [P, P, P, I, I, I, LL, LL, LL, I, I, I, F, P, LL, P, LL, I, P],
    "tpb_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, P],
    "tpb_rmsnorm_bwd": [P, P, P, P, P, P, P, I, I, P],
    "tpb_rope": [P, LL, I, I, I, P, P, P, I, I, I, I, P],
    "tpb_rope_strided": [P, LL, I, I, I, I, P, P, P, I, I, I, I, P],
    "tpb_swiglu_fwd": [P, P, I, I, P],
    "tpb_swiglu_bwd": [P, P, P, I, I, P],
    "tpb_ce_fwd_bwd": [P, LL, P, P, P, I, I, P],
    "tpb_adamw": [P, P, P, P, P, LL, F, F, F, F, F, F, F, P, I, P],
    "tpb_sumsq": [P, LL, I, P, P],
    "tpb_clip_coef": [P, F, P, P, P],
    "tpb_embedding_fwd": [P, P, P, I, I, LL, LL, P],
    "tpb_embedding_bwd": [P, P, P, I, I, LL, LL, I, P],
    "tpb_cast_f32_to_bf16": [P, P, LL, F, I, P],
  }
  for name, args in sigs.items():
    fn = getattr(L, name, None)
    if fn is None:
      continue
    fn.argtypes = args
    fn.restype = c_int
  L.tpb_status_clear.argtypes = []
  L.tpb_status_clear.restype = None
  _declare_optional(L)


_OPTIONAL_SIGS: dict[str, list] = {}


def register_signature(name: str, args: list):
  """Later-loaded operator modules declare the C signatures they use."""
  _OPTIONAL_SIGS[name] = args
  if _lib is not None:
    _declare_optional(_lib)


def _declare_optional(L):
  for name, args in _OPTIONAL_SIGS.items():
    fn = getattr(L, name, None)
    if fn is not None:
      fn.argtypes = args
      fn.restype = c_int


def stream_ptr() -> int:
  return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None):
  return None if t is None else t.data_ptr()


_LAUNCHES = [0]


def launch_count() -> int:
  """Number of kernel launches issued through this binding so far."""
  return _LAUNCHES[0]


def check(rc: int, what: str):
  _LAUNCHES[0] += 1
  if rc != 0:
    if rc == -2:
      raise KernelError(f"{what}: arguments rejected (alignment / shape constraints)")
    if rc in (-3, -4, -5):
      raise KernelError(f"{what}: could not create a TMA tensor map (code {rc})")
    if rc >= 1000:
      raise KernelError(f"{what}: CUDA launch failed with cudaError {rc - 1000}")
    raise KernelError(f"{what}: failed with code {rc}")


def status() -> tuple[int, int, int, int]:
  out = (c_int * 4)()
  lib().tpb_status(out)
  return tuple(out)


def raise_on_device_timeout():
  """Host-side check of the status block; call after a synchronisation point."""
  code, where, block, thread = status()
  if code != 0:
    lib().tpb_status_clear()
    raise KernelError(
      f"device-side bounded wait gave up: {_STATUS_NAMES.get(code, code)} "
      f"(site {where}, block {block}, thread {thread})"
    )
