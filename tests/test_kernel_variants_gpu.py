"""Kernel variants that a process selects once, from the environment, checked against the same fp32
oracles as the defaults: the CTA-pair (``cta_group::2``) GEMM forced for every dense shape, and the
two-tile, 128-key-step attention forward.  Each runs the numerics tests of the default kernels in a
child process with the switch set."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_tests(env_extra, target, keyword):
  env = dict(os.environ)
  env.update(env_extra)
  res = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", target), "-q", "-x", "-m", "gpu",
                        "-k", keyword, "-p", "no:cacheprovider"], env=env, cwd=ROOT, capture_output=True, text=True)
  assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
  assert " passed" in res.stdout


def test_cta_pair_gemm_for_every_dense_shape(cuda_lib):
  """TPB_GEMM_PAIR=2: layouts (all four operand orders, ragged shapes), epilogues and SwiGLU on 256 x 256
  pair tiles, also where the default heuristic would pick the single-CTA kernel."""
  _run_tests({"TPB_GEMM_PAIR": "2"}, "test_kernels_gpu.py", "gemm")


def test_single_cta_gemm_only(cuda_lib):
  _run_tests({"TPB_GEMM_PAIR": "0"}, "test_kernels_gpu.py", "gemm")


def test_two_tile_attention_forward(cuda_lib):
  """TPB_ATTN_FWD_V2=1: two 128-row query tiles per CTA, 128-key steps, softmax warpgroups with
  re-allocated registers; forward cases (masks, GQA, segments, positions) and the autograd path."""
  _run_tests({"TPB_ATTN_FWD_V2": "1"}, "test_attention_gpu.py", "forward or autograd")
