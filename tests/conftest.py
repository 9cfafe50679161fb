import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def cuda_lib():
  """The in-tree sm_100a library; GPU tests fail loudly if it is missing."""
  import torch
  assert torch.cuda.is_available(), "this test is marked gpu and needs a CUDA device"
  from torchprime_b200.ops import _lib
  return _lib.lib()


@pytest.fixture(autouse=True)
def _check_status_after_gpu_test(request):
  yield
  if request.node.get_closest_marker("gpu"):
    import torch
    if torch.cuda.is_available():
      from torchprime_b200.ops import _lib
      if _lib.available():
        torch.cuda.synchronize()
        _lib.raise_on_device_timeout()
