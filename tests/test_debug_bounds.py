"""The range-checked debug mode (TPB_DEBUG_BOUNDS=1): data-dependent indices are validated before launch."""

import pytest
import torch

from torchprime_b200.ops import _debug, kernels, moe


def test_mode_is_off_by_default(monkeypatch):
  monkeypatch.delenv("TPB_DEBUG_BOUNDS", raising=False)
  _debug.check_index("op", "idx", torch.tensor([5, 99]), 0, 4)      # no-op


def test_check_index_reports_count_and_first(monkeypatch):
  monkeypatch.setenv("TPB_DEBUG_BOUNDS", "1")
  _debug.check_index("op", "idx", torch.tensor([0, 3, -1]), 0, 4, also_allowed=-1)
  with pytest.raises(IndexError, match=r"op: 2 of 4 entries of `idx` are outside \[0, 4\); first at flat position 1: 7"):
    _debug.check_index("op", "idx", torch.tensor([0, 7, -1, -2]), 0, 4, also_allowed=-1)
  _debug.check_monotone("op", "start", torch.tensor([0, 2, 2, 5]), 0, 5)
  with pytest.raises(IndexError, match="not non-decreasing"):
    _debug.check_monotone("op", "start", torch.tensor([0, 3, 2]), 0, 5)


def test_wrappers_refuse_bad_indices_before_launch(monkeypatch):
  """The check precedes the library call, so it is visible without a GPU."""
  monkeypatch.setenv("TPB_DEBUG_BOUNDS", "1")
  x = torch.zeros(4, 8, dtype=torch.bfloat16)
  with pytest.raises(IndexError, match="moe_gather"):
    moe.gather_rows(x, torch.tensor([0, 4], dtype=torch.int32))
  with pytest.raises(IndexError, match="moe_combine"):
    moe.combine_rows(x, torch.tensor([[0, 9]], dtype=torch.int32))
  with pytest.raises(IndexError, match="ce_fwd_bwd"):
    kernels.ce_fwd_bwd_(torch.zeros(2, 16, dtype=torch.bfloat16), torch.tensor([3, 16]), torch.zeros(1))
  with pytest.raises(IndexError, match="rope"):
    kernels.rope_(torch.zeros(2, 8, dtype=torch.bfloat16), 0, 1, 8, torch.zeros(4, 4), torch.zeros(4, 4), 4,
                  pos=torch.tensor([0, 4], dtype=torch.int32))


def test_exchange_descriptors(monkeypatch):
  monkeypatch.setenv("TPB_DEBUG_BOUNDS", "1")
  # three blocks of 4, 0 and 6 rows: to rank 1 at row 0, skipped, to rank 0 at row 10
  good = torch.tensor([0, 4, 4, 10, 1, -1, 0, 0, 0, 10])
  _debug.check_exchange_descriptors("a2a", good, 3, 10, 2, 16)
  with pytest.raises(IndexError, match="`dst_rank`"):
    _debug.check_exchange_descriptors("a2a", torch.tensor([0, 4, 4, 10, 2, -1, 0, 0, 0, 10]), 3, 10, 2, 16)
  with pytest.raises(IndexError, match="block rows"):
    _debug.check_exchange_descriptors("a2a", good, 3, 10, 2, 15)       # the last block ends at row 16
  with pytest.raises(IndexError, match="not non-decreasing"):
    _debug.check_exchange_descriptors("a2a", torch.tensor([0, 5, 4, 10, 1, -1, 0, 0, 0, 10]), 3, 10, 2, 16)
  with pytest.raises(IndexError, match="`start`"):
    _debug.check_exchange_descriptors("a2a", good, 3, 9, 2, 16)        # only nine send rows
  with pytest.raises(IndexError, match="entries"):
    _debug.check_exchange_descriptors("a2a", good[:-1], 3, 10, 2, 16)
  monkeypatch.setenv("TPB_DEBUG_BOUNDS", "0")
  _debug.check_exchange_descriptors("a2a", good[:-1], 3, 10, 2, 16)    # off: nothing is looked at


@pytest.mark.gpu
def test_valid_indices_pass_and_bad_ones_leave_the_context_usable(cuda_lib, monkeypatch):
  monkeypatch.setenv("TPB_DEBUG_BOUNDS", "1")
  dev = torch.device("cuda")
  x = torch.randn(64, 256, device=dev, dtype=torch.bfloat16)
  src = torch.randint(0, 64, (128,), device=dev, dtype=torch.int32)
  out = moe.gather_rows(x, src)
  assert torch.equal(out, x[src.long()])
  src[5] = 64
  with pytest.raises(IndexError, match="first at flat position 5: 64"):
    moe.gather_rows(x, src)
  logits = torch.randn(8, 512, device=dev, dtype=torch.bfloat16)
  tgt = torch.randint(0, 512, (8,), device=dev)
  tgt[0] = -100
  kernels.ce_fwd_bwd_(logits, tgt, torch.zeros(1, device=dev))
  torch.cuda.synchronize()
