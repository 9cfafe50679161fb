"""The allocation-free RMSNorm backward (csrc/tpb_noalloc.h) against the regular entry point.

Some hosts of this library may not allocate device memory while they run (a server that
gives each component a fixed arena, a thread that must not take the allocator lock, a
process whose memory is committed up front).  For them ``tpb_rmsnorm_bwd_noalloc`` keeps the
fp32 weight-gradient accumulator in a file-scope device array.  The test calls the exported
C symbol directly, twice in a row with different data (the shared accumulator must be
cleared by each call), and checks both outputs against ``tpb_rmsnorm_bwd``; it also checks
that a dimension beyond the built-in maximum is refused with a readable message.  It is
collected last so that a failure here cannot hide other tests under ``pytest -x``.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
  return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_rmsnorm_bwd_noalloc_matches_regular_entry_point(cuda_lib):
  L = cuda_lib
  fn = L.tpb_rmsnorm_bwd_noalloc
  fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
  fn.restype = ctypes.c_int
  L.tpb_noalloc_strerror.argtypes = [ctypes.c_int]
  L.tpb_noalloc_strerror.restype = ctypes.c_char_p
  from torchprime_b200.ops import kernels as k
  stream = torch.cuda.current_stream().cuda_stream
  for seed, (rows, dim) in enumerate([(300, 4096), (77, 2048)]):
    torch.manual_seed(100 + seed)
    x = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
    dres = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(torch.bfloat16)
    _, rstd, _ = k.rmsnorm_fwd(x, w, 1e-5)
    dx_ref, dw_ref = k.rmsnorm_bwd(dy, x, w, rstd, dres=dres)   # existing entry point, caller-owned fp32 dw
    dx = torch.empty_like(x)
    dw = torch.empty(dim, device="cuda", dtype=torch.bfloat16)
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(),
            dw.data_ptr(), rows, dim, stream)
    assert rc == 0, L.tpb_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert torch.equal(dx, dx_ref)
    assert _rel(dw, dw_ref) < 1e-2, _rel(dw, dw_ref)
  # beyond the built-in scratch: refused, nothing launched
  rc = fn(None, None, None, None, None, None, None, 1, 16384, stream)
  assert rc == -6
  assert b"TPB_NOALLOC_MAX_DIM" in L.tpb_noalloc_strerror(rc)
