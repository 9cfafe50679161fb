"""Failure detection without faulting a device: failures are made on the host (a rank that raises,
exits or stalls; a corrupted checkpoint) and, on the GPU, a bounded wait is simply allowed to run
out — the kernel returns a status code and the context stays usable."""

import ctypes
import os
import sys
import time

import pytest
import torch

from torchprime_b200.dist.watchdog import Heartbeat, StepDeadlineExceeded, StepWatchdog


def test_watchdog_trips_on_a_stalled_step():
  hits = []
  wd = StepWatchdog(deadline_s=0.2, poll_s=0.05, on_timeout=lambda s, t: hits.append(s))
  wd.begin_step(3)
  time.sleep(0.5)
  with pytest.raises(StepDeadlineExceeded, match="step 3"):
    wd.end_step(3)
  wd.stop()
  assert hits == [3]
  wd = StepWatchdog(deadline_s=5.0, poll_s=0.05)
  wd.begin_step(0)
  wd.end_step(0)
  wd.stop()
  assert wd.tripped() is None


class _Store:
  def __init__(self):
    self.d = {}
  def set(self, k, v):
    self.d[k] = v.encode()
  def get(self, k):
    return self.d[k]
  def check(self, keys):
    return all(k in self.d for k in keys)


def test_heartbeat_reports_silent_ranks():
  st = _Store()
  hbs = [Heartbeat(st, r, 3) for r in range(3)]
  hbs[0].beat(1)
  hbs[2].beat(1)
  assert hbs[0].stale_ranks(max_age_s=10) == [1]       # rank 1 never joined
  st.d["hb/2"] = f"1:{time.time() - 100}".encode()      # rank 2 went silent
  assert hbs[0].stale_ranks(max_age_s=10) == [1, 2]


def _rank_that_dies(rank, world, port, out):
  os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
  import datetime
  import torch.distributed as dist
  dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
  t = torch.ones(1)
  dist.all_reduce(t)                # step 0: everyone is here
  if rank == 1:
    os._exit(0)                     # leaves between steps, nothing in flight
  try:
    dist.all_reduce(t)              # step 1: the peer is gone -> short timeout ends the collective
    out[rank] = "no error"
  except Exception as e:  # noqa: BLE001
    out[rank] = f"detected: {type(e).__name__}"


def test_surviving_rank_detects_peer_exit_through_collective_timeout():
  import torch.multiprocessing as mp
  mgr = mp.Manager()
  out = mgr.dict()
  ctx = mp.get_context("spawn")
  procs = [ctx.Process(target=_rank_that_dies, args=(r, 2, 29791, out)) for r in range(2)]
  for p in procs:
    p.start()
  for p in procs:
    p.join(60)
  assert out.get(0, "").startswith("detected"), dict(out)


def test_corrupt_training_state_is_rejected(tmp_path):
  from torchprime_b200.checkpoint import train_state
  class T:  # the loader checks the shard before touching the trainer
    pass
  with pytest.raises(FileNotFoundError):
    train_state.load(str(tmp_path), T())
  (tmp_path / "rank_00000.pt").write_bytes(b"not a checkpoint")
  with pytest.raises(Exception):
    train_state.load(str(tmp_path), T())


def test_kernel_error_when_library_missing(monkeypatch):
  from torchprime_b200.ops import _lib
  monkeypatch.setattr(_lib, "_lib", None)
  monkeypatch.setattr(_lib, "_LIB_PATH", "/nonexistent/libtpb200.so")
  with pytest.raises(_lib.KernelError, match="torchprime_b200.build"):
    _lib.lib()


@pytest.mark.gpu
def test_bounded_device_wait_times_out_with_status(cuda_lib):
  from torchprime_b200.ops import _lib
  L = cuda_lib
  L.tpb_bounded_wait.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
  L.tpb_bounded_wait.restype = ctypes.c_int
  flag = torch.zeros(1, dtype=torch.int32, device="cuda")      # nothing will ever set it
  result = torch.zeros(1, dtype=torch.int32, device="cuda")
  stream = torch.cuda.current_stream().cuda_stream
  t0 = time.time()
  assert L.tpb_bounded_wait(flag.data_ptr(), 1, 400_000_000, result.data_ptr(), stream) == 0   # ~0.2-0.3 s
  torch.cuda.synchronize()
  assert time.time() - t0 < 5.0
  assert result.item() == -1
  with pytest.raises(_lib.KernelError, match="flag written by a peer"):
    _lib.raise_on_device_timeout()
  assert _lib.status()[0] == 0                                   # cleared, context still usable
  flag.fill_(1)
  assert L.tpb_bounded_wait(flag.data_ptr(), 1, 400_000_000, result.data_ptr(), stream) == 0
  torch.cuda.synchronize()
  assert result.item() == 1 and (torch.ones(4, device="cuda") * 2).sum().item() == 8.0
