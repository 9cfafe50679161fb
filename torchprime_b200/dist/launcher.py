"""Spawns one training process per GPU on this box (a small, dependency-free torchrun).

  python -m torchprime_b200.dist.launcher --nproc 8 -m torchprime_b200.train model=llama-3-8b ici_mesh.fsdp=8

Sets RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR=127.0.0.1 / MASTER_PORT for every child, forwards
their exit codes and tears the job down when one rank fails: the first non-zero exit terminates the
remaining ranks (exact PIDs / process groups only), so a dead rank cannot leave the others
waiting in a collective.  There is a single NVSwitch box, hence no multi-node rendezvous.
"""

from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
import time


def free_port() -> int:
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def child_env(rank: int, world: int, port: int, base=None) -> dict:
  env = dict(base if base is not None else os.environ)
  env.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world), "MASTER_ADDR": "127.0.0.1",
              "MASTER_PORT": str(port), "OMP_NUM_THREADS": env.get("OMP_NUM_THREADS", "1")})
  return env


def launch(cmd: list[str], nproc: int, port: int | None = None, poll_s: float = 0.2, grace_s: float = 10.0) -> int:
  port = port or free_port()
  procs = [subprocess.Popen(cmd, env=child_env(r, nproc, port), start_new_session=True) for r in range(nproc)]
  exit_code = 0
  try:
    alive = set(range(nproc))
    while alive:
      for r in list(alive):
        rc = procs[r].poll()
        if rc is None:
          continue
        alive.discard(r)
        if rc != 0 and exit_code == 0:
          exit_code = rc
          sys.stderr.write(f"[launcher] rank {r} exited with code {rc}; stopping the other ranks\n")
          _terminate([procs[i] for i in alive], grace_s)
          alive.clear()
      time.sleep(poll_s)
  except KeyboardInterrupt:
    _terminate(procs, grace_s)
    exit_code = 130
  return exit_code


def _terminate(procs, grace_s: float):
  for p in procs:
    if p.poll() is None:
      try:
        os.killpg(p.pid, signal.SIGTERM)   # the child's own process group (start_new_session)
      except ProcessLookupError:
        pass
  deadline = time.time() + grace_s
  for p in procs:
    while p.poll() is None and time.time() < deadline:
      time.sleep(0.05)
    if p.poll() is None:
      try:
        os.killpg(p.pid, signal.SIGKILL)
      except ProcessLookupError:
        pass


def main(argv=None):
  ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
  ap.add_argument("--nproc", type=int, default=None, help="ranks to start (default: number of visible GPUs)")
  ap.add_argument("--master-port", type=int, default=None)
  ap.add_argument("-m", dest="module", default=None, help="run a module (python -m ...)")
  ap.add_argument("rest", nargs=argparse.REMAINDER)
  a = ap.parse_args(argv)
  nproc = a.nproc
  if nproc is None:
    import torch
    nproc = max(1, torch.cuda.device_count())
  cmd = [sys.executable] + (["-m", a.module] if a.module else []) + [x for x in a.rest if x != "--"]
  return launch(cmd, nproc, a.master_port)


if __name__ == "__main__":
  sys.exit(main())
