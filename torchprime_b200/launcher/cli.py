"""``tp`` — command line front end (the counterpart of the reference's launcher CLI,
torchprime/launcher/cli.py:272-805, whose job is to ship a script to a TPU cluster with xpk).

On a B200 box the same verbs act locally:

  tp use --gpus 8 --artifact-dir /data/runs        remember defaults in .config/default.toml
  tp run [--name N] <script.py | -m module> ARGS   start one rank per GPU, add profile_dir= / output_dir=
  tp test [pytest args]                            run the test suite
  tp doctor                                        check toolchain, GPUs, P2P, the kernel library
  tp build                                         compile the sm_100a kernel library
  tp mfu --config X --batch-size B ...             MFU calculator

``tp run`` exports the ``TORCHPRIME_*`` environment the reference's workloads expect
(ARTIFACT_DIR, JOBSET_NAME, USER, COMMENTS, ACCELERATOR_TYPE) and, like its ``thunk.py``
(launcher/thunk.py:69-95), appends ``profile_dir=`` and ``output_dir=`` under
``<artifact_dir>/<jobset>/`` to the workload's arguments and propagates the exit code.
"""

from __future__ import annotations

import argparse
import datetime
import getpass
import os
import re
import subprocess
import sys

try:
  import tomllib
except ModuleNotFoundError:  # pragma: no cover
  tomllib = None

CONFIG_PATH = os.path.join(".config", "default.toml")
FORWARDED_ENV = ("HF_TOKEN", "NCCL_DEBUG", "NCCL_NVLS_ENABLE", "CUDA_VISIBLE_DEVICES", "TPB_ATTN_BWD_DEBUG")


def load_config(path: str = CONFIG_PATH) -> dict:
  if not os.path.exists(path) or tomllib is None:
    return {}
  with open(path, "rb") as f:
    return tomllib.load(f)


def save_config(cfg: dict, path: str = CONFIG_PATH):
  os.makedirs(os.path.dirname(path), exist_ok=True)
  with open(path, "w") as f:
    for k, v in cfg.items():
      f.write(f"{k} = {v!r}\n" if not isinstance(v, str) else f'{k} = "{v}"\n')


def generate_jobset_name(name: str | None = None, now: datetime.datetime | None = None) -> str:
  """``<user>-<name>-<timestamp>`` restricted to DNS-label characters, at most 40 chars."""
  now = now or datetime.datetime.now()
  user = re.sub(r"[^a-z0-9]", "", getpass.getuser().lower())[:12] or "user"
  stem = re.sub(r"[^a-z0-9-]", "-", (name or "run").lower()).strip("-")
  return f"{user}-{stem}"[:24].rstrip("-") + "-" + now.strftime("%Y%m%d-%H%M%S")


def workload_env(cfg: dict, jobset: str, comments: str = "") -> dict:
  env = {k: os.environ[k] for k in FORWARDED_ENV if k in os.environ}
  artifact = cfg.get("artifact_dir", "outputs")
  env.update({
    "TORCHPRIME_ARTIFACT_DIR": artifact, "TORCHPRIME_JOBSET_NAME": jobset, "TORCHPRIME_USER": getpass.getuser(),
    "TORCHPRIME_COMMENTS": comments, "TORCHPRIME_ACCELERATOR_TYPE": f"b200-{cfg.get('gpus', 1)}",
    "TORCHPRIME_NUM_SLICES": "1",
  })
  return env


def workload_args(args: list[str], cfg: dict, jobset: str) -> list[str]:
  base = os.path.join(cfg.get("artifact_dir", "outputs"), jobset)
  out = list(args)
  if not any(a.startswith("profile_dir=") for a in out):
    out.append(f"profile_dir={os.path.join(base, 'profile', '0-0')}")
  if not any(a.startswith("output_dir=") for a in out):
    out.append(f"output_dir={os.path.join(base, 'outputs', '0-0')}")
  return out


def cmd_use(a):
  cfg = load_config()
  cfg.update({"gpus": a.gpus, "artifact_dir": a.artifact_dir})
  save_config(cfg)
  print(f"wrote {CONFIG_PATH}: {cfg}")
  return cmd_doctor(a)


def cmd_run(a):
  cfg = load_config()
  gpus = a.gpus or cfg.get("gpus", 1)
  cfg["gpus"] = gpus
  jobset = generate_jobset_name(a.name)
  rest = [x for x in a.args if x != "--"]
  if a.module:
    target = ["-m", a.module]
  else:
    if not rest:
      raise SystemExit("tp run: give a script path or -m module")
    target, rest = [rest[0]], rest[1:]
  full = [sys.executable, "-m", "torchprime_b200.dist.launcher", "--nproc", str(gpus)] + target + workload_args(rest, cfg, jobset)
  env = dict(os.environ)
  env.update(workload_env(cfg, jobset, a.comments or ""))
  print("[tp] " + " ".join(full))
  if a.dry_run:
    return 0
  return subprocess.call(full, env=env)


def cmd_test(a):
  return subprocess.call([sys.executable, "-m", "pytest", "tests"] + (a.args or ["-q", "-m", "not gpu"]))


def cmd_doctor(_a):
  from .doctor import run_checks
  return run_checks()


def cmd_build(_a):
  from .. import build
  print(build.build())
  return 0


def cmd_mfu(a):
  from ..metrics import mfu
  return mfu.main(a.args)


def main(argv=None):
  ap = argparse.ArgumentParser(prog="tp", description="torchprime_b200 launcher")
  sub = ap.add_subparsers(dest="cmd", required=True)
  p = sub.add_parser("use"); p.add_argument("--gpus", type=int, default=8); p.add_argument("--artifact-dir", default="outputs"); p.set_defaults(fn=cmd_use)
  p = sub.add_parser("run"); p.add_argument("--name"); p.add_argument("--gpus", type=int); p.add_argument("--comments")
  p.add_argument("--dry-run", action="store_true"); p.add_argument("-m", dest="module"); p.add_argument("args", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_run)
  p = sub.add_parser("test"); p.add_argument("args", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_test)
  p = sub.add_parser("doctor"); p.set_defaults(fn=cmd_doctor)
  p = sub.add_parser("build"); p.set_defaults(fn=cmd_build)
  p = sub.add_parser("mfu"); p.add_argument("args", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_mfu)
  a = ap.parse_args(argv)
  return a.fn(a) or 0


if __name__ == "__main__":
  sys.exit(main())
