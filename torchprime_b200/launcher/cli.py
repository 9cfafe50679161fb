"""``tp`` — command line front end (the counterpart of the reference's launcher CLI,
torchprime/launcher/cli.py:272-805, whose job is to ship a script to a TPU cluster with xpk).

On a B200 box the same verbs act locally:

  tp use --gpus 8 --artifact-dir /data/runs        remember defaults in .config/default.toml
  tp run [--name N] <script.py | -m module> ARGS   start one rank per GPU, add profile_dir= / output_dir=
  tp run -i ...                                    the same, started again whenever a source file changes
  tp save-hf-model-files --repo-id R --dest D      snapshot tokenizer / weights from the hub into a directory
  tp save-hf-dataset --dataset-name N --dest D     snapshot (or tokenise and pack) a hub dataset
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


class FileChangeWatcher:
  """Polls the modification times of the source files under ``root`` (``.gitignore`` rules applied, like
  the reference's interactive mode, launcher/cli.py:494-571).  ``changed()`` reports the paths that were
  added, removed or rewritten since the previous call."""

  SUFFIXES = (".py", ".yaml", ".yml", ".cu", ".cuh", ".h", ".toml", ".json")

  def __init__(self, root: str = "."):
    self.root = os.path.abspath(root)
    self._spec = None
    gi = os.path.join(self.root, ".gitignore")
    if os.path.exists(gi):
      try:
        import pathspec
        with open(gi) as f:
          self._spec = pathspec.PathSpec.from_lines("gitwildmatch", f)
      except ImportError:
        self._spec = None
    self._seen = self._scan()

  def _ignored(self, rel: str) -> bool:
    if rel.startswith(".git" + os.sep) or rel == ".git":
      return True
    return self._spec is not None and self._spec.match_file(rel)

  def _scan(self) -> dict:
    out = {}
    for base, dirs, files in os.walk(self.root):
      rel_base = os.path.relpath(base, self.root)
      dirs[:] = [d for d in dirs if not self._ignored(os.path.normpath(os.path.join(rel_base, d)) + os.sep)
                 and not self._ignored(os.path.normpath(os.path.join(rel_base, d)))]
      for name in files:
        if not name.endswith(self.SUFFIXES):
          continue
        rel = os.path.normpath(os.path.join(rel_base, name))
        if self._ignored(rel):
          continue
        try:
          out[rel] = os.stat(os.path.join(base, name)).st_mtime_ns
        except OSError:
          pass
    return out

  def changed(self) -> list[str]:
    now = self._scan()
    diff = sorted(k for k in set(now) | set(self._seen) if now.get(k) != self._seen.get(k))
    self._seen = now
    return diff


def run_interactive(start, watcher: FileChangeWatcher, poll_s: float = 1.0, max_runs: int | None = None,
                    sleep=None) -> int:
  """Start the workload with ``start()`` (returns a ``subprocess.Popen``-like object), and start it again,
  after stopping the running one, whenever a watched file changes.  Returns the last exit code; ends on
  Ctrl-C or after ``max_runs`` starts once the last one has exited."""
  import time
  sleep = sleep or time.sleep
  runs, proc, rc = 0, None, 0
  try:
    while True:
      if proc is None:
        proc = start()
        runs += 1
      sleep(poll_s)
      changes = watcher.changed()
      done = proc.poll() is not None
      if done:
        rc = proc.returncode
      if changes and (max_runs is None or runs < max_runs):
        print(f"[tp] {len(changes)} file(s) changed ({', '.join(changes[:3])}{' ...' if len(changes) > 3 else ''}); "
              "starting again")
        if not done:
          _stop(proc)
        proc = None
        continue
      if done and max_runs is not None and runs >= max_runs:
        return rc
  except KeyboardInterrupt:
    if proc is not None and proc.poll() is None:
      _stop(proc)
    return rc


def _stop(proc):
  """End the workload's own process group (the launcher and its ranks), nothing else."""
  import signal
  try:
    # only a process this launcher started in a session of its own has a group that is safe to signal
    if isinstance(proc, subprocess.Popen) and proc.pid > 1 and os.getpgid(proc.pid) == proc.pid:
      os.killpg(proc.pid, signal.SIGTERM)
    else:
      proc.terminate()
  except (ProcessLookupError, PermissionError, OSError):
    proc.terminate()
  try:
    proc.wait(timeout=20)
  except subprocess.TimeoutExpired:
    proc.kill()


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
  if a.interactive:
    return run_interactive(lambda: subprocess.Popen(full, env=env, start_new_session=True), FileChangeWatcher("."))
  return subprocess.call(full, env=env)


def cmd_save_hf_model_files(a):
  from . import save_hf_assets
  os.makedirs(a.dest, exist_ok=True)
  print("saved", save_hf_assets.save_repo(a.repo_id, a.dest, a.file_type, a.token))
  return 0


def cmd_save_hf_dataset(a):
  from . import save_hf_assets
  os.makedirs(a.dest, exist_ok=True)
  print("saved", save_hf_assets.save_dataset(a.dataset_name, a.dataset_config, a.dest, a.split, a.tokenizer,
                                             a.block_size))
  return 0


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
  p.add_argument("--dry-run", action="store_true"); p.add_argument("-m", dest="module")
  p.add_argument("-i", "--interactive", action="store_true", help="run again whenever a source file changes")
  p.add_argument("args", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_run)
  for verb in ("save-hf-model-files", "save-hf-model-files-to-gcs"):
    p = sub.add_parser(verb); p.add_argument("--repo-id", required=True); p.add_argument("--dest", required=True)
    p.add_argument("--file-type", nargs="+", default=["tokenizer", "model"], choices=["tokenizer", "model"])
    p.add_argument("--token", default=os.environ.get("HF_TOKEN")); p.set_defaults(fn=cmd_save_hf_model_files)
  p = sub.add_parser("save-hf-dataset"); p.add_argument("--dataset-name", required=True); p.add_argument("--dataset-config")
  p.add_argument("--dest", required=True); p.add_argument("--split", default="train"); p.add_argument("--tokenizer")
  p.add_argument("--block-size", type=int); p.set_defaults(fn=cmd_save_hf_dataset)
  p = sub.add_parser("test"); p.add_argument("args", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_test)
  p = sub.add_parser("doctor"); p.set_defaults(fn=cmd_doctor)
  p = sub.add_parser("build"); p.set_defaults(fn=cmd_build)
  p = sub.add_parser("mfu"); p.add_argument("args", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_mfu)
  a = ap.parse_args(argv)
  return a.fn(a) or 0


if __name__ == "__main__":
  sys.exit(main())
