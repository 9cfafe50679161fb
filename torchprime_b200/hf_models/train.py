"""Adapter that runs HuggingFace ``run_clm.py``-style training with this repo's config grammar
(reference: torchprime/hf_models/train.py turns a Hydra config into environment variables and a
``run_clm.py --k=v`` command line for its transformers fork with XLA FSDPv2).  Here the FSDP
settings are the PyTorch ones for GPUs; the script path comes from ``train_script.path``.

  python -m torchprime_b200.hf_models.train +train_script.path=/path/run_clm.py +train_script.args.block_size=1024
"""

from __future__ import annotations

import os
import subprocess
import sys

from ..config import compose, parse_cli, to_container


def build_command(config) -> tuple[list[str], dict]:
  ts = config.get("train_script", None)
  if ts is None or not ts.get("path", None):
    raise ValueError("set +train_script.path=<run_clm.py> (and +train_script.args.<flag>=<value>)")
  args = to_container(ts.get("args", {}) or {})
  args.setdefault("per_device_train_batch_size", max(1, config.task.global_batch_size // max(1, config.ici_mesh.fsdp)))
  args.setdefault("max_steps", config.task.max_steps)
  args.setdefault("output_dir", config.output_dir)
  args.setdefault("bf16", True)
  args.setdefault("fsdp", "full_shard auto_wrap")
  cmd = [sys.executable, ts.path] + [f"--{k}={v}" for k, v in args.items() if v is not None]
  env = {"TORCHPRIME_PROFILE_DIR": str(config.profile_dir), "TORCHPRIME_OUTPUT_DIR": str(config.output_dir)}
  return cmd, env


def main(argv=None):
  name, overrides = parse_cli(sys.argv[1:] if argv is None else argv)
  cfg = compose(name or "default", overrides)
  cmd, env = build_command(cfg)
  full_env = dict(os.environ)
  full_env.update(env)
  nproc = int(cfg.ici_mesh.fsdp) * int(cfg.ici_mesh.data)
  launcher = [sys.executable, "-m", "torchprime_b200.dist.launcher", "--nproc", str(nproc)] + cmd[1:]
  print("[hf_models] " + " ".join(launcher))
  return subprocess.call(launcher, env=full_env)


if __name__ == "__main__":
  sys.exit(main())
