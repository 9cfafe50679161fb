"""Training loop.

Public surface of the reference's ``Trainer`` (torchprime/torch_xla_models/trainer/
base_trainer.py:84-380): ``Trainer(model, config, train_dataset)``, ``train_loop()``,
``train_step(batch)``, ``clip_gradients()``, ``finalize_training(metrics_logger)``,
``Trainer._create_optimizer(config, params)``; same log lines (``Epoch: ..., step: ...,
loss: ..., grad_norm: ..., lr: ..., trace time: ... ms`` and ``Finished training run``),
TensorBoard tags and output files.

Execution differs by design: one process per GPU, eager PyTorch driving hand-written
kernels through the FSDP engine (parallel/fsdp.py) instead of one compiled XLA graph; the
step time comes from CUDA events on the compute stream (max over ranks) instead of from
the device profile; the profiling window produces a Chrome trace via ``torch.profiler``.
"""

from __future__ import annotations

import json
import logging
import math
import os
import time
from pathlib import Path

import torch
import torch.nn as nn

from ..config import to_container
from ..data.loader import ShardedBatchLoader
from ..dist import runtime as rt
from ..metrics.mfu import compute_mfu
from ..metrics.step_timer import StepTimer
from ..ops import functional as ops
from ..ops import reference as ref
from ..parallel.fsdp import FSDPEngine
from ..parallel.optimizer import LRScheduler, create_optimizer
from ..rewriting.assume_pure import mark_pure_modules
from ..rewriting.auto_trace import auto_trace
from ..rewriting.rematerialization_utils import add_activation_checkpointing_and_scan, add_optimization_barriers
from ..rewriting.sharding_initialization import setup_sharding_and_mesh
from ..utils import profiling
from ..utils.parallelism_utils import cp_enabled, lb_cp_enabled, reorder_sequence

logger = logging.getLogger(__name__)

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _remat_policy(v):
  """``engine.remat_layers``: all | none | auto | <number of layers that recompute>."""
  if isinstance(v, bool):
    return "all" if v else "none"
  if isinstance(v, int):
    return v
  v = str(v).lower()
  if v in ("all", "none", "auto"):
    return v
  return int(v)


class Trainer:
  minibatch: bool

  def __init__(self, model: nn.Module, config, train_dataset):
    self.config = config
    profiling.ensure_profile_end_step(self.config)
    self.device = rt.device()
    self.global_batch_size = self.config.task.global_batch_size
    self.train_dataset = train_dataset
    self._initialize_tensorboard_writer()

    eng = self.config.get("engine", {}) or {}
    if eng.get("kernels", "sm100") == "torch":
      ops.set_backend("torch")
    # One switch for every NVSwitch multicast binding (multimem stores of the fused all-gather and the
    # context-parallel K/V push, multimem reductions of the tensor-parallel GEMM epilogues).  A rank that
    # dies while its memory is bound to a multicast object can fault its peers' GPUs, so any mode that
    # ends a rank abruptly (a watchdog that aborts, elastic exit) has to run with it off.
    self.multicast = bool(eng.get("multicast", True))
    if not self.multicast:
      for key in ("TPB_AG_MULTICAST", "TPB_TP_FUSED", "TPB_CP_MULTICAST"):
        os.environ[key] = "0"
    if bool(eng.get("watchdog_abort", False)) and self.multicast and rt.world_size() > 1:
      raise ValueError("engine.watchdog_abort=true ends a rank without tearing down its peers: set "
                       "engine.multicast=false (and NCCL_NVLS_ENABLE=0 in the environment) with it")

    # -- model transformations (same order as the reference's constructor) --
    model = auto_trace(model)
    self.sharding = setup_sharding_and_mesh(model, config)
    self.mesh = self.sharding.mesh
    self.input_sharding_spec = self.sharding.input_sharding_spec
    self.minibatch = self.sharding.minibatch
    model = mark_pure_modules(model, config)
    self.remat_plan = add_activation_checkpointing_and_scan(model, config)
    model = add_optimization_barriers(model, config, self.remat_plan)
    self.model = model

    dtype = _DTYPES[str(self.config.get("torch_dtype", "bfloat16"))]
    if self.device.type == "cpu" and eng.get("cpu_dtype", None):
      dtype = _DTYPES[eng.cpu_dtype]
    self.engine = FSDPEngine(
      model, self.mesh, self.sharding.plan, device=self.device, param_dtype=dtype,
      grad_dtype=_DTYPES[eng.grad_dtype] if eng.get("grad_dtype", None) else None,
      master_weights=bool(eng.get("master_weights", True)),
      remat_classes=self.remat_plan.remat_classes, offload_tensors=self.remat_plan.offload_tensors,
      seed=int(self.config.get("seed", 42)), fused_collectives=bool(eng.get("fused_collectives", False)),
      remat_policy=_remat_policy(eng.get("remat_layers", "auto")),
      fused_expert_exchange=bool(eng.get("fused_expert_exchange", False)),
      collectives=str(eng.get("fsdp_collectives", "auto")), keep_gathered=eng.get("keep_gathered", "auto"),
      cuda_graphs=bool(eng.get("cuda_graphs", False)))
    _move_buffers(model, self.device)
    if hasattr(model, "return_logits"):
      model.return_logits = not bool(eng.get("chunked_ce", True))
    if cp_enabled(config) and hasattr(model, "cp"):
      from ..parallel.cp import ContextParallelAttention
      model.cp = ContextParallelAttention(self.mesh, load_balanced=lb_cp_enabled(config),
                                          fused_exchange=bool(eng.get("fused_collectives", False)) and self.device.type == "cuda")
      if getattr(model, "_head", None) is not None:
        model._head.loss_group = self.mesh.group("context")
      if hasattr(model, "model"):
        model.model.max_rope_positions = int(config.dataset.block_size)

    self.optimizer = type(self)._create_optimizer(config, self.engine)
    self.lr_scheduler = LRScheduler(
      base_lr=float(self.config.task.optimizer.learning_rate),
      kind=str(self.config.task.lr_scheduler.type),
      warmup_steps=int(self.config.task.lr_scheduler.warmup_steps),
      total_steps=int(self.config.task.max_steps))
    self.step_timer = StepTimer(use_cuda=self.device.type == "cuda")
    self._profiler = None
    self.start_step = 0
    self.watchdog = None
    if float(eng.get("watchdog_seconds", 0) or 0) > 0:
      from ..dist.watchdog import StepWatchdog
      # abort=False: a late step is logged with a stack dump and raised at the END of that step, which
      # cannot end a step that never finishes; engine.watchdog_abort=true exits the process instead
      self.watchdog = StepWatchdog(float(eng.watchdog_seconds), abort=bool(eng.get("watchdog_abort", False)))
    if eng.get("resume_from", None):
      from ..checkpoint import train_state
      self.start_step = train_state.load(eng.resume_from, self)
    if self.device.type == "cuda":
      torch.cuda.synchronize()

  # ------------------------------------------------------------------ factories
  @staticmethod
  def _create_optimizer(config, engine_or_params):
    """AdamW / Adafactor from ``task.optimizer``.  Given an FSDP engine the optimizer is the
    sharded fused one; given plain parameters (unit tests, small models) it is the
    torch / transformers implementation the reference uses."""
    if isinstance(engine_or_params, FSDPEngine):
      return create_optimizer(config.task, engine_or_params)
    oc = config.task.optimizer
    kind = str(oc.type).lower()
    params = list(engine_or_params)
    if kind == "adamw":
      kw = {"weight_decay": float(oc.weight_decay)} if oc.get("weight_decay", None) is not None else {}
      return torch.optim.AdamW(params, lr=float(oc.learning_rate), **kw)
    if kind == "adafactor":
      if oc.get("weight_decay", None):
        raise ValueError("Adafactor does not support weight decay.")
      from transformers.optimization import Adafactor
      return Adafactor(params, lr=float(oc.learning_rate), relative_step=False, scale_parameter=False)
    raise ValueError(f"Unsupported optimizer type: {oc.type}. Supported types are 'adafactor' and 'adamw'.")

  def _initialize_tensorboard_writer(self):
    self.summary_writer = None
    if not rt.is_main():
      return
    run_name = self.config.get("run_name", None) or time.strftime("%b%d_%H-%M-%S")
    tb_dir = Path(self.config.output_dir) / "runs" / run_name
    try:
      from torch.utils.tensorboard import SummaryWriter
      self.summary_writer = SummaryWriter(log_dir=str(tb_dir))
      logger.info("Tensorboard logging to %s", tb_dir)
    except Exception as e:  # noqa: BLE001 - TensorBoard is optional
      logger.warning("TensorBoard writer unavailable: %s", e)

  def _log_to_tensorboard(self, epoch, step, loss, learning_rate, grad_norm):
    w = self.summary_writer
    if w is None:
      return
    w.add_scalar("train/epoch", epoch, step)
    w.add_scalar("train/loss", loss, step)
    w.add_scalar("train/learning_rate", learning_rate, step)
    w.add_scalar("train/grad_norm", grad_norm, step)
    w.flush()

  # ------------------------------------------------------------------ data
  def _get_train_dataloader(self) -> ShardedBatchLoader:
    if self.train_dataset is None:
      raise ValueError("Trainer: training requires a train_dataset.")
    axes = self.sharding.batch_axes
    replicas, index = self.mesh.size(axes), self.mesh.index(axes)
    logger.info("Num replicas: %d", replicas)
    return ShardedBatchLoader(self.train_dataset, self.global_batch_size, replicas, index, self.device,
                              shuffle=True, seed=0)

  def _prepare_batch(self, batch: dict) -> dict:
    """Shift labels on the token grid, then (context parallel) permute and split the sequence."""
    batch = dict(batch)
    if "labels" in batch:
      batch["labels"] = ref.shift_labels(batch["labels"])
      batch["labels_are_shifted"] = True
    cp = self.mesh.size("context")
    if cp > 1:
      s = batch["input_ids"].shape[1]
      pos = torch.arange(s, device=batch["input_ids"].device)[None].expand_as(batch["input_ids"])
      tensors = {k: v for k, v in batch.items() if isinstance(v, torch.Tensor) and v.dim() >= 2}
      tensors["position_ids"] = pos
      r = self.mesh.index("context")
      for k, v in tensors.items():
        if lb_cp_enabled(self.config):
          v = reorder_sequence(v, cp_size=cp, seq_dim=1, to_contiguous=False)
        batch[k] = v.chunk(cp, dim=1)[r].contiguous()
    if not _accepts(self.model, "labels_are_shifted"):
      batch.pop("labels_are_shifted", None)
    return batch

  # ------------------------------------------------------------------ loop
  def train_loop(self) -> None:
    self.model.train()
    self.optimizer.zero_grad()
    max_step = self.config.task.max_steps
    loader = self._get_train_dataloader()
    steps_per_epoch = loader.epoch_batches
    if self.start_step:
      loader.load_state_dict({"cursor": self.start_step})
    self._loader = loader

    logger.info("Starting training")
    logger.info("    Max step: %d", max_step)
    logger.info("    Global batch size: %d", self.global_batch_size)

    ckpt_every = int((self.config.get("engine", {}) or {}).get("checkpoint_every", 0) or 0)
    for step in range(self.start_step, max_step):
      if self.watchdog is not None:
        self.watchdog.begin_step(step)
      self.step_timer.mark(step)
      batch = self._prepare_batch(loader.next_batch())
      t0 = time.perf_counter()
      loss, grad_norm = self.train_step(batch)
      t1 = time.perf_counter()
      self._check_device_status(step, synchronize=False)

      if step % self.config.logging_steps == 0:
        lr = self.lr_scheduler.get_last_lr()[0]
        loss_v, gn_v = float(loss.detach().item()), float(grad_norm.detach().item())
        logger.info("Epoch: %.4f, step: %d, loss: %.4f, grad_norm: %.4f, lr: %.2e, trace time: %.2f ms",
                    step / steps_per_epoch, step, loss_v, gn_v, lr, (t1 - t0) * 1000)
        self._log_to_tensorboard(step / steps_per_epoch, step, loss_v, lr, gn_v)
        if math.isnan(loss_v):
          raise ValueError(f"Loss is NaN at step {step}")
        self._check_device_status(step, synchronize=False)   # loss.item() above synchronised the device

      if step == self.config.profile_start_step:
        self._start_profile()
      if step == self.config.profile_end_step:
        self._stop_profile()
      if ckpt_every and (step + 1) % ckpt_every == 0:
        from ..checkpoint import train_state
        self._check_device_status(step, synchronize=True)    # never checkpoint a state a timed-out wait produced
        train_state.save(os.path.join(self.config.output_dir, "checkpoints", f"step_{step + 1}"), self, step + 1)
      if self.watchdog is not None:
        self.watchdog.end_step(step)

    self.step_timer.mark(max_step)
    self._stop_profile()
    if self.device.type == "cuda":
      torch.cuda.synchronize()
      from ..ops import _lib
      if _lib.available():
        _lib.raise_on_device_timeout()
    if self.watchdog is not None:
      self.watchdog.stop()
    logger.info("Finished training run")

  def _check_device_status(self, step: int, synchronize: bool):
    """Raise if a bounded device-side wait (peer flag, barrier, mbarrier) gave up.  The status block is
    host-mapped memory, so reading it costs no device round trip and is done every step; a kernel that
    gave up let its consumers read partial data, so the run must not continue or be checkpointed."""
    if self.device.type != "cuda":
      return
    from ..ops import _lib
    if not _lib.available():
      return
    if synchronize:
      torch.cuda.synchronize()
    try:
      _lib.raise_on_device_timeout()
    except _lib.KernelError as e:
      raise _lib.KernelError(f"at training step {step}: {e}") from e

  def _start_profile(self):
    if self._profiler is not None:
      return
    if self.device.type == "cuda":
      torch.cuda.synchronize()
    os.makedirs(self.config.profile_dir, exist_ok=True)
    acts = [torch.profiler.ProfilerActivity.CPU]
    if self.device.type == "cuda":
      acts.append(torch.profiler.ProfilerActivity.CUDA)
    profiling.set_tracing(True)
    self._profiler = torch.profiler.profile(activities=acts)
    self._profiler.__enter__()

  def _stop_profile(self):
    if self._profiler is None:
      return
    if self.device.type == "cuda":
      torch.cuda.synchronize()
    self._profiler.__exit__(None, None, None)
    profiling.set_tracing(False)
    path = os.path.join(self.config.profile_dir, f"trace_rank{rt.rank()}.json")
    try:
      self._profiler.export_chrome_trace(path)
    except Exception as e:  # noqa: BLE001
      logger.warning("could not write profile %s: %s", path, e)
    self._profiler = None

  # ------------------------------------------------------------------ one step
  def train_step(self, batch: dict) -> tuple[torch.Tensor, torch.Tensor]:
    _logits, loss = self.model(**batch)
    loss.backward()
    self.engine.finish_grad_sync()
    grad_norm = self.clip_gradients()
    self.optimizer.step(self.lr_scheduler.get_last_lr()[0])
    self.lr_scheduler.step()
    self.optimizer.zero_grad()
    return loss, grad_norm

  def clip_gradients(self):
    """Global L2 norm (clipping to ``task.max_grad_norm`` when > 0, else only measured), and
    optional element-wise clamping to ``task.max_grad_value``."""
    max_norm = self.config.task.get("max_grad_norm", None)
    max_value = self.config.task.get("max_grad_value", None)
    return self.optimizer.clip_gradients(max_norm if (max_norm and max_norm > 0) else None, max_value)

  # ------------------------------------------------------------------ wrap-up
  def _accelerator_name(self) -> str | None:
    name = os.environ.get("TORCHPRIME_ACCELERATOR_TYPE") or os.environ.get("TORCHPRIME_TPU_TYPE")
    if name:
      return name
    if self.device.type == "cuda" and "B200" in torch.cuda.get_device_name(self.device):
      return f"b200-{rt.world_size()}"
    return None

  def finalize_training(self, metrics_logger) -> None:
    cfg = self.config
    if cfg.profile_start_step >= 0 and cfg.profile_end_step >= 0:
      lo, hi = cfg.profile_start_step, cfg.profile_end_step
    else:
      lo, hi = min(self.start_step + 2, cfg.task.max_steps - 1), None
    step_duration = self.step_timer.step_duration(lo, hi)
    if step_duration:
      metrics_logger.log_step_execution_time(step_duration)
      tokens = cfg.dataset.block_size * cfg.task.global_batch_size
      metrics_logger.log_tokens_per_second(tokens // step_duration)
      logger.info("tokens/s (exact): %.2f  device step time: %.6f s", tokens / step_duration, step_duration)
      metrics_logger.log_num_steps(cfg.task.max_steps)
      name = self._accelerator_name()
      if name and "hidden_size" in cfg.model:
        try:
          mfu = compute_mfu(config=to_container(cfg.model), batch_size=cfg.task.global_batch_size,
                            step_duration=step_duration, tpu_name=name, sequence_length=cfg.dataset.block_size,
                            torch_dtype=str(cfg.get("torch_dtype", "bfloat16")))
          metrics_logger.log_mfu(mfu.mfu)
        except (KeyError, ValueError, AssertionError) as e:
          logger.warning("MFU not computed: %s", e)
    metrics = metrics_logger.finalize()
    logger.info("***** train metrics *****\n%s", metrics)
    if rt.is_main():
      metrics.save(Path(cfg.output_dir) / "train_metrics.json")
      with open(Path(cfg.output_dir) / "train_config.json", "w") as f:
        json.dump(to_container(cfg), f, indent=2)


def _move_buffers(model: nn.Module, device):
  for mod in model.modules():
    for name, buf in list(mod.named_buffers(recurse=False)):
      if buf is not None and buf.device != device and not buf.is_meta:
        mod._buffers[name] = buf.to(device)


def _accepts(model: nn.Module, kwarg: str) -> bool:
  import inspect
  try:
    return kwarg in inspect.signature(model.forward).parameters
  except (TypeError, ValueError):
    return False
