"""Multi-rank behaviour on CPU (gloo): FSDP, tensor-, context- and expert-parallel runs must
reproduce the single-rank loss / gradient-norm trajectory; checkpoints round-trip; resume works."""

import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _train_worker(rank, world, port, overrides, steps, out, extra_action):
  os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                     "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
  sys.path.insert(0, ROOT)
  torch.set_num_threads(1)
  import torch.distributed as dist
  from torchprime_b200.config import compose
  from torchprime_b200.data.synthetic import make_synthetic_dataset
  from torchprime_b200.dist import runtime as rt
  from torchprime_b200.models.model_utils import initialize_model_class
  from torchprime_b200.trainer import Trainer
  try:
    rt.init(device="cpu")
    cfg = compose("default", ["dataset=synthetic", "task.optimizer.type=adamw", "task.optimizer.learning_rate=1e-3",
                              "profile_start_step=-1", "+engine.cpu_dtype=float32", f"task.max_steps={steps}"]
                  + overrides)
    torch.manual_seed(0)
    model = initialize_model_class(cfg.model, device="meta")
    data = make_synthetic_dataset(vocab_size=cfg.model.vocab_size, block_size=cfg.dataset.block_size, num_samples=64)
    tr = Trainer(model=model, config=cfg, train_dataset=data)
    loader = tr._get_train_dataloader()
    if tr.start_step:
      loader.load_state_dict({"cursor": tr.start_step})
    traj = []
    for step in range(tr.start_step, steps):
      loss, gn = tr.train_step(tr._prepare_batch(loader.next_batch()))
      l = loss.detach().clone().float()
      if dist.is_initialized():
        dist.all_reduce(l)
        l /= world
      traj.append((l.item(), gn.item()))
      if extra_action and extra_action.startswith("save_at_2:") and step + 1 == 2:
        from torchprime_b200.checkpoint import train_state
        tr._loader = loader
        train_state.save(extra_action[10:], tr, 2)
    result = {"traj": traj}
    if extra_action == "state_dict":
      sd = tr.engine.full_state_dict()
      result["norm"] = {k: v.float().norm().item() for k, v in sd.items()}
    if extra_action and extra_action.startswith("dcp:"):
      from torchprime_b200.checkpoint import dcp_io
      folder = extra_action[4:]
      dcp_io.save_distributed_checkpoint(None, folder, engine=tr.engine)
      rt.barrier()
      want = tr.engine.full_state_dict()
      if rank == 0:
        got = dcp_io.load_full_state_from_distcp(folder)
        assert got.keys() == want.keys(), (sorted(got)[:4], sorted(want)[:4])
        result["dcp_max_diff"] = max((got[k].float() - want[k].float()).abs().max().item() for k in want)
        result["dcp_files"] = sorted(os.listdir(folder))
    if rank == 0:
      out.update(result)
    rt.barrier()
  except Exception as e:  # noqa: BLE001
    import traceback
    out["error"] = "".join(traceback.format_exception(e))
  finally:
    rt.shutdown()


_PORT = [29700]


def run(world, overrides, steps=3, extra_action=None):
  _PORT[0] += 1
  mgr = mp.Manager()
  out = mgr.dict()
  if world == 1:
    _train_worker(0, 1, _PORT[0], overrides, steps, out, extra_action)
  else:
    mp.spawn(_train_worker, args=(world, _PORT[0], overrides, steps, out, extra_action), nprocs=world, join=True)
  assert "error" not in out, out["error"]
  return dict(out)


def close(a, b, tol=2e-4):
  for (la, ga), (lb, gb) in zip(a, b):
    assert abs(la - lb) < tol * max(1, abs(lb)), (a, b)
    assert abs(ga - gb) < 5 * tol * max(1, abs(gb)), (a, b)


LLAMA = ["model=llama-tiny", "dataset.block_size=64", "task.global_batch_size=4"]


@pytest.fixture(scope="module")
def llama_single():
  return run(1, LLAMA + ["ici_mesh.fsdp=1"])["traj"]


def test_fsdp2_matches_single(llama_single):
  close(run(2, LLAMA + ["ici_mesh.fsdp=2"])["traj"], llama_single)


@pytest.mark.parametrize("policy", ["none", "1"])
def test_fsdp2_saved_activations_match_single(llama_single, policy):
  """Units that keep their activations (parameters re-gathered before their backward) and a mix of
  kept and recomputed units both reproduce the single-rank run."""
  close(run(2, LLAMA + ["ici_mesh.fsdp=2", f"engine.remat_layers={policy}"])["traj"], llama_single)


def test_data2_matches_single(llama_single):
  close(run(2, LLAMA + ["ici_mesh.fsdp=1", "ici_mesh.data=2"])["traj"], llama_single)


def test_tensor2_matches_single(llama_single):
  close(run(2, LLAMA + ["ici_mesh.fsdp=1", "ici_mesh.tensor=2", "model/sharding=llama-fsdp-tp"])["traj"], llama_single)


@pytest.mark.parametrize("lb", [False, True])
def test_context2_matches_single(llama_single, lb):
  ov = LLAMA + ["ici_mesh.fsdp=1", "ici_mesh.context=2", "+model.context=2", f"+model.load_balance_cp={str(lb).lower()}",
                "model.attention_kernel=splash_attention", "model/sharding=llama-fsdp-tp-cp"]
  close(run(2, ov)["traj"], llama_single)


def test_adafactor_sharded_matches_single():
  base = LLAMA + ["task.optimizer.type=adafactor"]
  close(run(2, base + ["ici_mesh.fsdp=2"])["traj"], run(1, base + ["ici_mesh.fsdp=1"])["traj"], tol=5e-4)


MIX = ["model=mixtral-tiny", "dataset.block_size=64", "task.global_batch_size=4", "model.moe_implementation=gmm"]


def test_mixtral_expert_parallel_folded_matches_single():
  single = run(1, MIX + ["ici_mesh.fsdp=1"])["traj"]
  close(run(2, MIX + ["ici_mesh.fsdp=2"])["traj"], single)
  ep = run(2, MIX + ["ici_mesh.fsdp=2", "ici_mesh.expert=2", "expert_axis_mode=folded",
                     "model/sharding=mixtral-fsdp-ep"])["traj"]
  close(ep, single)


def test_mixtral_expert_parallel_orthogonal_matches_single():
  """An orthogonal expert axis is also a batch axis: dense gradients must be averaged over it and
  the gradient norm must count every expert rank's slices once."""
  single = run(1, MIX + ["ici_mesh.fsdp=1"])["traj"]
  ep = run(2, MIX + ["ici_mesh.fsdp=1", "ici_mesh.expert=2", "expert_axis_mode=orthogonal",
                     "model/sharding=mixtral-fsdp-ep"])["traj"]
  close(ep, single)


def test_mixtral_tensor_parallel_matches_single():
  """Attention heads and the experts' FFN dimension split over two ranks (router replicated)."""
  single = run(1, MIX + ["ici_mesh.fsdp=1"])["traj"]
  tp = run(2, MIX + ["ici_mesh.fsdp=1", "ici_mesh.tensor=2", "model/sharding=mixtral-fsdp-tp-ep"])["traj"]
  close(tp, single)


DSK = ["model=deepseek-tiny", "dataset.block_size=64", "task.global_batch_size=4"]


def test_deepseek_tensor_parallel_matches_single():
  """MLA heads, dense / shared MLPs and the grouped experts' FFN dimension split over two ranks; the
  low-rank projections, their norms and the router stay replicated and must see full gradients."""
  single = run(1, DSK + ["ici_mesh.fsdp=1"])["traj"]
  tp = run(2, DSK + ["ici_mesh.fsdp=1", "ici_mesh.tensor=2"])["traj"]
  close(tp, single)
  both = run(2, DSK + ["ici_mesh.fsdp=1", "ici_mesh.tensor=2"], steps=1, extra_action="state_dict")["norm"]
  one = run(1, DSK + ["ici_mesh.fsdp=1"], steps=1, extra_action="state_dict")["norm"]
  assert one.keys() == both.keys()
  for k in one:
    assert abs(one[k] - both[k]) < 2e-4 * max(1.0, one[k]), k


L4 = ["model=llama-4-text-only-dummy", "model.hidden_size=128", "model.num_attention_heads=4",
      "model.num_key_value_heads=2", "model.head_dim=32", "model.intermediate_size=48",
      "model.intermediate_size_mlp=96", "model.num_local_experts=4", "model.vocab_size=256",
      "model.num_hidden_layers=3", "model.moe_layers=[0,2]", "model.no_rope_layers=[1,1,0]",
      "model.floor_scale=16", "dataset.block_size=64", "task.global_batch_size=4"]


@pytest.mark.parametrize("impl", ["original", "sequential", "expert_parallelism"])
def test_llama4_tensor_parallel_matches_single(impl):
  """Heads, the shared expert and the fused gate|up expert weights (sliced half by half) split over two
  ranks, for every MoE formulation; the dense layer's MLP is not named by the config and stays whole."""
  base = L4 + [f"model.moe_implementation={impl}"]
  single = run(1, base + ["ici_mesh.fsdp=1"])["traj"]
  tp = run(2, base + ["ici_mesh.fsdp=1", "ici_mesh.tensor=2", "model/sharding=llama4-fsdp-tp"])["traj"]
  close(tp, single)


def test_resume_from_training_state(tmp_path):
  ov = LLAMA + ["ici_mesh.fsdp=2"]
  full = run(2, ov, steps=4, extra_action=f"save_at_2:{tmp_path}/ckpt")["traj"]
  resumed = run(2, ov + [f"engine.resume_from={tmp_path}/ckpt"], steps=4)["traj"]
  close(resumed, full[2:], tol=1e-5)


def test_full_state_dict_gathers_all_parameters():
  one = run(1, LLAMA + ["ici_mesh.fsdp=1"], steps=1, extra_action="state_dict")["norm"]
  two = run(2, LLAMA + ["ici_mesh.fsdp=2"], steps=1, extra_action="state_dict")["norm"]
  assert one.keys() == two.keys() and "model.layers.1.mlp.down_proj.weight" in one
  for k in one:
    assert abs(one[k] - two[k]) < 1e-4 * max(1.0, one[k]), k


@pytest.mark.parametrize("ov", [LLAMA + ["ici_mesh.fsdp=2"],
                                MIX + ["ici_mesh.fsdp=2", "ici_mesh.expert=2", "expert_axis_mode=folded",
                                       "model/sharding=mixtral-fsdp-ep"]], ids=["llama_fsdp2", "mixtral_fsdp2_ep2"])
def test_distributed_checkpoint_is_a_dcp_directory(tmp_path, ov):
  """Format B is readable by torch.distributed.checkpoint and holds every parameter whole, also with
  expert-parallel slices (which live outside the fsdp-sharded region of the flat buffers)."""
  res = run(2, ov, steps=1, extra_action=f"dcp:{tmp_path}/ckpt")
  assert res["dcp_max_diff"] == 0.0
  files = res["dcp_files"]
  assert ".metadata" in files and all(any(f.startswith(f"__{r}_") and f.endswith(".distcp") for f in files)
                                      for r in range(2)), files
