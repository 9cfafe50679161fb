"""MoE kernels (router, grouped GEMMs, gather/combine) and MoE models on the GPU."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from torchprime_b200.ops import _lib, moe, reference as ref


def _rel(a, b):
  return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("E,K", [(8, 2), (64, 6), (256, 8)])
def test_router_softmax(cuda_lib, E, K):
  torch.manual_seed(0)
  logits = torch.randn(333, E, device="cuda")
  w, idx, probs = moe.router_topk(logits, K, mode="softmax")
  w_ref, idx_ref, p_ref = ref.router_softmax_topk(logits, K)
  assert torch.equal(idx.long().sort(-1)[0], idx_ref.sort(-1)[0])
  assert torch.allclose(w.sort(-1)[0], w_ref.sort(-1)[0], atol=1e-5)
  assert torch.allclose(probs, p_ref, atol=1e-6)


@pytest.mark.parametrize("E,K,ng,tg", [(64, 6, 1, 1), (256, 8, 8, 4), (8, 2, 2, 1)])
def test_router_sigmoid_groups(cuda_lib, E, K, ng, tg):
  torch.manual_seed(1)
  logits = torch.randn(200, E, device="cuda")
  bias = 0.1 * torch.randn(E, device="cuda")
  w, idx, _ = moe.router_topk(logits, K, mode="sigmoid", bias=bias, n_group=ng, topk_group=tg, norm_topk=True, scale=2.5)
  w_ref, idx_ref, _ = ref.router_sigmoid_group_topk(logits, bias, K, ng, tg, True, 2.5)
  assert torch.equal(idx.long().sort(-1)[0], idx_ref.sort(-1)[0])
  assert torch.allclose(w.sort(-1)[0], w_ref.sort(-1)[0], atol=1e-5, rtol=1e-4)


def test_router_gradient(cuda_lib):
  torch.manual_seed(2)
  logits = torch.randn(64, 8, device="cuda", requires_grad=True)
  w, idx, _ = moe.router_topk(logits, 2, mode="softmax")
  g = torch.randn_like(w)
  w.backward(g)
  lr = logits.detach().clone().requires_grad_(True)
  wr, ir, _ = ref.router_softmax_topk(lr, 2)
  order = ir.argsort(-1)
  mine = idx.long().argsort(-1)
  (wr.gather(1, order) * g.gather(1, mine)).sum().backward()
  assert torch.allclose(logits.grad, lr.grad, atol=1e-5)


@pytest.mark.parametrize("capacity", [None, 24])
def test_dispatch_plan(cuda_lib, capacity):
  torch.manual_seed(3)
  T, K, E = 100, 2, 4
  idx = torch.randint(0, E, (T, K), device="cuda", dtype=torch.int32)
  plan = moe.build_dispatch_plan(idx, E, capacity, rows_per_group=50)
  dest = plan.dest.long()
  kept = dest >= 0
  assert plan.k_offsets[-1].item() % 128 == 0
  # every kept pair sits in its expert's segment and the inverse maps agree
  for e in range(E):
    lo, hi = plan.k_offsets[e].item(), plan.k_offsets[e + 1].item()
    d = dest[(idx == e) & kept]
    assert ((d >= lo) & (d < lo + plan.counts[e])).all() and hi - lo >= plan.counts[e]
  rows = dest[kept]
  assert torch.equal(plan.src_pair[rows], torch.nonzero(kept.reshape(-1)).squeeze(1))
  assert (plan.src_row >= 0).sum().item() == kept.sum().item()
  if capacity is None:
    assert kept.all()
  else:
    for g in range(2):
      for e in range(E):
        assert ((idx[g * 50:(g + 1) * 50] == e) & kept[g * 50:(g + 1) * 50]).sum() <= capacity
  te = plan.tile_expert
  for i, e in enumerate(te.tolist()):
    if e >= 0:
      assert plan.k_offsets[e] <= i * 128 < plan.k_offsets[e + 1]


@pytest.mark.parametrize("T,K,E", [(3000, 6, 64), (1111, 8, 256), (5, 1, 3), (8192, 2, 8)])
def test_dispatch_plan_kernel_equals_the_sort_based_plan(cuda_lib, T, K, E):
  """One-CTA counting sort against the torch formulation (stable argsort): identical rows."""
  torch.manual_seed(11)
  idx = torch.randint(0, E, (T, K), device="cuda", dtype=torch.int32)
  if E > 4:
    idx[idx == 1] = 2                                       # an expert that receives nothing
  for align in (128, 256):
    a = moe.build_dispatch_plan(idx, E, use_kernel=True, row_align=align)
    b = moe.build_dispatch_plan(idx, E, use_kernel=False, row_align=align)
    assert a.row_align == align and all(v % align == 0 for v in a.k_offsets.tolist())
    assert torch.equal(a.k_offsets, b.k_offsets) and torch.equal(a.dest, b.dest)
    assert torch.equal(a.tile_expert, b.tile_expert) and torch.equal(a.src_pair, b.src_pair)
  assert a.num_rows == b.num_rows
  assert torch.equal(a.counts.long(), b.counts.long()) and torch.equal(a.k_offsets, b.k_offsets)
  assert torch.equal(a.dest, b.dest) and torch.equal(a.src_pair, b.src_pair) and torch.equal(a.src_row, b.src_row)
  assert torch.equal(a.tile_expert, b.tile_expert)
  again = moe.build_dispatch_plan(idx, E, use_kernel=True, row_align=256)
  assert torch.equal(a.dest, again.dest)


def test_grouped_mlp_on_cta_pair_tiles(cuda_lib):
  """Enough rows per expert for 256-row segments: the forward, input-gradient and weight-gradient
  grouped GEMMs run on 256x256 CTA-pair tiles; one expert gets no rows at all."""
  torch.manual_seed(5)
  T, K, E, D, Fd = 2048, 2, 4, 1024, 2048
  x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
  wg = (torch.randn(E, D, Fd, device="cuda") / D ** 0.5).to(torch.bfloat16).requires_grad_(True)
  wu = (torch.randn(E, D, Fd, device="cuda") / D ** 0.5).to(torch.bfloat16).requires_grad_(True)
  wd = (torch.randn(E, Fd, D, device="cuda") / Fd ** 0.5).to(torch.bfloat16).requires_grad_(True)
  logits = torch.randn(T, E, device="cuda")
  logits[:, 3] = -1e9                                        # expert 3 is never chosen
  w, idx, _ = moe.router_topk(logits, K, mode="softmax")
  assert moe.build_dispatch_plan(idx, E).row_align == 256
  w = w.detach().requires_grad_(True)
  y = moe.grouped_mlp(x, w, idx, wg, wu, wd)
  dy = torch.randn_like(y)
  y.backward(dy)
  xs, wgs, wus, wds, ws = (t.detach().float().requires_grad_(True) for t in (x, wg, wu, wd, w))
  yr = moe.grouped_mlp_reference(xs, ws, idx, wgs, wus, wds)
  yr.backward(dy.float())
  assert _rel(y, yr) < 2e-2 and _rel(x.grad, xs.grad) < 3e-2
  assert _rel(wd.grad, wds.grad) < 3e-2 and _rel(wg.grad, wgs.grad) < 3e-2 and _rel(wu.grad, wus.grad) < 3e-2
  assert float(wd.grad[3].abs().max()) == 0.0 and float(wg.grad[3].abs().max()) == 0.0
  _lib.raise_on_device_timeout()


@pytest.mark.parametrize("E,K,D,Fd,fused", [(4, 2, 128, 256, False), (8, 2, 256, 192, False), (4, 1, 128, 128, True)])
def test_grouped_mlp_forward_backward(cuda_lib, E, K, D, Fd, fused):
  torch.manual_seed(4)
  T = 300
  x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
  wg = (torch.randn(E, D, 2 * Fd if fused else Fd, device="cuda") / D ** 0.5).to(torch.bfloat16).requires_grad_(True)
  wu = (torch.randn(E, D, Fd, device="cuda") / D ** 0.5).to(torch.bfloat16).requires_grad_(True)
  wd = (torch.randn(E, Fd, D, device="cuda") / Fd ** 0.5).to(torch.bfloat16).requires_grad_(True)
  logits = torch.randn(T, E, device="cuda")
  w, idx, _ = moe.router_topk(logits, K, mode="softmax")
  w = w.detach().requires_grad_(True)
  y = moe.grouped_mlp(x, w, idx, wg, wu, wd, fused_gate_up=fused)
  dy = torch.randn_like(y)
  y.backward(dy)
  xs, wgs, wus, wds, ws = (t.detach().float().requires_grad_(True) for t in (x, wg, wu, wd, w))
  yr = moe.grouped_mlp_reference(xs, ws, idx, wgs, wus, wds, fused_gate_up=fused)
  yr.backward(dy.float())
  assert _rel(y, yr) < 2e-2
  assert _rel(x.grad, xs.grad) < 3e-2
  assert _rel(wd.grad, wds.grad) < 3e-2
  assert _rel(wg.grad, wgs.grad) < 3e-2
  if not fused:
    assert _rel(wu.grad, wus.grad) < 3e-2
  assert _rel(w.grad, ws.grad) < 3e-2


def test_grouped_mlp_empty_expert_and_capacity(cuda_lib):
  torch.manual_seed(5)
  T, K, E, D, Fd = 256, 2, 8, 128, 128
  x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
  wg, wu = (torch.randn(E, D, Fd, device="cuda").to(torch.bfloat16) * 0.05 for _ in range(2))
  wd = torch.randn(E, Fd, D, device="cuda").to(torch.bfloat16) * 0.05
  idx = torch.randint(0, 3, (T, K), device="cuda", dtype=torch.int32)   # experts 3..7 get nothing
  w = torch.rand(T, K, device="cuda")
  y = moe.grouped_mlp(x, w, idx, wg, wu, wd)
  assert _rel(y, moe.grouped_mlp_reference(x.float(), w, idx, wg.float(), wu.float(), wd.float())) < 2e-2
  yc = moe.grouped_mlp(x, w, idx, wg, wu, wd, capacity=40, rows_per_group=128)
  dropped = moe.build_dispatch_plan(idx, E, 40, 128).dest < 0
  assert dropped.any()
  yr = moe.grouped_mlp_reference(x.float(), w, idx, wg.float(), wu.float(), wd.float(), dropped=dropped)
  assert _rel(yc, yr) < 2e-2


@pytest.mark.parametrize("model,extra", [
  ("mixtral-tiny", ["model.hidden_size=128", "model.intermediate_size=256", "model.num_attention_heads=2",
                    "model.num_key_value_heads=1", "model.moe_implementation=gmm"]),
  ("mixtral-tiny", ["model.hidden_size=128", "model.intermediate_size=256", "model.num_attention_heads=2",
                    "model.num_key_value_heads=1", "model.moe_implementation=dropping"]),
  ("deepseek-tiny", ["model.hidden_size=128", "model.intermediate_size=256", "model.moe_intermediate_size=128",
                     "model.num_attention_heads=2", "model.num_key_value_heads=2", "model.qk_rope_head_dim=64",
                     "model.qk_nope_head_dim=128", "model.qk_head_dim=192", "model.v_head_dim=128",
                     "model.head_dim=64", "model.kv_lora_rank=64", "model.q_lora_rank=64"]),
])
def test_moe_models_train_on_gpu_and_match_torch_backend(cuda_lib, model, extra, tmp_path):
  """Three optimizer steps with the sm_100a kernels track the cuBLAS/eager backend."""
  from torchprime_b200.config import compose
  from torchprime_b200.data.synthetic import make_synthetic_dataset
  from torchprime_b200.models.model_utils import initialize_model_class
  from torchprime_b200.ops import functional as ops
  from torchprime_b200.trainer import Trainer
  losses = {}
  for backend in ("auto", "torch"):
    ops.set_backend(backend)
    try:
      cfg = compose("default", [f"model={model}", "dataset=synthetic", "dataset.block_size=256",
                                "task.global_batch_size=2", "task.max_steps=3", "task.optimizer.type=adamw",
                                "task.optimizer.learning_rate=1e-3", "ici_mesh.fsdp=1", "profile_start_step=-1",
                                f"output_dir={tmp_path}/{backend}"] + extra)
      m = initialize_model_class(cfg.model, device="meta")
      data = make_synthetic_dataset(vocab_size=cfg.model.vocab_size, block_size=256, num_samples=16)
      tr = Trainer(model=m, config=cfg, train_dataset=data)
      loader = tr._get_train_dataloader()
      out = []
      for _ in range(3):
        loss, gn = tr.train_step(tr._prepare_batch(loader.next_batch()))
        out.append((loss.item(), gn.item()))
      losses[backend] = out
    finally:
      ops.set_backend("auto")
  for (la, ga), (lb, gb) in zip(losses["auto"], losses["torch"]):
    assert abs(la - lb) < 0.05, losses
    assert abs(ga - gb) / max(gb, 1e-6) < 0.1, losses
