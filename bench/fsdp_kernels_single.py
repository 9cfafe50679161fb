"""Single-GPU run of the kernels behind the peer-memory FSDP collectives, for profiling one launch of each
(world = 1: the only staging slot and the only shard are this GPU's own, every flag is already set):

  python bench/fsdp_kernels_single.py            # 3 launches each: ag-wait GEMM, rs-store GEMM, slot reduction

Shapes: one Llama-3-8B projection with 4096 tokens (operands and outputs together about 300 MB, beyond L2).
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
  from torchprime_b200.ops import _lib, kernels as k
  from torchprime_b200.ops._lib import check, lib, ptr, stream_ptr
  from torchprime_b200.parallel import fsdp_comm  # noqa: F401  (registers the C signatures)
  import ctypes
  dev = torch.device("cuda", 0)
  torch.manual_seed(0)
  T, N, K = 4096, 14336, 4096
  L = lib()
  x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
  w = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)          # the "gathered buffer" is the weight itself
  flags = torch.ones(1, dtype=torch.int32, device=dev)
  y = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
  dy = torch.randn(T, N, device=dev, dtype=torch.bfloat16)
  stage = torch.empty(N * K, device=dev, dtype=torch.bfloat16)
  table = (ctypes.c_void_p * 1)(stage.data_ptr())
  red = torch.empty(N * K, device=dev, dtype=torch.bfloat16)
  for _ in range(3):
    check(L.tpb_gemm_ag_wait_bf16(ptr(x), ptr(y), T, N, K, K, N, _lib.EPI_BF16, None, 0, None, 0, w.data_ptr(), 0, 1,
                                  N * K, N * K, flags.data_ptr(), 1, stream_ptr()), "gemm_ag_wait")
    check(L.tpb_gemm_rs_store_bf16(ptr(dy), ptr(x), N, K, T, N, K, K, 1, 1, 1.0, table, 1, N * K, 0, 0, stream_ptr()),
          "gemm_rs_store")
    check(L.tpb_rs_reduce_bf16(stage.data_ptr(), 1, N * K, N * K, red.data_ptr(), 0, 0, 1.0, stream_ptr()), "reduce")
  torch.cuda.synchronize()
  want_y = x.float() @ w.float().t()
  want_dw = dy.float().t() @ x.float()
  e1 = ((y.float() - want_y).norm() / want_y.norm()).item()
  e2 = ((red.view(N, K).float() - want_dw).norm() / want_dw.norm()).item()
  _lib.raise_on_device_timeout()
  assert e1 < 1e-2 and e2 < 1e-2, (e1, e2)
  print(f"ok: ag-wait GEMM rel err {e1:.2e}, rs-store GEMM + reduction rel err {e2:.2e}")


if __name__ == "__main__":
  main()
