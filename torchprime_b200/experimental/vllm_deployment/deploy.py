"""Load a checkpoint exported by this framework with vLLM and generate a few tokens.

  python torchprime_b200/experimental/vllm_deployment/deploy.py --model-dir outputs/export --prompt "1 + 1 ="

Shows that ``model.export()`` / ``task.convert_to_safetensors`` write a directory any HF-compatible
runtime can serve (sharded safetensors + index + config and tokenizer files), as the reference does
with experimental/vllm_tpu_deployment/deploy.py:1-42.
"""

from __future__ import annotations

import argparse


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--model-dir", required=True)
  ap.add_argument("--prompt", default="The capital of France is")
  ap.add_argument("--max-tokens", type=int, default=32)
  ap.add_argument("--tensor-parallel-size", type=int, default=1)
  a = ap.parse_args(argv)
  from vllm import LLM, SamplingParams
  llm = LLM(model=a.model_dir, tensor_parallel_size=a.tensor_parallel_size, dtype="bfloat16")
  out = llm.generate([a.prompt], SamplingParams(temperature=0.0, max_tokens=a.max_tokens))
  print(out[0].outputs[0].text)


if __name__ == "__main__":
  main()
