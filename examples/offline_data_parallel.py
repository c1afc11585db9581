"""Data-parallel replicas (attention DP) under torchrun: every rank serves every world-th prompt and
the replicas advance in lock-step; with a MoE preset and ``ep`` the experts are sharded over the
replicas and tokens travel through the fused dispatch / combine kernels.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/offline_data_parallel.py qwen3-30b-a3b ep
"""
import os
import sys

from vllm_ascend_b200 import LLM, SamplingParams

model = sys.argv[1] if len(sys.argv) > 1 else "qwen3-8b"
ep = len(sys.argv) > 2 and sys.argv[2] == "ep"
llm = LLM(model, tensor_parallel_size=1, enable_expert_parallel=ep, max_model_len=4096)
prompts = [[i + 1] * (8 + i) for i in range(16)]
outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16))
print(f"rank {os.environ.get('RANK', '0')}: served {len(outs)} prompts")
llm.shutdown()
