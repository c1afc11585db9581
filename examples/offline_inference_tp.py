"""Tensor-parallel (or expert-parallel) offline generation, one process per GPU.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/offline_inference_tp.py
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/offline_inference_tp.py qwen3-30b-a3b ep

Every rank builds the same engine and calls generate() with the same prompts; rank 0 prints.
VLLM_B200_TP_COMM=fused (default) runs the linear layers' collectives inside the GEMM kernels over
peer memory, VLLM_B200_TP_COMM=nccl uses NCCL all-reduce.
"""
import os
import sys

from vllm_ascend_b200 import LLM, SamplingParams

model = sys.argv[1] if len(sys.argv) > 1 else "qwen3-8b"
ep = len(sys.argv) > 2 and sys.argv[2] == "ep"
world = int(os.environ.get("WORLD_SIZE", "1"))
llm = LLM(model, tensor_parallel_size=1 if ep else world, enable_expert_parallel=ep, max_model_len=4096)
outs = llm.generate([[1, 2, 3, 4, 5, 6, 7, 8]] * 4, SamplingParams(temperature=0.0, max_tokens=16))
if int(os.environ.get("RANK", "0")) == 0:
    for o in outs:
        print(o.outputs[0].token_ids)
llm.shutdown()
