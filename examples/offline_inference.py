"""Offline generation on one GPU.

    python examples/offline_inference.py [preset-or-checkpoint-dir]

A preset name (``qwen3-8b``, ``tiny-qwen`` ...) builds random weights of that architecture; a
directory is read as an HF safetensors checkpoint.  Prompts are token ids: the framework ships no
tokenizer of its own (pass ids from ``transformers.AutoTokenizer`` when a checkpoint has one).
"""
import sys

from vllm_ascend_b200 import LLM, SamplingParams

model = sys.argv[1] if len(sys.argv) > 1 else "qwen3-8b"
llm = LLM(model, max_model_len=4096, enable_prefix_caching=True)
prompts = [[1, 2, 3, 4, 5, 6, 7, 8], [11, 12, 13], list(range(100, 164))]
params = SamplingParams(temperature=0.8, top_p=0.95, max_tokens=32, seed=0)
for out in llm.generate(prompts, params):
    print(out.request_id, out.outputs[0].token_ids, out.outputs[0].finish_reason)
