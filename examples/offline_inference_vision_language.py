"""Vision-language generation (Qwen2.5-VL style): one placeholder token per image in the prompt,
pixels as an array; the engine patchifies, runs the vision tower and merges the embeddings.

    python examples/offline_inference_vision_language.py [checkpoint-dir]
"""
import sys

import numpy as np

from vllm_ascend_b200 import LLM, SamplingParams
from vllm_ascend_b200.config import get_model_config

model = sys.argv[1] if len(sys.argv) > 1 else "tiny-vl"
cfg = get_model_config(model)
llm = LLM(cfg, max_model_len=4096)
image = (np.random.default_rng(0).random((224, 336, 3)) * 255).astype(np.uint8)
prompt = [1, 2, 3, cfg.image_token_id, 4, 5, 6]
out = llm.generate([{"prompt_token_ids": prompt, "multi_modal_data": {"image": [image]}}],
                   SamplingParams(temperature=0.0, max_tokens=16))[0]
print(len(out.prompt_token_ids), "prompt tokens after placeholder expansion ->", out.outputs[0].token_ids)
