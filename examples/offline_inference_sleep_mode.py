"""Sleep / wake-up around an external weight update (RL rollout workers).

Level 1 moves the weights to pinned host memory and drops the KV cache; level 2 drops both, the
weights are then re-sent by the trainer (``B200Worker.update_weights`` / the weight-transfer engines).
"""
import torch

from vllm_ascend_b200 import LLM, SamplingParams

llm = LLM("qwen3-8b", enable_sleep_mode=True, max_model_len=2048)
sp = SamplingParams(temperature=0.0, max_tokens=8)
before = llm.generate([[1, 2, 3, 4]], sp)[0].outputs[0].token_ids
free0 = torch.cuda.mem_get_info()[0]
llm.sleep(level=1)
print(f"asleep: {(torch.cuda.mem_get_info()[0] - free0) / 2**30:.1f} GiB returned to the device")
llm.wake_up()
assert llm.generate([[1, 2, 3, 4]], sp)[0].outputs[0].token_ids == before
print("weights restored, same tokens")
