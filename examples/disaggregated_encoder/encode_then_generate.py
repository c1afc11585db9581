"""Disaggregated vision encoder (E | PD): an encoder instance runs the vision tower and publishes
the outputs by content hash; the serving instance receives hashes instead of pixels.

Both instances run in this one process for the demonstration; in a deployment they are separate
processes (or nodes) that share only the store address.
"""
import numpy as np

from vllm_ascend_b200 import LLM, SamplingParams
from vllm_ascend_b200.config import get_model_config
from vllm_ascend_b200.distributed.kv_transfer.kv_pool import KVStoreServer

store = KVStoreServer()                                  # in-memory store; share its port with both sides
ec = lambda role: {"ec_connector": "ECStoreConnector", "ec_role": role,                      # noqa: E731
                   "ec_connector_extra_config": {"store_port": store.port}}
cfg = get_model_config("tiny-vl")
encoder = LLM(cfg, ec_transfer_config=ec("ec_producer"), max_model_len=1024)
server = LLM(cfg, ec_transfer_config=ec("ec_consumer"), max_model_len=1024)

image = (np.random.default_rng(0).random((112, 112, 3)) * 255).astype(np.uint8)
descriptors = encoder.encode_multimodal({"image": [image]})
prompt = [1, 2, cfg.image_token_id, 3]
out = server.generate([{"prompt_token_ids": prompt,
                        "multi_modal_data": {"image": [{"hash": d["hash"], "grid_thw": d["grid_thw"]}
                                                       for d in descriptors]}}],
                      SamplingParams(temperature=0.0, max_tokens=8))[0]
print(out.outputs[0].token_ids, server.engine.runner.mm.stats)
store.close()
