"""Child process of the 2-GPU disaggregated-prefill test.

``prefill <dir>``: engine on cuda:0, prefills the prompts with do_remote_decode, writes the
returned kv_transfer_params to <dir>/params.json and keeps serving the side channel until
<dir>/stop appears.  ``decode <dir>``: engine on cuda:1, pulls the KV over CUDA IPC and
decodes; prints the tokens next to a monolithic run on the same GPU."""
import json
import os
import sys
import time

import numpy as np
import torch

from vllm_ascend_b200.config import ModelConfig
from vllm_ascend_b200.engine.llm import LLM
from vllm_ascend_b200.engine.request import SamplingParams


def _cfg():
    return ModelConfig(name="t", architecture="Qwen3ForCausalLM", vocab_size=2048, hidden_size=512,
                       intermediate_size=1024, num_hidden_layers=3, num_attention_heads=8,
                       num_key_value_heads=2, head_dim=128, qk_norm=True, rope_theta=1e6,
                       dtype="bfloat16", init_std=0.05)


def _prompts():
    rng = np.random.default_rng(7)
    return [rng.integers(0, 2048, size=n).tolist() for n in (150, 40, 333, 129, 257)]


def _llm(role, engine_id, port=0, dev=0):
    ktc = None if role is None else {"kv_connector": "NVLinkConnector", "kv_role": role,
                                     "engine_id": engine_id, "kv_port": port}
    return LLM(_cfg(), device=f"cuda:{dev}", seed=0, max_model_len=512, max_num_seqs=8,
               max_num_batched_tokens=256, num_gpu_blocks_override=40, enforce_eager=True,
               kv_transfer_config=ktc)


def run_recording(llm, prompts, sp):
    """generate() that also returns, per prompt, the KV rows of its first len-1 tokens (every layer,
    K and V) as they sit in the paged cache when the request finishes prefill."""
    eng = llm.engine
    rids = [eng.add_request(p["prompt_token_ids"], sp, kv_transfer_params=p.get("kv_transfer_params"))
            for p in prompts]
    reqs = {r: eng.scheduler.requests[r] for r in rids}
    blocks = {r: [] for r in rids}
    while eng.has_unfinished():
        eng.step()
        for r, q in reqs.items():
            if len(q.block_ids) > len(blocks[r]):
                blocks[r] = list(q.block_ids)
    rows = [kv_rows(llm, blocks[r], reqs[r].num_prompt_tokens - 1) for r in rids]
    return [list(reqs[r].output_token_ids or []) for r in rids], rows, reqs


def kv_rows(llm, block_ids, n):
    """[2 * layers, n, H, D]: the first n token rows of a sequence's K and V in every layer."""
    torch.cuda.synchronize()
    runner = llm.engine.runner
    idx = torch.tensor(list(block_ids), device=runner.device, dtype=torch.long)
    per_layer = []
    for pair in runner.kv_caches:
        for c in pair:
            g = c[idx]                                     # [nb, bs, H, D] logical
            per_layer.append(g.reshape(-1, *g.shape[2:])[:n].float().cpu())
    return torch.stack(per_layer)


def kv_equal(a, b) -> bool:
    return all(x.shape == y.shape and torch.equal(x, y) for x, y in zip(a, b))


def prefill(d):
    torch.cuda.set_device(0)
    llm = _llm("kv_producer", "P", int(os.environ.get("KV_PORT", "0")))
    sp1 = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
    outs = llm.generate([{"prompt_token_ids": p, "kv_transfer_params": {"do_remote_decode": True}}
                         for p in _prompts()], sp1)
    tmp = os.path.join(d, "params.tmp")
    with open(tmp, "w") as f:
        json.dump([o.kv_transfer_params for o in outs], f)
    os.replace(tmp, os.path.join(d, "params.json"))
    c = llm.engine.kv_connector
    t0 = time.time()
    while not os.path.exists(os.path.join(d, "stop")) and time.time() - t0 < 120:
        c.reap(llm.engine.scheduler)
        time.sleep(0.05)
    c.reap(llm.engine.scheduler)
    print("RESULT " + json.dumps({"released": c.stats["released"], "delayed": c.num_delayed,
                                  "first": [o.outputs[0].token_ids[0] for o in outs]}), flush=True)
    c.close()


def decode(d):
    dev = 1 if torch.cuda.device_count() > 1 else 0
    torch.cuda.set_device(dev)
    sp = SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True)
    mono = _llm(None, "M", dev=dev)
    want, want_kv, _ = run_recording(mono, [{"prompt_token_ids": p} for p in _prompts()], sp)
    del mono
    llm = _llm("kv_consumer", "D", dev=dev)
    path = os.path.join(d, "params.json")
    t0 = time.time()
    while not os.path.exists(path):
        if time.time() - t0 > 120:
            raise TimeoutError("prefill process never wrote its parameters")
        time.sleep(0.05)
    params = json.load(open(path))
    got, got_kv, _ = run_recording(llm, [{"prompt_token_ids": p, "kv_transfer_params": k}
                                         for p, k in zip(_prompts(), params)], sp)
    c = llm.engine.kv_connector
    modes = sorted({"ipc" if m.get("_base") else "other" for m in c._remote_meta.values()})
    res = {"want": want, "got": got, "kv_equal": kv_equal(got_kv, want_kv), "stats": c.stats, "modes": modes,
           "prefill_tokens": int(llm.engine.runner.stats.get("num_prefill_tokens", -1))}
    c.close()
    time.sleep(0.3)          # let the done messages leave before the producer is told to stop
    open(os.path.join(d, "stop"), "w").close()
    print("RESULT " + json.dumps(res), flush=True)


if __name__ == "__main__":
    {"prefill": prefill, "decode": decode}[sys.argv[1]](sys.argv[2])
