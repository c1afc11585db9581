"""Random sampling must not depend on the process, the batch or the scheduling mode.

* tensor-parallel ranks sample independently from identical logits: without a process-independent
  seed they would draw different tokens and their KV caches, stop conditions and collectives would
  diverge;
* a seeded request draws the same tokens alone, inside a batch, and with synchronous or asynchronous
  scheduling;
* speculative verification applies the request's constraints to the draft positions too.
"""
import json
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from vllm_ascend_b200.config import get_model_config
from vllm_ascend_b200.engine.llm import LLM
from vllm_ascend_b200.engine.request import SamplingParams

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    from vllm_ascend_b200.config import get_model_config
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    cfg = get_model_config("tiny-qwen")
    llm = LLM(cfg, device="cpu", tensor_parallel_size=2, max_model_len=128, max_num_seqs=4,
              max_num_batched_tokens=32, block_size=16)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, cfg.vocab_size, size=20).tolist() for _ in range(3)]
    outs = llm.generate(prompts, SamplingParams(temperature=1.0, top_k=50, max_tokens=8, ignore_eos=True))
    print("TOKENS " + json.dumps([o.outputs[0].token_ids for o in outs]), flush=True)
    llm.shutdown()
    sys.stdout.flush()
    os._exit(0)
""")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_tp2_unseeded_random_sampling_draws_identical_tokens_on_both_ranks():
    script = WORKER.format(root=ROOT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE="2",
               OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, "-c", script],
                              env=dict(env, RANK=str(r), LOCAL_RANK=str(r), PYTHONHASHSEED=str(11 + r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    toks = []
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-3000:]
        toks.append(json.loads([l for l in o.splitlines() if l.startswith("TOKENS ")][-1][7:]))
    assert toks[0] == toks[1]
    assert len({tuple(t) for t in toks[0]}) > 1          # really sampled, not a constant


def _llm(async_scheduling, **kw):
    return LLM(get_model_config("tiny-qwen"), device="cpu", max_model_len=128, max_num_seqs=8,
               max_num_batched_tokens=64, block_size=16, async_scheduling=async_scheduling, **kw)


def test_seeded_request_same_alone_in_batch_sync_and_async():
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, 1024, size=12 + 3 * i).tolist() for i in range(4)]
    sp = SamplingParams(temperature=1.0, top_p=0.95, seed=1234, max_tokens=10, ignore_eos=True)
    other = SamplingParams(temperature=0.8, seed=7, max_tokens=10, ignore_eos=True)
    results = []
    for async_sched in (False, True):
        llm = _llm(async_sched)
        alone = llm.generate([prompts[0]], sp)[0].outputs[0].token_ids
        batch = llm.generate([prompts[1], prompts[2], prompts[0], prompts[3]], [other, other, sp, other])
        assert batch[2].outputs[0].token_ids == alone
        results.append(alone)
    assert results[0] == results[1]
    # consecutive tokens use consecutive stream positions (no position is used twice)
    assert len(set(results[0])) > 1


def test_min_tokens_ban_lifts_on_time_with_async_scheduling():
    prompt = list(range(1, 17))
    lens = []
    for async_sched in (False, True):
        llm = _llm(async_sched)
        llm.engine.eos_token_id = None
        # every token is a stop token: generation must continue exactly until min_tokens is reached
        sp = SamplingParams(temperature=0.0, max_tokens=12, min_tokens=5,
                            stop_token_ids=list(range(1024)))
        out = llm.generate([prompt], sp)[0].outputs[0].token_ids
        lens.append(len(out))
    assert lens[0] == lens[1] and lens[0] in (5, 6), lens


def test_speculative_verification_respects_allowed_token_ids():
    allowed = list(range(100, 140))
    llm = _llm(False, speculative_config={"method": "ngram", "num_speculative_tokens": 3,
                                          "prompt_lookup_max": 3, "prompt_lookup_min": 1})
    rng = np.random.default_rng(9)
    base = rng.integers(100, 140, size=6).tolist()
    prompts = [base * 4, (base[::-1]) * 4]
    for temp in (0.0, 1.0):
        sp = SamplingParams(temperature=temp, seed=3, max_tokens=16, ignore_eos=True, allowed_token_ids=allowed,
                            bad_words_token_ids=[[base[0]]])
        for o in llm.generate(prompts, sp):
            toks = o.outputs[0].token_ids
            assert len(toks) == 16
            assert all(100 <= t < 140 for t in toks), toks
            assert base[0] not in toks
    assert llm.engine.runner.spec_stats["draft_tokens"] > 0


def test_malformed_sampling_parameters_are_rejected_up_front():
    llm = _llm(False)
    with pytest.raises(ValueError):
        SamplingParams(repetition_penalty=0.0)
    with pytest.raises(ValueError):
        SamplingParams(min_p=1.5)
    with pytest.raises(ValueError):
        SamplingParams(allowed_token_ids=[-1, 3])
    with pytest.raises(ValueError):
        llm.generate([[1, 2, 3]], SamplingParams(allowed_token_ids=[5, 1024], max_tokens=2))
    # the engine is still usable afterwards
    out = llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, allowed_token_ids=[5, 6], max_tokens=3))
    assert set(out[0].outputs[0].token_ids) <= {5, 6}
