"""The benchmark script's workloads on CPU ranks (tiny model): fixed-concurrency serving through
``LLM.generate(max_concurrency=...)`` and the disaggregated prefill -> decode mode, where two
engines in one launch hand KV blocks over through the connector."""
import json
import os
import socket
import subprocess
import sys

import numpy as np

from vllm_ascend_b200.config import get_model_config
from vllm_ascend_b200.engine.llm import LLM
from vllm_ascend_b200.engine.request import SamplingParams

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_generate_with_max_concurrency_keeps_the_limit_and_the_tokens():
    llm = LLM(get_model_config("tiny-qwen"), device="cpu", max_model_len=128, max_num_seqs=8,
              max_num_batched_tokens=64, block_size=16)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 1024, size=10 + i).tolist() for i in range(9)]
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    eng = llm.engine
    seen = []
    orig = eng.step

    def counting_step():
        seen.append(eng.scheduler.num_unfinished)
        return orig()
    eng.step = counting_step
    got = llm.generate(prompts, sp, max_concurrency=3)
    assert [o.outputs[0].token_ids for o in got] == want          # input order, same tokens
    assert max(seen) <= 3 and max(seen) == 3
    # admission time is the arrival time: later requests arrive later
    arr = [o.metrics.arrival_time for o in got]
    assert arr[-1] > arr[0]


def test_bench_pd_mode_hands_kv_blocks_from_the_prefill_to_the_decode_engine():
    port = _free_port()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "bench.py"),
           "--gpus", "2", "--mode", "pd", "--model", "tiny-qwen", "--num-prompts", "12", "--input-len", "24",
           "--output-len", "6", "--concurrency", "4", "--steps", "1", "--warmup", "1", "--max-num-seqs", "8",
           "--max-num-batched-tokens", "64"]
    env = dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-3000:]
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith('{"metric"')][-1])
    assert line["config"]["mode"] == "pd" and line["n_gpus"] == 2
    assert line["config"]["kv_blocks_pulled"] > 0 and line["config"]["kv_pull_failures"] == 0
    assert line["value"] > 0 and line["p50_ttft_s"] is not None
