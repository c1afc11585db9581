"""Chunk-size predictor and the scheduler that sizes prefill chunks for equal step latency."""
import numpy as np
import pytest

from vllm_ascend_b200.config import CacheConfig, SchedulerConfig
from vllm_ascend_b200.core.profiling_chunk import ChunkSizePredictor, ProfilingChunkScheduler
from vllm_ascend_b200.engine.request import Request, SamplingParams
from vllm_ascend_b200.platform_config import clear_b200_config, init_b200_config

A, B, C, D = 2e-9, 3e-6, 1e-7, 4e-4          # a synthetic device: seconds


def truth(chunk, hist):
    return A * chunk * (chunk + hist) + B * chunk + C * hist + D


@pytest.fixture(autouse=True)
def _clean():
    yield
    clear_b200_config()


def test_predictor_not_ready_then_fits_and_solves_for_the_chunk():
    p = ChunkSizePredictor(smooth_factor=1.0, min_chunk=64)
    assert p.predict(0, 4096) == 4096 and not p.fitted                  # no model: the full budget
    rng = np.random.default_rng(0)
    for _ in range(30):
        c, h = int(rng.integers(64, 4096)), int(rng.integers(0, 30000))
        p.observe(c, h, truth(c, h))
    assert p.fitted
    assert p.a == pytest.approx(A, rel=1e-3) and p.b == pytest.approx(B, rel=1e-2)
    assert p.c == pytest.approx(C, rel=1e-2) and p.d == pytest.approx(D, rel=1e-2)
    p.set_target(4096)
    assert p.target_latency == pytest.approx(truth(4096, 0), rel=1e-3)
    # without history the chunk that meets the target is the base chunk; with history chunks shrink
    sizes = [p.predict(h, 4096) for h in (0, 8192, 32768, 131072)]
    assert abs(sizes[0] - 4096) <= 2 and sizes == sorted(sizes, reverse=True) and sizes[-1] < sizes[0] // 2
    for h, c in zip((8192, 32768), sizes[1:3]):
        assert truth(c, h) == pytest.approx(p.target_latency, rel=2e-2)  # equal-latency chunks
    # history so long that its own term exceeds the target: the floor
    assert p.predict(10 ** 9, 4096) == 64


def test_predictor_batch_samples_smoothing_and_degenerate_fits():
    p = ChunkSizePredictor(smooth_factor=0.5, min_chunk=16)
    rng = np.random.default_rng(1)
    for _ in range(20):
        batch = [(int(rng.integers(1, 512)), int(rng.integers(0, 4000))) for _ in range(int(rng.integers(1, 5)))]
        p.observe_batch(batch, sum(truth(c, h) - D for c, h in batch) + D)
    assert p.fitted and p.a == pytest.approx(A, rel=1e-2)
    p.set_target(512)
    first = p.predict(0, 512)
    second = p.predict(20000, 512)                                        # smoothed towards the last answer
    raw = ChunkSizePredictor(smooth_factor=1.0, min_chunk=16)
    raw.samples, raw.target_latency = list(p.samples), p.target_latency
    raw.fit()
    assert raw.predict(20000, 512) < second < first
    # latencies that fall with size: refused, the old state stays
    bad = ChunkSizePredictor()
    for c in (100, 200, 300, 400, 500, 600):
        bad.observe(c, 0, 1.0 / c)
    assert not bad.fitted and bad.predict(0, 2048) == 2048


def _sched(budget=256, **cfg):
    init_b200_config({"scheduler_config": {"profiling_chunk_config": dict({"enabled": True, "min_chunk": 16}, **cfg)}},
                     refresh=True)
    sc = SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=budget, max_model_len=4096)
    return ProfilingChunkScheduler(sc, CacheConfig(block_size=16), 512)


def test_start_up_profiling_runs_once_skips_failures_and_sets_the_target():
    s = _sched()
    calls = []

    def fn(n):
        calls.append(n)
        if n == 240:
            raise RuntimeError("boom")
        return truth(n, 0) * (5 if len(calls) == 1 else 1)                # the first call is a slow warm-up
    assert s.run_profiling(fn)
    assert calls[0] == calls[1] == 256 and calls[-1] == 16 and len(calls) == 17
    assert s.predictor.fitted and s.predictor.target_latency == pytest.approx(truth(256, 0), rel=1e-2)
    n = len(calls)
    assert s.run_profiling(fn) and len(calls) == n                        # second call: nothing runs
    none = _sched()
    assert not none.run_profiling(None) and not none.predictor.fitted
    failing = _sched()
    assert not failing.run_profiling(lambda n: (_ for _ in ()).throw(RuntimeError("x"))) and not failing.predictor.fitted


def test_scheduler_shrinks_chunks_of_a_long_prompt_and_learns_online():
    s = _sched(budget=256)
    s.predictor.smooth = 1.0
    big = 40
    s.run_profiling(lambda n: A * big * n * n + B * n + D)               # strongly quadratic device
    r = Request(request_id="long", prompt_token_ids=list(range(1, 2001)),
                sampling_params=SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))
    s.add_request(r)
    sizes = []
    for _ in range(6):
        out = s.schedule()
        (req, n), = out.scheduled
        sizes.append(n)
        s.update_from_output(out, {})
        s.record_step(out, A * big * n * (n + req.num_computed_tokens - n) + B * n + D)
    assert sizes[0] == 256 and sizes == sorted(sizes, reverse=True) and sizes[-1] < sizes[0]
    assert s.cfg.max_num_batched_tokens == 256                           # the budget override does not leak
    assert len(s.predictor.samples) == 16 + 6
    # decode-only steps are not samples
    before = len(s.predictor.samples)
    fake = type("O", (), {"scheduled": [(r, 1)]})()
    s.record_step(fake, 0.001)
    assert len(s.predictor.samples) == before


def test_engine_profiles_at_start_and_tokens_equal_fcfs():
    from vllm_ascend_b200.engine.llm import LLM
    rng = np.random.default_rng(7)
    prompts = [rng.integers(1, 400, size=n).tolist() for n in (90, 20, 64)]
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=64)
    want = [o.outputs[0].token_ids for o in LLM("tiny-qwen", **kw).generate(prompts, sp)]
    llm = LLM("tiny-qwen", additional_config={"scheduler_config": {"profiling_chunk_config": {
        "enabled": True, "min_chunk": 8}}}, **kw)
    s = llm.engine.scheduler
    assert isinstance(s, ProfilingChunkScheduler) and s.profiled and len(s.predictor.samples) >= 8
    n0 = len(s.predictor.samples)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == want and len(s.predictor.samples) > n0                 # online samples arrived
