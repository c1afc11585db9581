"""Batch-job-aware scheduler: job names, the decode-length estimator, the block reserve, the
length buckets, the job queue's ordering rules, and a whole engine run on the policy."""
from types import SimpleNamespace as NS

import numpy as np
import pytest

from vllm_ascend_b200.config import CacheConfig, SchedulerConfig
from vllm_ascend_b200.core.batch_job_aware import (BatchJobAwareScheduler, BlockReserve, JobDecodeEstimator,
                                                   JobNameParser, LengthBuckets)
from vllm_ascend_b200.engine.request import Request, RequestStatus, SamplingParams
from vllm_ascend_b200.platform_config import clear_b200_config, init_b200_config


def _req(rid, n_prompt, job=None, max_tokens=16):
    return Request(request_id=rid, prompt_token_ids=list(range(1, n_prompt + 1)),
                   sampling_params=SamplingParams(max_tokens=max_tokens, temperature=0.0, ignore_eos=True),
                   job_id=job)


def _sched(num_blocks=64, **cfg):
    init_b200_config({"scheduler_config": {"batch_job_sched_config": dict({"enabled": True}, **cfg)}}, refresh=True)
    sc = SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=64, max_model_len=512, reserve_full_sequence=False)
    return BatchJobAwareScheduler(sc, CacheConfig(block_size=16), num_blocks)


@pytest.fixture(autouse=True)
def _clean():
    yield
    clear_b200_config()


# ---------------------------------------------------------------- job names
def test_job_name_parser():
    p = JobNameParser()
    assert p.parse("cmpl-#job_name[summaries]#-17") == "summaries"
    assert p.parse("cmpl-17") == "_default"
    assert p.parse("x#job_name[]#y") == "_default"
    assert len(p) == 3
    assert p.parse("cmpl-17") == "_default" and len(p) == 3          # cached, not re-added
    p.remove("cmpl-17")
    p.remove("never-seen")                                           # no error
    assert len(p) == 2
    p.clear()
    assert len(p) == 0
    # an explicit job id on the request wins over the tag
    assert p.parse(_req("a#job_name[x]#", 4, job="explicit")) == "explicit"


# ---------------------------------------------------------------- estimator
def test_estimator_cold_start_ewma_and_limits():
    e = JobDecodeEstimator(max_jobs=2, max_samples=4)
    assert e.predict("a") == 128 and e.get_stats() == {}
    e.observe("a", 200)
    assert e.predict("a") == 200                                     # first sample is taken as is
    e.observe("a", 100)
    assert e.predict("a") == int(0.1 * 100 + 0.9 * 200)
    e.observe("b", 10)
    assert e.predict("b") == 10 and e.predict("a") == 190            # independent jobs
    with pytest.raises(RuntimeError, match="max_jobs=2"):
        e.observe("c", 5)
    e.observe("a", 100)
    e.observe("a", 100)
    frozen = e.predict("a")
    e.observe("a", 100000)                                           # fifth sample: ignored
    assert e.predict("a") == frozen and e.samples("a") == 4
    st = e.get_stats()
    assert st["a"]["samples"] == 4 and st["b"]["predicted_decode"] == 10
    unlimited = JobDecodeEstimator(max_jobs=0, max_samples=0)
    for i in range(50):
        unlimited.observe(f"j{i}", i)
    for _ in range(200):
        unlimited.observe("j0", 50)
    assert 45 <= unlimited.predict("j0") <= 50                       # converges


# ---------------------------------------------------------------- reserve
def test_block_reserve_per_request_cases():
    fake = NS(block_size=16, spec_slack=0, cfg=NS(max_num_batched_tokens=64), running=[])
    r = BlockReserve(fake, margin_blocks=0, max_blocks=0)

    def rq(done, prompt):
        return NS(num_computed_tokens=done, num_prompt_tokens=prompt)
    # prefill, 200-token prompt, nothing computed: this step takes 64, the next another 64 -> 4 new blocks
    assert r.one(rq(0, 200)) == 4
    # prefill ends this step (after = 100, 4 slots free in block 7); next step decodes one token: no new block
    assert r.one(rq(64, 100)) == 0
    # decode in the middle of a block
    assert r.one(rq(105, 100)) == 0
    # decode that fills its block this step: the next token needs a new block
    assert r.one(rq(111, 100)) == 1
    # speculative tokens count
    fake.spec_slack = 3
    assert r.one(rq(108, 100)) == 1        # after = 112 (boundary), next step 4 tokens -> 1 block
    assert r.one(rq(104, 100)) == 0        # after = 108, 4 free slots, 4 tokens


def test_block_reserve_cache_margin_and_cap():
    fake = NS(block_size=16, spec_slack=0, cfg=NS(max_num_batched_tokens=64), running=[])
    r = BlockReserve(fake, margin_blocks=2, max_blocks=5)
    calls = []
    one = r.one
    r.one = lambda q: (calls.append(q), one(q))[1]
    assert r.predict() == 2                                           # empty running set: the margin
    a, b = NS(num_computed_tokens=111, num_prompt_tokens=100), NS(num_computed_tokens=15, num_prompt_tokens=10)
    fake.running = [a]
    assert r.predict() == 3 and calls == [a]                          # grew by one: only the new request
    assert r.predict() == 3 and calls == [a]                          # unchanged: cached
    fake.running = [a, b]
    assert r.predict() == 4 and calls == [a, b]
    fake.running = [b]                                                # anything else: recomputed
    assert r.predict() == 3 and calls == [a, b, b]
    r.invalidate()
    assert r.predict() == 3 and calls == [a, b, b, b]
    fake.running = [a] * 10
    assert r.predict() == 5                                           # capped


# ---------------------------------------------------------------- buckets
def test_length_buckets_best_fit():
    b = LengthBuckets()
    assert not b and len(b) == 0 and b.peek_best_fit(100) is None and b.peek_shortest() is None
    b.put(None)
    rs = {n: _req(f"r{n}", n) for n in (10, 40, 40, 100)}
    twin = _req("r40b", 40)
    for r in list(rs.values()) + [twin]:
        b.put(r)
    b.put(twin)                                                       # twice: still one entry
    assert len(b) == 4 and bool(b)
    assert b.peek_best_fit(100) is rs[100]
    assert b.peek_best_fit(99) is rs[40]                              # nearest below, oldest of that length
    assert b.peek_best_fit(9) is None
    assert b.peek_shortest() is rs[10]
    assert [r.request_id for r in b] == ["r10", "r40", "r40b", "r100"]
    assert b.remove(rs[40]) and b.peek_best_fit(50) is twin
    assert not b.remove(rs[40]) and not b.remove(None) and not b.remove(_req("zz", 7))
    assert b.remove(twin) and b.peek_best_fit(50) is rs[10]           # the empty length is gone
    assert b.remove(rs[10]) and b.remove(rs[100]) and not b


# ---------------------------------------------------------------- queue ordering
def test_queue_cold_start_then_job_order_by_free_space():
    s = _sched(num_blocks=1024, cold_start_requests=1, low_available_tokens_threshold=4096,
               short_decode_token_threshold=32, reserve_margin_blocks=0)
    q = s.waiting
    s.estimator.observe("long", 300)
    s.estimator.observe("mid", 100)
    s.estimator.observe("short", 8)
    first = {}
    for job in ("short", "long", "mid"):
        for i, n in enumerate((30, 50, 20)):
            r = _req(f"{job}-{i}", n, job=job)
            first.setdefault(job, r)
            s.add_request(r)
    assert len(q) == 9 and len(list(q)) == 9
    # the first request of every job goes ahead of any ordering
    for job in ("short", "long", "mid"):
        head = q.peek()
        assert head is first[job]
        q.remove(head)
    # plenty of space (1023 blocks * 16 tokens): long decodes first, longest prompt that fits first
    assert q.admission_budget() > 4096
    assert q.peek().request_id == "long-1"
    long_, short = q.classify_jobs()
    assert sorted(long_) == [("long", 300), ("mid", 100)] and short == [("short", 8)]
    assert [j for j, _ in q.sort_jobs(10000, long_, short)] == ["long", "mid", "short"]
    # scarce space: short decodes first
    assert [j for j, _ in q.sort_jobs(100, long_, short)] == ["short", "long", "mid"]
    # only one class present: descending when space is plentiful, ascending when scarce
    assert [j for j, _ in q.sort_jobs(10000, long_, [])] == ["long", "mid"]
    assert [j for j, _ in q.sort_jobs(100, long_, [])] == ["mid", "long"]
    two_short = [("s1", 5), ("s2", 20)]
    assert [j for j, _ in q.sort_jobs(10000, [], two_short)] == ["s2", "s1"]
    assert [j for j, _ in q.sort_jobs(100, [], two_short)] == ["s1", "s2"]


def test_queue_budget_and_preempted_requests():
    s = _sched(num_blocks=9, cold_start_requests=0, reserve_margin_blocks=2)      # 8 usable blocks
    q = s.waiting
    for n in (200, 90, 40):
        s.add_request(_req(f"r{n}", n, job="j"))
    # idle engine: budget (8 - 2) * 16 = 96 tokens -> the 90-token prompt is the best fit
    assert q.admission_budget() == 96
    assert q.peek().request_id == "r90"
    # something is running and the pool is exhausted: nothing is admittable, but the queue is not empty
    s.running.append(_req("busy", 10))
    taken = s.pool.allocate(s.pool.num_free_blocks)
    assert q.admission_budget() == 0 and q.peek() is None and bool(q) and len(q) == 3
    # a preempted request is served first whatever the budget
    pre = _req("pre", 500, job="j")
    pre.status = RequestStatus.PREEMPTED
    q.appendleft(pre)
    assert q.peek() is pre and q[0] is pre and pre in q
    assert q.popleft() is pre and pre not in q
    s.pool.free(taken)
    s.running.clear()
    with pytest.raises(ValueError):
        q.remove(_req("ghost", 3, job="j"))
    # too many jobs
    s2 = _sched(max_jobs=1)
    s2.add_request(_req("a", 5, job="one"))
    with pytest.raises(RuntimeError, match="max_jobs=1"):
        s2.add_request(_req("b", 5, job="two"))


def test_config_validation():
    from vllm_ascend_b200.platform_config import _validate_scheduler_ext, get_b200_config
    engine_cfg = NS(scheduler=NS(enable_chunked_prefill=True))
    for bad in ({"max_jobs": -1}, {"reserve_margin_blocks": -2}, {"low_available_tokens_threshold": 0},
                {"short_decode_token_threshold": 0}):
        init_b200_config({"scheduler_config": {"batch_job_sched_config": dict({"enabled": True}, **bad)}}, refresh=True)
        with pytest.raises(ValueError, match="batch_job_sched_config"):
            _validate_scheduler_ext(get_b200_config().scheduler_config, engine_cfg)
    init_b200_config({"scheduler_config": {"batch_job_sched_config": {"enabled": True}}}, refresh=True)
    _validate_scheduler_ext(get_b200_config().scheduler_config, engine_cfg)


# ---------------------------------------------------------------- engine
def test_engine_on_the_batch_job_policy_learns_lengths_and_matches_fcfs():
    from vllm_ascend_b200.engine.llm import LLM
    rng = np.random.default_rng(3)
    prompts = [rng.integers(1, 400, size=n).tolist() for n in (20, 35, 12, 50, 8, 27, 40, 16)]
    lens = [3, 12, 3, 12, 3, 12, 3, 12]
    sps = [SamplingParams(max_tokens=m, temperature=0.0, ignore_eos=True) for m in lens]
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=3, max_num_batched_tokens=64)
    base = LLM("tiny-qwen", **kw)
    want = [o.outputs[0].token_ids for o in base.generate(prompts, sps)]
    llm = LLM("tiny-qwen", additional_config={"scheduler_config": {"batch_job_sched_config": {
        "enabled": True, "cold_start_requests": 1, "short_decode_token_threshold": 6}}}, **kw)
    sched = llm.engine.scheduler
    assert isinstance(sched, BatchJobAwareScheduler)
    # half of the requests name their job in the request id, the other half in a field of the prompt
    tagged = []
    for i, (p, m) in enumerate(zip(prompts, lens)):
        job = "brief" if m == 3 else "essay"
        tagged.append({"prompt_token_ids": p, "request_id": f"#job_name[{job}]#-{i}"} if i < 4
                      else {"prompt_token_ids": p, "job_id": job})
    outs = llm.generate(tagged, sps)
    assert [o.outputs[0].token_ids for o in outs] == want            # order of admission does not change tokens
    st = sched.job_stats()
    assert st["brief"]["predicted_decode"] == 3 and st["essay"]["predicted_decode"] == 12
    assert st["brief"]["samples"] == 4 and len(sched.parser) == 0    # names of finished requests are dropped
    assert not sched.waiting and len(sched.waiting) == 0
