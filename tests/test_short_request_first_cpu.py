"""Short-request-first queue: lanes, aging, the pinned head, the starvation warning, periodic stats."""
import logging

import pytest

from vllm_ascend_b200.config import CacheConfig, SchedulerConfig
from vllm_ascend_b200.core.short_request_first import ShortRequestFirstScheduler
from vllm_ascend_b200.engine.request import Request, RequestStatus, SamplingParams
from vllm_ascend_b200.platform_config import clear_b200_config, init_b200_config


class Clock:
    def __init__(self):
        self.t = 100.0

    def __call__(self):
        return self.t


def _req(rid, n):
    return Request(request_id=rid, prompt_token_ids=list(range(1, n + 1)),
                   sampling_params=SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))


def _sched(clock, threshold=32, long_max_wait_ms=1000.0, **kw):
    init_b200_config({"scheduler_config": {"short_request_first_config": {
        "enabled": True, "threshold": threshold, "long_max_wait_ms": long_max_wait_ms}}}, refresh=True)
    sc = SchedulerConfig(max_num_seqs=64, max_num_batched_tokens=4096, max_model_len=1024)
    return ShortRequestFirstScheduler(sc, CacheConfig(block_size=16), 4096, clock=clock, **kw)


@pytest.fixture(autouse=True)
def _clean():
    yield
    clear_b200_config()


def test_lanes_and_dispatch_priority():
    s = _sched(Clock(), immediate_predicate=lambda r: r.request_id.startswith("vip"))
    reqs = [_req("long-a", 100), _req("short-a", 32), _req("vip-a", 500), _req("short-b", 5), _req("long-b", 33)]
    for r in reqs:
        s.add_request(r)
    assert [r.request_id for r in s.immediate] == ["vip-a"]
    assert [r.request_id for r in s.short] == ["short-a", "short-b"]          # at the threshold counts as short
    assert [r.request_id for r in s.long] == ["long-a", "long-b"]
    pre = _req("pre", 10)
    pre.status = RequestStatus.PREEMPTED
    s.waiting.appendleft(pre)
    order = [s.waiting.popleft().request_id for _ in range(len(s.waiting))]
    assert order == ["pre", "vip-a", "short-a", "short-b", "long-a", "long-b"]
    assert s.dispatched == {"immediate": 2, "short": 2, "long": 2, "aged_long": 0}


def test_aged_long_request_overtakes_short_ones_and_zero_disables_aging():
    clk = Clock()
    s = _sched(clk, long_max_wait_ms=1000.0)
    s.add_request(_req("long", 100))
    s.add_request(_req("short-1", 5))
    s.add_request(_req("short-2", 5))
    assert s._pick_waiting().request_id == "short-1"
    s._pop_waiting(s._pick_waiting())
    clk.t += 1.5
    assert s._pick_waiting().request_id == "long"                             # waited 1.5 s > 1 s
    s._pop_waiting(s._pick_waiting())
    assert s.aged_long_promotions == 1 and s.dispatched["aged_long"] == 1
    assert s._pick_waiting().request_id == "short-2"
    off = _sched(clk, long_max_wait_ms=0.0)
    off.add_request(_req("long", 100))
    off.add_request(_req("short", 5))
    clk.t += 1e6
    assert off._pick_waiting().request_id == "short" and off.aged_long_promotions == 0


def test_the_head_chosen_by_a_peek_stays_until_it_is_popped():
    clk = Clock()
    s = _sched(clk, long_max_wait_ms=1000.0)
    s.add_request(_req("long", 100))
    s.add_request(_req("short", 5))
    head = s._pick_waiting()
    assert head.request_id == "short"
    clk.t += 5.0                                  # the long request ages between the peek and the pop
    assert s._pick_waiting() is head and s.waiting[0] is head
    s._pop_waiting(head)
    assert s.dispatched["short"] == 1 and s.dispatched["aged_long"] == 0
    # the next peek is free to choose again; with no short request left the long one is not "aged"
    assert s._pick_waiting().request_id == "long"
    s._pop_waiting(s._pick_waiting())
    assert s.aged_long_promotions == 0
    # a new arrival releases the pin
    s.add_request(_req("long-2", 100))
    assert s._pick_waiting().request_id == "long-2"
    s.add_request(_req("short-2", 5))
    assert s._pick_waiting().request_id == "short-2"
    # an abort is not a dispatch
    s.abort_request("short-2")
    assert s.dispatched["short"] == 1 and s._pick_waiting().request_id == "long-2"


def test_run_of_aged_promotions_warns_once_and_resets_after_a_short_dispatch(caplog):
    clk = Clock()
    s = _sched(clk, long_max_wait_ms=10.0)
    n = s.AGED_STREAK_WARNING
    for i in range(2 * n + 6):
        s.add_request(_req(f"long-{i}", 100))
    for i in range(3):
        s.add_request(_req(f"short-{i}", 5))
    clk.t += 1.0
    with caplog.at_level(logging.WARNING, logger="vllm_ascend_b200"):
        for _ in range(n + 3):
            s._pop_waiting(s._pick_waiting())
        warned = [r for r in caplog.records if "long requests in a row" in r.getMessage()]
        assert len(warned) == 1 and s.aged_streak == n + 3
        # a short dispatch ends the run (aging is switched off for it), the next run warns again
        s.long_max_wait_ms = 0.0
        assert s._pick_waiting().request_id == "short-0"
        s._pop_waiting(s._pick_waiting())
        assert s.aged_streak == 0
        s.long_max_wait_ms = 10.0
        for _ in range(n):
            s._pop_waiting(s._pick_waiting())
        warned = [r for r in caplog.records if "long requests in a row" in r.getMessage()]
        assert len(warned) == 2


def test_stats_are_logged_every_five_seconds(caplog):
    clk = Clock()
    s = _sched(clk)
    s.add_request(_req("a", 5))
    with caplog.at_level(logging.INFO, logger="vllm_ascend_b200"):
        s._pick_waiting()
        s._pinned = None
        clk.t += 4.0
        s._pick_waiting()
        assert not [r for r in caplog.records if "waiting immediate=" in r.getMessage()]
        s._pinned = None
        clk.t += 1.5
        s._pick_waiting()
        s._pinned = None
        s._pick_waiting()
        assert len([r for r in caplog.records if "waiting immediate=" in r.getMessage()]) == 1


def test_engine_tokens_on_the_policy_equal_fcfs():
    import numpy as np
    from vllm_ascend_b200.engine.llm import LLM
    rng = np.random.default_rng(5)
    prompts = [rng.integers(1, 400, size=n).tolist() for n in (60, 8, 45, 5, 70, 12)]
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    kw = dict(device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=2, max_num_batched_tokens=64)
    want = [o.outputs[0].token_ids for o in LLM("tiny-qwen", **kw).generate(prompts, sp)]
    llm = LLM("tiny-qwen", additional_config={"scheduler_config": {"short_request_first_config": {
        "enabled": True, "threshold": 16}}}, **kw)
    assert isinstance(llm.engine.scheduler, ShortRequestFirstScheduler)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == want
    d = llm.engine.scheduler.dispatched
    assert d["short"] == 3 and d["long"] == 3
