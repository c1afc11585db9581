"""Short-request-first waiting queue with aging.

Behaviour of vllm_ascend/core/short_request_first_scheduler.py:37-384: three lanes
(immediate / short / long).  Requests whose prompt is at most ``threshold`` tokens
go to the short lane and are admitted before long ones; a long request that has
waited ``long_max_wait_ms`` is promoted ahead of the short lane so it cannot
starve.  Preempted requests re-enter the immediate lane, and so does whatever an optional
predicate names.  The head chosen by a peek stays the head until it is popped; a run of aged
long requests overtaking waiting short ones is reported once per run; lane sizes and dispatch
counts are logged every few seconds.
"""
from __future__ import annotations

import time
from collections import deque
from typing import Optional

from ..engine.request import Request, RequestStatus
from ..engine.scheduler import Scheduler
from ..logger import logger
from ..platform_config import get_b200_config


class ShortRequestFirstScheduler(Scheduler):
    AGED_STREAK_WARNING = 8        # aged long requests dispatched in a row, with short ones waiting
    STATS_INTERVAL_S = 5.0

    def __init__(self, sched_cfg, cache_cfg, num_blocks, kv_connector=None, engine_cfg=None,
                 clock=time.monotonic, immediate_predicate=None):
        super().__init__(sched_cfg, cache_cfg, num_blocks, kv_connector)
        c = get_b200_config().scheduler_config.short_request_first_config
        self.threshold = c.threshold
        self.long_max_wait_ms = c.long_max_wait_ms
        self.clock = clock
        # Every rank of a replica runs its own copy of this queue and all copies must pick alike, but their
        # clocks differ: whether the oldest long request has aged is decided by the first rank and shared.
        self._agree = None
        from ..parallel import state as pstate
        groups = [g for g in (pstate.get_tp_group(), pstate.get_pp_group()) if g.world_size > 1]
        if groups:
            def agree(flag: bool) -> bool:
                for g in groups:
                    flag = bool(g.broadcast_object(bool(flag), src=0))
                return flag
            self._agree = agree
        # requests that bypass both lanes: preempted ones always, plus whatever the deployment names
        # (e.g. requests whose KV is already on the device after a remote prefill)
        self.immediate_predicate = immediate_predicate
        self.immediate: deque[Request] = deque()
        self.short: deque[Request] = deque()
        self.long: deque[Request] = deque()
        self._long_enqueued: dict[str, float] = {}
        self._pinned: Optional[tuple[deque, Request, bool]] = None     # (lane, head, aged) chosen by the last peek
        self.dispatched = {"immediate": 0, "short": 0, "long": 0, "aged_long": 0}
        self.aged_long_promotions = 0
        self.aged_streak = 0
        self._last_stats = clock()
        self.waiting = _LaneView(self)      # keeps the base-class bookkeeping working

    def _classify(self, req: Request) -> deque:
        if req.status == RequestStatus.PREEMPTED or req.num_preemptions > 0 or req.block_ids:
            return self.immediate
        if self.immediate_predicate is not None and self.immediate_predicate(req):
            return self.immediate
        return self.short if req.num_prompt_tokens <= self.threshold else self.long

    def _enqueue(self, req: Request, front: bool = False) -> None:
        lane = self._classify(req)
        (lane.appendleft if front else lane.append)(req)
        if lane is self.long:
            self._long_enqueued.setdefault(req.request_id, self.clock())
        self._pinned = None

    def _pick_waiting(self) -> Optional[Request]:
        """The head to admit next.  The choice is pinned until that request is popped: the admission
        loop peeks, checks the budget and pops, and the answer must not flip in between because a long
        request crossed its waiting limit meanwhile."""
        pin = self._pinned
        if pin is not None and pin[0] and pin[0][0] is pin[1]:
            return pin[1]
        self._maybe_log_stats()
        lane, aged = None, False
        if self.immediate:
            lane = self.immediate
        elif self.long and self.short and self.long_max_wait_ms > 0 and self._aged():
            lane, aged = self.long, True
        elif self.short:
            lane = self.short
        elif self.long:
            lane = self.long
        if lane is None:
            self._pinned = None
            return None
        self._pinned = (lane, lane[0], aged)
        return lane[0]

    def _aged(self) -> bool:
        waited_ms = (self.clock() - self._long_enqueued.get(self.long[0].request_id, self.clock())) * 1e3
        flag = waited_ms >= self.long_max_wait_ms
        return self._agree(flag) if self._agree is not None else flag

    def _pop_waiting(self, req: Request, dispatched: bool = True) -> None:
        pin, self._pinned = self._pinned, None
        for name, lane in (("immediate", self.immediate), ("short", self.short), ("long", self.long)):
            if lane and lane[0] is req:
                lane.popleft()
            elif req in lane:
                lane.remove(req)
            else:
                continue
            if dispatched:
                self._account(name, pin is not None and pin[1] is req and pin[2])
            break
        self._long_enqueued.pop(req.request_id, None)

    def _account(self, lane: str, aged: bool) -> None:
        self.dispatched[lane] += 1
        if aged:
            self.dispatched["aged_long"] += 1
            self.aged_long_promotions += 1
            self.aged_streak += 1
            if self.aged_streak == self.AGED_STREAK_WARNING:
                logger.warning("short-request-first: %d long requests in a row overtook %d waiting short ones "
                               "after long_max_wait_ms=%.0f; the long lane is backlogged",
                               self.aged_streak, len(self.short), self.long_max_wait_ms)
        elif lane == "short":
            self.aged_streak = 0

    def _maybe_log_stats(self) -> None:
        now = self.clock()
        if now - self._last_stats >= self.STATS_INTERVAL_S:
            self._last_stats = now
            logger.info("short-request-first: waiting immediate=%d short=%d long=%d; dispatched %s",
                        len(self.immediate), len(self.short), len(self.long), self.dispatched)


class _LaneView:
    """Deque-like facade over the three lanes used by the base scheduler."""

    def __init__(self, s: ShortRequestFirstScheduler):
        self.s = s

    def _all(self):
        return list(self.s.immediate) + list(self.s.short) + list(self.s.long)

    def append(self, req):
        self.s._enqueue(req)

    def appendleft(self, req):
        self.s._enqueue(req, front=True)

    def remove(self, req):
        self.s._pop_waiting(req, dispatched=False)      # aborts and rotations are not dispatches

    def popleft(self):
        req = self.s._pick_waiting()
        self.s._pop_waiting(req)
        return req

    def __len__(self):
        return len(self.s.immediate) + len(self.s.short) + len(self.s.long)

    def __bool__(self):
        return len(self) > 0

    def __iter__(self):
        return iter(self._all())

    def __contains__(self, req):
        return any(req in lane for lane in (self.s.immediate, self.s.short, self.s.long))

    def __getitem__(self, i):
        if i == 0:
            return self.s._pick_waiting()
        return self._all()[i]
