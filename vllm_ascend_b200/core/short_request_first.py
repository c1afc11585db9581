"""Short-request-first waiting queue with aging.

Behaviour of vllm_ascend/core/short_request_first_scheduler.py:37-384: three lanes
(immediate / short / long).  Requests whose prompt is at most ``threshold`` tokens
go to the short lane and are admitted before long ones; a long request that has
waited ``long_max_wait_ms`` is promoted ahead of the short lane so it cannot
starve.  Preempted requests re-enter the immediate lane.
"""
from __future__ import annotations

import time
from collections import deque
from typing import Optional

from ..engine.request import Request, RequestStatus
from ..engine.scheduler import Scheduler
from ..platform_config import get_b200_config


class ShortRequestFirstScheduler(Scheduler):
    def __init__(self, sched_cfg, cache_cfg, num_blocks, kv_connector=None, engine_cfg=None,
                 clock=time.monotonic):
        super().__init__(sched_cfg, cache_cfg, num_blocks, kv_connector)
        c = get_b200_config().scheduler_config.short_request_first_config
        self.threshold = c.threshold
        self.long_max_wait_ms = c.long_max_wait_ms
        self.clock = clock
        self.immediate: deque[Request] = deque()
        self.short: deque[Request] = deque()
        self.long: deque[Request] = deque()
        self._long_enqueued: dict[str, float] = {}
        self.aged_long_promotions = 0
        self.waiting = _LaneView(self)      # keeps the base-class bookkeeping working

    def _classify(self, req: Request) -> deque:
        if req.status == RequestStatus.PREEMPTED or req.num_preemptions > 0:
            return self.immediate
        return self.short if req.num_prompt_tokens <= self.threshold else self.long

    def _enqueue(self, req: Request, front: bool = False) -> None:
        lane = self._classify(req)
        (lane.appendleft if front else lane.append)(req)
        if lane is self.long:
            self._long_enqueued.setdefault(req.request_id, self.clock())

    def _pick_waiting(self) -> Optional[Request]:
        if self.immediate:
            return self.immediate[0]
        if self.long and self.short and self.long_max_wait_ms > 0:
            waited = (self.clock() - self._long_enqueued.get(self.long[0].request_id, self.clock())) * 1e3
            if waited >= self.long_max_wait_ms:
                self.aged_long_promotions += 1
                return self.long[0]
        if self.short:
            return self.short[0]
        return self.long[0] if self.long else None

    def _pop_waiting(self, req: Request) -> None:
        for lane in (self.immediate, self.short, self.long):
            if lane and lane[0] is req:
                lane.popleft()
                break
        else:
            for lane in (self.immediate, self.short, self.long):
                if req in lane:
                    lane.remove(req)
                    break
        self._long_enqueued.pop(req.request_id, None)


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
        self.s._pop_waiting(req)

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
