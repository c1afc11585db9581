"""Dynamic load balancing of requests between data-parallel ranks by KV-cache pressure.

Every scheduling step the DP ranks share (KV usage, waiting tokens, running sequences).  A rank
whose pressure exceeds the least loaded rank's by more than a threshold hands over some of
its not-yet-started requests to that rank; the receiver queues them as its own.  Behaviour of
the reference's DyntraLB scheduler for decode-side DP balancing
(vllm_ascend/core/dyntra_lb_scheduler.py:113-1205, patch_dyntra_lb_core.py:411-493), with the
hand-over carried by two small CPU all-gathers instead of an engine-core side channel.
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np

from ..engine.request import Request, RequestStatus
from ..engine.scheduler import Scheduler, SchedulerOutput
from ..parallel import state as pstate


def _pack(req: Request) -> dict:
    return {"request_id": req.request_id, "prompt": np.asarray(req.prompt_token_ids).tolist(),
            "sampling_params": req.sampling_params, "eos_token_id": req.eos_token_id,
            "arrival_time": req.arrival_time, "priority": req.priority, "job_id": req.job_id,
            "client_index": getattr(req, "client_index", None), "origin_rank": getattr(req, "origin_rank", None)}


def _unpack(d: dict) -> Request:
    req = Request(d["request_id"], np.asarray(d["prompt"], dtype=np.int32), d["sampling_params"],
                  eos_token_id=d["eos_token_id"], priority=d["priority"], job_id=d["job_id"])
    req.arrival_time = d["arrival_time"]
    req.client_index, req.origin_rank = d["client_index"], d["origin_rank"]
    return req


class DyntraLBScheduler(Scheduler):
    def __init__(self, sched_cfg, cache_cfg, num_blocks, kv_connector=None, engine_cfg=None,
                 gather_fn: Optional[Callable] = None, rank: Optional[int] = None, world: Optional[int] = None):
        super().__init__(sched_cfg, cache_cfg, num_blocks, kv_connector)
        dp = pstate.get_dp_group()
        self.rank = dp.rank_in_group if rank is None else rank
        self.world = dp.world_size if world is None else world
        self._gather = gather_fn or (lambda v: dp.all_gather_object(v))
        from ..platform_config import get_b200_config
        c = get_b200_config().scheduler_config.dyntra_lb_config
        self.threshold = float(getattr(c, "imbalance_threshold", 0.15))
        self.max_migrations = int(getattr(c, "max_migrations_per_step", 4))
        self.migrated_out = 0
        self.migrated_in = 0

    # ------------------------------------------------------------------
    def pressure(self) -> float:
        """KV blocks in use plus the blocks the waiting prompts will need, as a fraction."""
        used = self.pool.num_blocks - self.pool.num_free_blocks
        waiting = sum((r.num_tokens + self.block_size - 1) // self.block_size
                      for r in self.waiting if r.status == RequestStatus.WAITING and not r.block_ids)
        return (used + waiting) / max(1, self.pool.num_blocks)

    def _movable(self) -> list[Request]:
        return [r for r in self.waiting if r.status == RequestStatus.WAITING and r.num_computed_tokens == 0
                and not r.block_ids and r.kv_transfer_params is None and r.lora_request is None]

    def balance(self) -> None:
        loads = self._gather((self.pressure(), len(self.waiting), len(self.running)))
        press = [l[0] for l in loads]
        lo = int(np.argmin(press))
        outbox: list[tuple[int, dict]] = []
        if self.rank != lo and press[self.rank] - press[lo] > self.threshold:
            movable = self._movable()
            # hand over the most recent arrivals: the oldest keep their place here
            per_req = 1.0 / max(1, self.pool.num_blocks)
            budget = (press[self.rank] - press[lo]) / 2
            for req in reversed(movable[-self.max_migrations:]):
                cost = ((req.num_tokens + self.block_size - 1) // self.block_size) * per_req
                if cost > budget:
                    continue
                budget -= cost
                outbox.append((lo, _pack(req)))
                self._pop_waiting(req)
                self.requests.pop(req.request_id, None)
                self._hashes.pop(req.request_id, None)
                self.migrated_out += 1
        for box in self._gather(outbox):
            for dst, payload in box:
                if dst == self.rank:
                    self.add_request(_unpack(payload))
                    self.migrated_in += 1

    def schedule(self) -> SchedulerOutput:
        if self.world > 1:
            self.balance()
        return super().schedule()
