"""Recompute scheduler for decode instances of a disaggregated deployment.

Behaviour of vllm_ascend/core/recompute_scheduler.py:102-1329: when the KV pull for
a request fails (``kv_connector.take_failed_requests``) or the pool is under
pressure, the request is not failed — it is reset and re-queued for a local
prefill ("recompute"), or, with policy "fail", aborted.  Requests kicked back to
the client/proxy for re-prefill are reported in ``recomputed_requests``.
"""
from __future__ import annotations

from ..engine.request import Request, RequestStatus
from ..engine.scheduler import Scheduler, SchedulerOutput
from ..platform_config import get_b200_config


class RecomputeScheduler(Scheduler):
    def __init__(self, sched_cfg, cache_cfg, num_blocks, kv_connector=None, engine_cfg=None):
        super().__init__(sched_cfg, cache_cfg, num_blocks, kv_connector)
        self.policy = get_b200_config().kv_load_failure_policy
        self.recomputed_requests: list[str] = []
        self.num_recomputes = 0

    def _handle_kv_failures(self) -> None:
        if self.kv_connector is None:
            return
        for rid in self.kv_connector.take_failed_requests():
            req = self.requests.get(rid)
            if req is None or req.is_finished:
                continue
            if self.policy == "fail":
                self.abort_request(rid)
                continue
            # drop whatever was (partially) loaded and prefill locally
            if req in self.running:
                self.running.remove(req)
            elif req in self.waiting:
                self.waiting.remove(req)
            self.pool.free(req.block_ids)
            req.block_ids = []
            req.num_computed_tokens = 0
            req.kv_transfer_params = None
            req.status = RequestStatus.WAITING
            self._release_row(req)
            self.waiting.appendleft(req)
            self.recomputed_requests.append(rid)
            self.num_recomputes += 1

    def schedule(self) -> SchedulerOutput:
        self._handle_kv_failures()
        return super().schedule()

    def _preempt(self, req: Request, out: SchedulerOutput) -> None:
        # under KV pressure a decode node hands the request back for re-prefill
        super()._preempt(req, out)
        req.kv_transfer_params = None
        self.recomputed_requests.append(req.request_id)
