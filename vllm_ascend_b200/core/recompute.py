"""Recompute scheduler for decode instances of a disaggregated deployment.

Behaviour of vllm_ascend/core/recompute_scheduler.py:102-1329: when the KV pull for
a request fails (``kv_connector.take_failed_requests``) or the pool is under
pressure, the request is not failed — it is reset and re-queued for a local
prefill ("recompute"), or, with policy "fail", aborted.  Under KV pressure a victim whose KV
the connector cannot park on the host is handed back to the proxy (``recompute_hand_back``):
it finishes with stop reason ``"recomputed"`` ahead of the step's regular outputs.
``recomputed_requests`` lists every request that took one of these routes.
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
        ktc = getattr(engine_cfg, "kv_transfer_config", None) or {}
        self.kv_role = ktc.get("kv_role", "")
        # hand requests back to the proxy under KV pressure (needs a proxy that re-routes them):
        # kv_connector_extra_config["recompute_hand_back"]
        self.hand_back = bool((ktc.get("kv_connector_extra_config") or {}).get("recompute_hand_back", False))
        self._handed_back: list[Request] = []

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

    def _is_consumer(self) -> bool:
        role = (self.kv_role or "").lower()
        return role in ("kv_consumer", "kv_both", "")

    def _preempt(self, req: Request, out: SchedulerOutput) -> None:
        """KV pressure on a decode node.  When the connector keeps a host copy of the victim's KV
        (``request_preempted`` accepts it) the request is preempted as usual and resumes from that
        copy.  Otherwise re-prefilling a long prompt here would stall every decode of the node, so
        the request is handed back: it finishes through the normal cleanup with stop reason
        ``"recomputed"`` and the tokens produced so far; the proxy in front re-routes prompt +
        output to a prefill node (vllm_ascend/core/recompute_scheduler.py:350-398, 976-995)."""
        hook = getattr(self.kv_connector, "request_preempted", None)
        if not self.hand_back or not self._is_consumer():
            super()._preempt(req, out)
            if hook is None:
                req.kv_transfer_params = None
            self.recomputed_requests.append(req.request_id)
            return
        if hook is not None and hook(req, req.block_ids):
            super()._preempt(req, out, parked=True)
            return
        self.running.remove(req)
        req.stop_reason = "recomputed"
        self._finish(req, RequestStatus.FINISHED_STOPPED)
        self.num_preemptions += 1
        self.recomputed_requests.append(req.request_id)
        self._handed_back.append(req)
        out.preempted.append(req)

    def update_from_output(self, out: SchedulerOutput, sampled: dict) -> list[Request]:
        finished = super().update_from_output(out, sampled)
        if self._handed_back:
            # the notification precedes the step's regular outputs
            finished = self._handed_back + [r for r in finished if r not in self._handed_back]
            self._handed_back = []
        return finished
