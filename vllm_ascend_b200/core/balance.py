"""Balance scheduling across data-parallel ranks.

Behaviour of vllm_ascend/patch/platform/patch_balance_schedule.py:104-912: before
admitting new prefills every DP rank shares how many requests it is running (a CPU
all-gather); a rank only admits waiting requests while it is not ahead of the
least-loaded rank by more than one request, so prefill bursts spread evenly and
decode batches stay the same size on every rank.
"""
from __future__ import annotations

from typing import Callable, Optional

from ..engine.scheduler import Scheduler, SchedulerOutput
from ..parallel import state as pstate


class BalanceScheduler(Scheduler):
    def __init__(self, sched_cfg, cache_cfg, num_blocks, kv_connector=None, engine_cfg=None,
                 gather_fn: Optional[Callable[[int], list[int]]] = None):
        super().__init__(sched_cfg, cache_cfg, num_blocks, kv_connector)
        self._gather = gather_fn or (lambda v: pstate.get_dp_group().all_gather_object(v))
        self._peer_running: list[int] = []
        self.max_lead = 1

    def schedule(self) -> SchedulerOutput:
        self._peer_running = self._gather(len(self.running))
        return super().schedule()

    def _can_admit(self, req, num_new_blocks: int) -> bool:
        if self._peer_running and len(self.running) - min(self._peer_running) >= self.max_lead \
                and min(self._peer_running) < self.cfg.max_num_seqs and len(self.running) > 0:
            # some peer still has fewer sequences: let it catch up first
            if any(p < len(self.running) for p in self._peer_running):
                return False
        return super()._can_admit(req, num_new_blocks)
