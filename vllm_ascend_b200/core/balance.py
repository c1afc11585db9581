"""Balance scheduling across data-parallel ranks.

Data-parallel replicas of a MoE model meet in the expert-parallel collectives of every layer, so a
step lasts as long as the slowest replica's batch.  Admitting requests greedily lets one replica
fill up to ``max_num_seqs`` while others still run small batches, and from then on every step
pays for the full replica.  This scheduler keeps the running sets even:

* once per step every replica shares ``len(running)`` (one CPU all-gather).  The gather runs on
  every replica every step, including replicas that have nothing to do (``collective_schedule``:
  the engine calls ``schedule()`` on idle replicas too), because a collective that one rank skips
  blocks the others;
* if any replica was at its running cap at the end of the previous step, nobody admits new
  requests in this step (any-rank-at-cap => global freeze): the full replica drains a little
  before the others grow further, and every replica reaches the decision from the same snapshot,
  without a leader;
* optionally (``max_lead`` > 0) a replica also waits while it is ahead of the least loaded
  replica by that many sequences and that replica still has room.

Behaviour of vllm_ascend/patch/platform/patch_balance_schedule.py:104-163 (gather outside the
per-rank early exits) and :393-403 (the freeze inside the admission loop).
"""
from __future__ import annotations

from typing import Callable, Optional

from ..engine.scheduler import Scheduler, SchedulerOutput
from ..parallel import state as pstate


class BalanceScheduler(Scheduler):
    def __init__(self, sched_cfg, cache_cfg, num_blocks, kv_connector=None, engine_cfg=None,
                 gather_fn: Optional[Callable[[int], list[int]]] = None, world: Optional[int] = None,
                 max_lead: int = 0):
        super().__init__(sched_cfg, cache_cfg, num_blocks, kv_connector)
        if gather_fn is None:
            group = pstate.get_dp_group()
            world = group.world_size if world is None else world
            gather_fn = group.all_gather_object
        self._gather = gather_fn
        self.world = int(world or 1)
        self.collective_schedule = self.world > 1
        self.max_lead = int(max_lead)
        self.peer_running: list[int] = []
        self.frozen_steps = 0           # steps in which admission was held back
        self._frozen = False

    def balance_gather(self) -> list[int]:
        self.peer_running = [int(v) for v in self._gather(len(self.running))] if self.world > 1 else []
        return self.peer_running

    def schedule(self) -> SchedulerOutput:
        self.balance_gather()
        cap = self.cfg.max_num_seqs
        self._frozen = bool(self.peer_running) and max(self.peer_running) >= cap
        if self._frozen and self.waiting:
            self.frozen_steps += 1
        return super().schedule()

    def _can_admit(self, req, num_new_blocks: int) -> bool:
        if self._frozen and not req.block_ids:          # resumed requests hold state already
            return False
        if self.max_lead > 0 and self.peer_running and self.running:
            least = min(self.peer_running)
            if len(self.running) - least >= self.max_lead and least < self.cfg.max_num_seqs:
                return False
        return super()._can_admit(req, num_new_blocks)
