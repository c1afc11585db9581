"""Dynamic load balancing of requests between data-parallel ranks by KV-cache load.

Decode-side data parallelism steps in lock-step: a step is as slow as the rank with the most KV to
read, so ranks should hold about the same number of KV blocks.  Arrival order does not give that
(long and short requests land where the front end put them, ranks finish at different times).

Every scheduling step the DP ranks all-gather a small report (blocks of every running request,
blocks of every request still waiting, pool size) and each runs the same deterministic planner on
the gathered reports.  The plan is, per rank:

* ``out_blk``: block counts of requests this rank gives up (taken from its waiting queue first; from
  its running set when the queue does not hold enough, newest first, never a request longer than
  ``long_req_block_threshold`` blocks: what a migrated running request computed is recomputed by
  the receiver, so long ones stay),
* ``in_blk``: block counts of requests it receives,
* ``freeze``: the rank admits nothing new this step (it is above the mean by more than the
  threshold and requests are on their way out).

A request given up is removed from this rank (a running one is paused: blocks freed, batch row
released) and travels with its generated tokens; the receiver queues it like a resumed request, so
its next step recomputes prompt + generated tokens and decoding continues where it stopped.
Results are attributed through ``origin_rank`` / ``client_index`` as for any DP request.

Role of the reference's DyntraLB scheduler (vllm_ascend/core/dyntra_lb_scheduler.py:113-1205:
``prepare_dyntra_lb_step`` / ``_apply_load_balance_modifications`` with ``out_blk`` / ``in_blk`` /
``freeze`` modifications, pausing of running requests, block-count load unit, diagnostics line;
patch_dyntra_lb_core.py:411-493 computes the plan across ranks).  The reports and the hand-over
travel in two small CPU all-gathers per step instead of an engine-core side channel.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np

from ..engine.request import Request, RequestStatus
from ..engine.scheduler import Scheduler, SchedulerOutput
from ..logger import logger
from ..parallel import state as pstate


def _pack(req: Request) -> dict:
    return {"request_id": req.request_id, "prompt": np.asarray(req.prompt_token_ids).tolist(),
            "sampling_params": req.sampling_params, "eos_token_id": req.eos_token_id,
            "arrival_time": req.arrival_time, "priority": req.priority, "job_id": req.job_id,
            "client_index": getattr(req, "client_index", None), "origin_rank": getattr(req, "origin_rank", None),
            "outputs": list(req.output_token_ids or []), "first_token_time": req.first_token_time,
            "logprobs": req.logprobs}


def _unpack(d: dict) -> Request:
    req = Request(d["request_id"], np.asarray(d["prompt"], dtype=np.int32), d["sampling_params"],
                  eos_token_id=d["eos_token_id"], priority=d["priority"], job_id=d["job_id"])
    req.arrival_time = d["arrival_time"]
    req.client_index, req.origin_rank = d["client_index"], d["origin_rank"]
    outs = d.get("outputs") or []
    if outs:                                   # a paused running request: resumes after recomputing its tokens
        req.output_token_ids = list(outs)
        req.num_output_tokens = len(outs)
        req.first_token_time = d.get("first_token_time")
        req.logprobs = d.get("logprobs")
        req.status = RequestStatus.PREEMPTED
    return req


@dataclass
class RankReport:
    """What one rank tells the others before a balancing decision."""
    running: list = field(default_factory=list)     # blocks of every running request (movable or not)
    movable_running: list = field(default_factory=list)   # blocks of running requests that may be paused
    waiting: list = field(default_factory=list)     # blocks of every waiting request that may move
    pool_blocks: int = 1

    @property
    def load(self) -> int:
        return int(sum(self.running) + sum(self.waiting))


@dataclass
class Modification:
    out_blk: list = field(default_factory=list)
    out_to: list = field(default_factory=list)      # destination rank of every entry of out_blk
    in_blk: list = field(default_factory=list)
    freeze: bool = False


def plan_balance(reports: list, threshold: float, max_moves: int) -> list:
    """Deterministic plan from all ranks' reports (every rank computes the same one).

    Loads are block counts; the gap that triggers a move is ``threshold`` times the mean pool size.
    Each move goes from the currently most loaded rank to the least loaded one and is the largest
    waiting request that does not overshoot (a running one only when no waiting request fits)."""
    n = len(reports)
    mods = [Modification() for _ in range(n)]
    if n < 2:
        return mods
    loads = [r.load for r in reports]
    gap_min = threshold * (sum(r.pool_blocks for r in reports) / n)
    mean = sum(loads) / n
    # movable requests per rank: [waiting, running]; waiting ones go first (nothing to recompute)
    avail = [[sorted(r.waiting), sorted(r.movable_running)] for r in reports]
    moves = [0] * n

    def choose(pool: list, gap: int):
        """Index of the largest request that does not overshoot (leaves the donor at or above the
        receiver); failing that of the smallest one, if moving it still narrows the gap."""
        fit = [k for k, b in enumerate(pool) if 0 < 2 * b <= gap]
        if fit:
            return max(fit, key=lambda k: (pool[k], -k))
        small = [k for k, b in enumerate(pool) if 0 < b < gap]
        return min(small, key=lambda k: (pool[k], k)) if small else None

    for _ in range(n * max(1, max_moves)):
        donor = max(range(n), key=lambda i: (loads[i], -i))
        recv = min(range(n), key=lambda i: (loads[i], i))
        if donor == recv or loads[donor] - loads[recv] <= gap_min or moves[donor] >= max_moves:
            break
        gap = loads[donor] - loads[recv]
        src, pick = None, None
        for pool in avail[donor]:
            pick = choose(pool, gap)
            if pick is not None:
                src = pool
                break
        if src is None:
            break
        b = src.pop(pick)
        mods[donor].out_blk.append(b)
        mods[donor].out_to.append(recv)
        mods[recv].in_blk.append(b)
        loads[donor] -= b
        loads[recv] += b
        moves[donor] += 1
    for i in range(n):
        # a rank well above the mean that is shedding load takes nothing new this step
        mods[i].freeze = bool(mods[i].out_blk) and (reports[i].load - mean) > gap_min
    return mods


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
        self.long_req_blocks = int(getattr(c, "long_req_block_threshold", 64))
        self.start_step = int(getattr(c, "start_step", 0))
        self.end_step = int(getattr(c, "end_step", 0))
        self.migrate_running = getattr(c, "mode", "kv_load") == "kv_load"
        self.diagnostics = bool(getattr(c, "enable_diagnostics", False))
        self.lb_freeze = False
        # schedule() runs collectives: the engine calls it on every DP rank every step, busy or not
        self.collective_schedule = self.world > 1
        self.migrated_out = 0
        self.migrated_in = 0
        self.paused_running = 0
        self.last_modification: Optional[Modification] = None

    # ------------------------------------------------------------------ load accounting
    def _blocks(self, req: Request) -> int:
        return (req.num_tokens + self.block_size - 1) // self.block_size

    def pressure(self) -> float:
        """KV blocks in use plus the blocks the waiting prompts will need, as a fraction."""
        used = self.pool.num_blocks - self.pool.num_free_blocks
        waiting = sum(self._blocks(r) for r in self.waiting if r.status == RequestStatus.WAITING and not r.block_ids)
        return (used + waiting) / max(1, self.pool.num_blocks)

    def _movable(self) -> list[Request]:
        return [r for r in self.waiting if r.status in (RequestStatus.WAITING, RequestStatus.PREEMPTED)
                and r.num_computed_tokens == 0 and not r.block_ids and r.kv_transfer_params is None
                and r.lora_request is None and not r.mm_inputs and r.guided is None]

    def _movable_running(self) -> list[Request]:
        """Running requests that may be paused and resumed elsewhere: decoding (prefill done), nothing
        in flight, no state another rank cannot rebuild from the tokens, not long."""
        if not self.migrate_running:
            return []
        return [r for r in self.running if self._resumable(r) and self._blocks(r) <= self.long_req_blocks]

    @staticmethod
    def _resumable(r: Request) -> bool:
        # sampling state is a function of (seed, request id, tokens sampled so far): it travels with the tokens
        return (r.num_inflight == 0 and not r.spec_token_ids and r.num_computed_tokens >= r.num_prompt_tokens
                and r.kv_transfer_params is None and r.lora_request is None and not r.mm_inputs and r.guided is None)

    def report(self) -> RankReport:
        return RankReport(running=[self._blocks(r) for r in self.running],
                          movable_running=[self._blocks(r) for r in self._movable_running()],
                          waiting=[self._blocks(r) for r in self._movable()],
                          pool_blocks=self.pool.num_blocks)

    # ------------------------------------------------------------------ applying a plan
    def _pause_running(self, req: Request) -> None:
        """Take a running request out of this rank: blocks and batch row go back, its tokens stay with it."""
        self.running.remove(req)
        self.pool.free(req.block_ids)
        req.block_ids = []
        req.num_computed_tokens = 0
        self._uncommit_blocks(req)
        self._release_row(req)
        self.paused_running += 1

    def _take(self, blocks: int, taken: set) -> Optional[Request]:
        """A request of exactly ``blocks`` blocks to give up: newest waiting first, then newest running."""
        for r in reversed(self._movable()):
            if r.request_id not in taken and self._blocks(r) == blocks:
                self._pop_waiting(r)
                return r
        for r in reversed(self._movable_running()):
            if r.request_id not in taken and self._blocks(r) == blocks:
                self._pause_running(r)
                return r
        return None

    def balance(self) -> None:
        step = self.step_id + 1
        active = step >= self.start_step and (self.end_step <= 0 or step <= self.end_step)
        rep = self.report() if active else RankReport(pool_blocks=self.pool.num_blocks)
        reports = self._gather(rep)
        # a bus that returns one contribution (tests) or ranks running an older report format
        reports = [r if isinstance(r, RankReport) else RankReport() for r in reports]
        outbox: list[tuple[int, dict]] = []
        self.lb_freeze = False
        if len(reports) == self.world and active:
            mod = plan_balance(reports, self.threshold, self.max_migrations)[self.rank]
            self.last_modification = mod
            self.lb_freeze = mod.freeze
            taken: set = set()
            for blocks, dst in zip(mod.out_blk, mod.out_to):
                req = self._take(blocks, taken)
                if req is None:
                    continue                    # state moved since the report: the planner retries next step
                taken.add(req.request_id)
                outbox.append((dst, _pack(req)))
                self.requests.pop(req.request_id, None)
                self._hashes.pop(req.request_id, None)
                self.migrated_out += 1
        for box in self._gather(outbox):
            for dst, payload in box:
                if dst == self.rank:
                    self._adopt(_unpack(payload))
        if self.diagnostics:
            self._print_summary()

    def _adopt(self, req: Request) -> None:
        self.requests[req.request_id] = req
        if req.status == RequestStatus.PREEMPTED:
            self.waiting.appendleft(req)        # it was already running: resumes before new arrivals
        else:
            req.status = RequestStatus.WAITING
            self.waiting.append(req)
        self.migrated_in += 1

    def _can_admit(self, req: Request, num_new_blocks: int) -> bool:
        if self.lb_freeze and req.status != RequestStatus.PREEMPTED and req.num_computed_tokens == 0:
            return False
        return super()._can_admit(req, num_new_blocks)

    def _print_summary(self) -> None:
        waiting = list(self.waiting)
        logger.info("schedule() | req num [running=%d, waiting=%d, remote_kv=%d, preempted=%d] | blk num "
                    "[running=%d, waiting=%d] | lb [out=%d, in=%d, paused=%d, freeze=%s]",
                    len(self.running), len(waiting),
                    sum(r.status == RequestStatus.WAITING_FOR_REMOTE_KVS for r in waiting),
                    sum(r.status == RequestStatus.PREEMPTED for r in waiting),
                    sum(self._blocks(r) for r in self.running), sum(self._blocks(r) for r in waiting),
                    self.migrated_out, self.migrated_in, self.paused_running, self.lb_freeze)

    def schedule(self) -> SchedulerOutput:
        if self.world > 1:
            self.balance()
        return super().schedule()
