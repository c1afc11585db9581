"""Continuous-batching scheduler with chunked prefill, prefix caching and
recompute preemption.

Running requests are served first (one decode token, or the next prompt chunk),
then waiting requests are admitted while the token budget and the KV pool allow.
The waiting-queue order is a pluggable policy — the scheduler extensions of
``vllm_ascend/core`` (short-request-first, batch-job-aware, recompute, balance)
subclass this and override ``_pick_waiting`` / the admission hooks.
KV-connector hooks follow the scheduler-side contract of
vllm_ascend/distributed/kv_transfer/kv_p2p/mooncake_connector.py:1843-2001.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from ..config import CacheConfig, SchedulerConfig
from .block_pool import BlockPool
from .request import Request, RequestStatus


@dataclass
class SchedulerOutput:
    scheduled: list                      # [(Request, num_new_tokens)], decodes first
    num_scheduled_tokens: int = 0
    preempted: list = field(default_factory=list)
    finished_ids: list = field(default_factory=list)
    new_block_rows: list = field(default_factory=list)   # requests whose block list grew
    kv_connector_metadata: Optional[object] = None
    step_id: int = 0

    @property
    def is_empty(self) -> bool:
        return not self.scheduled


class Scheduler:
    def __init__(self, sched_cfg: SchedulerConfig, cache_cfg: CacheConfig, num_blocks: int,
                 kv_connector=None):
        self.cfg = sched_cfg
        self.block_size = cache_cfg.block_size
        self.pool = BlockPool(num_blocks, cache_cfg.block_size, cache_cfg.enable_prefix_caching)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.requests: dict[str, Request] = {}
        self.finished_since_last: list[str] = []
        self.kv_connector = kv_connector
        self.num_draft_tokens = 0
        self.spec_slack = 0        # num_speculative_tokens when speculative decoding is on
        self.num_accepted_tokens = 0
        self.max_loras = 0          # set by the engine when LoRA is enabled
        self.step_id = 0
        # blocks promised to admitted requests for their whole life (prompt + max_tokens);
        # admission keeps the sum within the pool so decode never has to preempt
        self.reserve_full = getattr(sched_cfg, "reserve_full_sequence", True)
        self._committed_blocks = 0
        self._commit: dict[str, int] = {}
        self.decode_batch_alignment = getattr(sched_cfg, "decode_batch_alignment", 1)
        self._free_rows = list(range(sched_cfg.max_num_seqs - 1, -1, -1))
        self._hashes: dict[str, list[bytes]] = {}
        # stats
        self.num_preemptions = 0

    # ------------------------------------------------------------------ API
    def add_request(self, req: Request) -> None:
        if req.num_prompt_tokens + 1 > self.cfg.max_model_len:
            raise ValueError(f"prompt of {req.num_prompt_tokens} tokens exceeds max_model_len "
                             f"{self.cfg.max_model_len}")
        self.requests[req.request_id] = req
        req.status = RequestStatus.WAITING
        self.waiting.append(req)

    def abort_request(self, request_id: str) -> None:
        req = self.requests.get(request_id)
        if req is None or req.is_finished:
            return
        if req in self.running:
            self.running.remove(req)
        elif req in self.waiting:
            self.waiting.remove(req)
        self._finish(req, RequestStatus.FINISHED_ABORTED)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    @property
    def num_unfinished(self) -> int:
        return len(self.waiting) + len(self.running)

    # ------------------------------------------------------------------ policy hooks
    def _pick_waiting(self) -> Optional[Request]:
        """Next candidate from the waiting queue (FCFS)."""
        return self.waiting[0] if self.waiting else None

    def _pop_waiting(self, req: Request) -> None:
        if self.waiting and self.waiting[0] is req:
            self.waiting.popleft()
        else:
            self.waiting.remove(req)

    def _final_blocks(self, req: Request) -> int:
        # draft tokens under verification occupy KV slots past the last accepted token
        n = min(req.num_prompt_tokens + req.sampling_params.max_tokens + self.spec_slack, self.cfg.max_model_len)
        return (n + self.block_size - 1) // self.block_size

    def _can_admit(self, req: Request, num_new_blocks: int) -> bool:
        if not self.pool.can_allocate(num_new_blocks):
            return False
        if self.max_loras and req.lora_request is not None:
            # a batch can address at most max_loras adapter slots
            active = {r.lora_request.lora_int_id for r in self.running if r.lora_request is not None}
            if req.lora_request.lora_int_id not in active and len(active) >= self.max_loras:
                return False
        if self.reserve_full and self.running:
            fb = self._final_blocks(req)
            room = self.pool.num_blocks - 1 - self._committed_blocks
            if fb > room:
                return False
            # Decode GEMMs work on tiles of `decode_batch_alignment` rows.  When the KV pool
            # (not max_num_seqs) limits the batch, stopping at a full tile instead of a few
            # rows into the next one avoids computing a mostly empty tile on every step.
            a = self.decode_batch_alignment
            n = len(self.running)
            if a > 1 and n >= a and n % a == 0:
                fit = room // max(fb, 1)
                if fit < a and len(self.waiting) > fit and n + fit < self.cfg.max_num_seqs:
                    return False
        return True

    def _commit_blocks(self, req: Request) -> None:
        if req.request_id not in self._commit:
            n = self._final_blocks(req)
            self._commit[req.request_id] = n
            self._committed_blocks += n

    def _uncommit_blocks(self, req: Request) -> None:
        self._committed_blocks -= self._commit.pop(req.request_id, 0)

    def _select_preemption_victim(self) -> Optional[Request]:
        # a request with a token still in flight cannot be rolled back before that step reports
        for req in reversed(self.running):
            if req.num_inflight == 0:
                return req
        return None

    # ------------------------------------------------------------------ core
    def _blocks_needed(self, req: Request, num_tokens_after: int) -> int:
        need = (num_tokens_after + self.block_size - 1) // self.block_size
        return max(0, need - len(req.block_ids))

    def try_extend(self, req: Request, num_tokens_after: int) -> bool:
        """Allocate the blocks ``req`` needs to hold ``num_tokens_after`` tokens if they are
        free right now (never preempts); used to give draft tokens KV slots ahead of time."""
        need = self._blocks_needed(req, num_tokens_after)
        if need > self.pool.num_free_blocks:
            return False
        if need:
            req.block_ids.extend(self.pool.allocate(need))
        return True

    def _preempt(self, req: Request, out: SchedulerOutput, parked: Optional[bool] = None) -> None:
        self.running.remove(req)
        # a connector may keep a host copy of what the request computed: it then frees the blocks
        # itself once the copy has finished (``parked``: a subclass already asked it)
        if parked is None:
            hook = getattr(self.kv_connector, "request_preempted", None)
            parked = hook is not None and bool(hook(req, req.block_ids))
        if not parked:
            self.pool.free(req.block_ids)
        req.block_ids = []
        req.num_computed_tokens = 0
        req.status = RequestStatus.PREEMPTED
        req.num_preemptions += 1
        self.num_preemptions += 1
        self._uncommit_blocks(req)
        self._release_row(req)
        self.waiting.appendleft(req)
        out.preempted.append(req)

    def release_row_id(self, row: int) -> None:
        """Return a batch row a connector held back after its request finished."""
        if row >= 0 and row not in self._free_rows:
            self._free_rows.append(row)

    def _release_row(self, req: Request) -> None:
        if req.row >= 0:
            self._free_rows.append(req.row)
            req.row = -1

    def schedule(self) -> SchedulerOutput:
        self.step_id += 1
        out = SchedulerOutput(scheduled=[], step_id=self.step_id)
        out.finished_ids, self.finished_since_last = self.finished_since_last, []
        budget = self.cfg.max_num_batched_tokens
        decodes: list = []
        prefills: list = []

        # ---- running requests
        i = 0
        while i < len(self.running) and budget > 0:
            req = self.running[i]
            spec = len(req.spec_token_ids)
            remaining = req.num_tokens + req.num_inflight + spec - req.num_computed_tokens
            if req.num_inflight and (req.num_output_tokens + req.num_inflight >= req.sampling_params.max_tokens
                                     or req.num_tokens + req.num_inflight >= self.cfg.max_model_len):
                remaining = 0           # its last token is already on the way
            n = min(remaining, budget)
            if spec and n < remaining:       # the token budget cuts into the draft tokens
                del req.spec_token_ids[max(0, spec - (remaining - n)):]
            if n <= 0:
                i += 1
                continue
            if not self.cfg.enable_chunked_prefill and n < remaining:
                i += 1
                continue
            need = self._blocks_needed(req, req.num_computed_tokens + n)
            preempted_self = False
            while need > self.pool.num_free_blocks:
                victim = self._select_preemption_victim()
                if victim is None:
                    break
                # victims scheduled earlier in this step must be dropped from the batch
                decodes = [(r, k) for r, k in decodes if r is not victim]
                prefills = [(r, k) for r, k in prefills if r is not victim]
                vi = self.running.index(victim)
                self._preempt(victim, out)
                if victim is req:
                    preempted_self = True
                    break
                if vi < i:
                    i -= 1
            if preempted_self:
                continue
            if need > self.pool.num_free_blocks:
                break
            if need:
                req.block_ids.extend(self.pool.allocate(need))
                out.new_block_rows.append(req)
            (decodes if n == 1 and req.num_computed_tokens >= req.num_prompt_tokens
             else prefills).append((req, n))
            budget -= n
            i += 1

        # ---- admit waiting requests
        while self.waiting and budget > 0 and len(self.running) < self.cfg.max_num_seqs \
                and not out.preempted:
            req = self._pick_waiting()
            if req is None:
                break
            if req.status == RequestStatus.WAITING_FOR_REMOTE_KVS:
                if self.kv_connector is None or not self.kv_connector.is_ready(req):
                    # rotate so it does not block the queue head
                    self._pop_waiting(req)
                    self.waiting.append(req)
                    if all(r.status == RequestStatus.WAITING_FOR_REMOTE_KVS for r in self.waiting):
                        break
                    continue
                req.status = RequestStatus.WAITING
            # prefix cache
            cached_blocks: list[int] = []
            if self.pool.enable_prefix_caching and req.num_computed_tokens == 0 and not req.block_ids \
                    and req.sampling_params.prompt_logprobs is None:      # every prompt position must be computed
                hashes = self._hashes.get(req.request_id)
                if hashes is None:
                    extra = BlockPool.request_key_extra(req)
                    hashes = [] if extra is None else self.pool.block_hashes(req.prompt_token_ids, extra)
                    self._hashes[req.request_id] = hashes
                # never treat the whole prompt as cached: the last token must be computed
                max_hit = (req.num_prompt_tokens - 1) // self.block_size
                cached_blocks = self.pool.find_cached_prefix(hashes[:max_hit])
            num_cached = len(cached_blocks) * self.block_size
            # external KV (disaggregated prefill): tokens the connector will load
            num_external, load_async = 0, False
            if self.kv_connector is not None and req.num_computed_tokens == 0:
                num_external, load_async = self.kv_connector.get_num_new_matched_tokens(req, num_cached)
            computed = max(req.num_computed_tokens, num_cached + num_external)
            remaining = req.num_tokens - computed
            n = min(remaining, budget) if not load_async else 0
            if not self.cfg.enable_chunked_prefill and n < remaining and not load_async:
                break
            total_after = computed + n
            need = (total_after + self.block_size - 1) // self.block_size - len(cached_blocks) \
                - len(req.block_ids)
            need = max(need, 0)
            if not self._can_admit(req, need):
                break
            self._pop_waiting(req)
            if cached_blocks:
                self.pool.touch(cached_blocks)
                req.block_ids = list(cached_blocks)
                req.num_cached_tokens = num_cached
            if need:
                req.block_ids.extend(self.pool.allocate(need))
            req.num_computed_tokens = computed
            if req.row < 0:
                req.row = self._free_rows.pop()
            out.new_block_rows.append(req)
            if self.kv_connector is not None:
                self.kv_connector.update_state_after_alloc(req, req.block_ids, num_external)
            if load_async:
                req.status = RequestStatus.WAITING_FOR_REMOTE_KVS
                self.waiting.append(req)
                continue
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            self._commit_blocks(req)
            if n > 0:
                prefills.append((req, n))
                budget -= n

        out.scheduled = decodes + prefills
        out.num_scheduled_tokens = sum(n for _, n in out.scheduled)
        if self.kv_connector is not None:
            out.kv_connector_metadata = self.kv_connector.build_connector_meta(out)
        return out

    # ------------------------------------------------------------------ results
    def advance(self, out: SchedulerOutput) -> None:
        """Asynchronous scheduling: account for a step at launch time instead of at completion.
        Every request's computed count moves now, and a request whose step will sample gets one
        in-flight token, so the next ``schedule()`` can plan the following step while this one
        is still running."""
        for req, n in out.scheduled:
            req.num_computed_tokens += n
            if req.num_computed_tokens >= req.num_tokens + req.num_inflight:
                req.num_inflight += 1
        out.advanced = True

    def update_from_output(self, out: SchedulerOutput, sampled: dict) -> list[Request]:
        """``sampled`` maps request_id -> list of new token ids (empty for a partial
        prefill chunk).  Returns the requests that finished in this step."""
        finished: list[Request] = []
        advanced = getattr(out, "advanced", False)
        for req, n in out.scheduled:
            if req.status != RequestStatus.RUNNING:
                continue
            if advanced:
                if sampled.get(req.request_id):
                    req.num_inflight = max(0, req.num_inflight - 1)
                n_spec, n = 0, 0
            else:
                # draft tokens verified in this step: only the accepted ones leave valid KV behind
                n_spec = max(0, req.num_computed_tokens + n - req.num_tokens)
            req.num_computed_tokens += n
            if n_spec:
                emitted = len(sampled.get(req.request_id) or ())
                req.num_computed_tokens -= n_spec - max(emitted - 1, 0)
                self.num_draft_tokens += n_spec
                self.num_accepted_tokens += max(emitted - 1, 0)
            req.spec_token_ids = []
            if self.pool.enable_prefix_caching:
                hashes = self._hashes.get(req.request_id)
                if hashes:
                    full = min(req.num_computed_tokens, req.num_prompt_tokens) // self.block_size
                    self.pool.cache_full_blocks(req.block_ids, hashes, full)
            toks = sampled.get(req.request_id)
            if not toks:
                continue
            if req.output_token_ids is None:
                req.output_token_ids = []
            sp = req.sampling_params
            for t in toks:
                req.output_token_ids.append(int(t))
                req.num_output_tokens += 1
                stop = None
                if req.num_output_tokens >= sp.max_tokens or req.num_tokens >= self.cfg.max_model_len:
                    stop = RequestStatus.FINISHED_LENGTH
                if req.num_output_tokens >= sp.min_tokens:
                    if (not sp.ignore_eos and req.eos_token_id is not None and t == req.eos_token_id) \
                            or (sp.stop_token_ids and t in sp.stop_token_ids):
                        stop = RequestStatus.FINISHED_STOPPED
                if stop is not None:
                    self.running.remove(req)
                    self._finish(req, stop)
                    finished.append(req)
                    break
        return finished

    def _finish(self, req: Request, status: RequestStatus) -> None:
        import time
        req.status = status
        req.num_inflight = 0
        req.finish_time = time.monotonic()
        delay_free = False
        if self.kv_connector is not None:
            delay_free, params = self.kv_connector.request_finished(req, req.block_ids)
            if params is not None:
                req.kv_transfer_params = params
        if not delay_free:
            self.free_blocks(req)
        self._uncommit_blocks(req)
        if delay_free and getattr(self.kv_connector, "holds_state_rows", False):
            req.row = -1          # the connector keeps the row (recurrent state) until the pull is done
        else:
            self._release_row(req)
        self._hashes.pop(req.request_id, None)
        self.finished_since_last.append(req.request_id)

    def free_blocks(self, req: Request) -> None:
        self.pool.free(req.block_ids)
        req.block_ids = []

    def finish_decode_fast(self, req: Request, status: RequestStatus) -> None:
        """Used by the vectorised decode loop of the engine."""
        self.running.remove(req)
        self._finish(req, status)
