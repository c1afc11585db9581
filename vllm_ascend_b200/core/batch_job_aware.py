"""Batch-job-aware scheduler for offline throughput.

Offline workloads arrive as *jobs*: thousands of requests that share a prompt template and
therefore a typical output length.  This scheduler learns that length per job and uses it to
order admissions so that the KV pool stays full without preempting running requests.

Pieces (behaviour of vllm_ascend/core/batch_job_aware_scheduler.py:57-660):

* ``JobNameParser``: the job of a request is ``Request.job_id`` or a ``#job_name[NAME]#`` tag in
  its request id (``_default`` otherwise); parsed once per request id.
* ``JobDecodeEstimator``: EWMA (alpha 0.1) of the observed decode lengths per job, 128 before the
  first sample, frozen after ``max_samples`` observations; at most ``max_jobs`` jobs (0 = no limit).
* ``BlockReserve``: KV blocks the running set will ask for in the step after the one being
  scheduled (a request still in prefill takes another chunk, a decoding one crosses a block
  boundary or not), plus a margin, capped.  Summed once per scheduling step and extended by one
  request at a time while the admission loop runs.
* ``LengthBuckets``: the waiting requests of one job keyed by prompt length; "longest prompt that
  fits N tokens" is one bisection.
* ``JobQueue``: the waiting queue.  Preempted requests resume first; then the first few requests
  of every job (cold start: they produce the samples the estimator needs); then jobs ordered by
  predicted decode length: long decodes first while more than ``low_available_tokens_threshold``
  tokens of KV are free (they are the ones that must overlap with everything else to finish in
  time), short decodes first when space is scarce (they return their blocks soonest).  Inside a
  job the longest prompt that fits the free space goes first.  The queue offers the deque
  interface the base scheduler uses, every operation in O(log n) or better, so a job of 100 000
  queued requests costs no more per step than ten.
"""
from __future__ import annotations

import bisect
import re
from collections import OrderedDict, deque
from typing import Iterator, Optional

from ..engine.request import Request, RequestStatus
from ..engine.scheduler import Scheduler
from ..platform_config import get_b200_config

_JOB_RE = re.compile(r"#job_name\[(.*?)\]#")
DEFAULT_JOB = "_default"


def _cdiv(a: int, b: int) -> int:
    return -(-a // b)


class JobNameParser:
    def __init__(self):
        self._cache: dict[str, str] = {}

    def parse(self, req_or_id) -> str:
        if isinstance(req_or_id, Request):
            if req_or_id.job_id:
                return req_or_id.job_id
            rid = req_or_id.request_id
        else:
            rid = req_or_id
        job = self._cache.get(rid)
        if job is None:
            m = _JOB_RE.search(rid)
            job = (m.group(1) if m else "") or DEFAULT_JOB
            self._cache[rid] = job
        return job

    def remove(self, request_id: str) -> None:
        self._cache.pop(request_id, None)

    def clear(self) -> None:
        self._cache.clear()

    def __len__(self) -> int:
        return len(self._cache)


def parse_job_name(req: Request) -> str:
    """Job of one request without a cache (helpers and tests)."""
    return JobNameParser().parse(req)


class JobDecodeEstimator:
    COLD_START_DEFAULT = 128
    ALPHA = 0.1

    def __init__(self, max_jobs: int = 0, max_samples: int = 10):
        self.max_jobs, self.max_samples = int(max_jobs), int(max_samples)
        self._mean: dict[str, float] = {}
        self._count: dict[str, int] = {}

    def predict(self, job: str) -> int:
        m = self._mean.get(job)
        return self.COLD_START_DEFAULT if m is None else int(m)

    def samples(self, job: str) -> int:
        return self._count.get(job, 0)

    def observe(self, job: str, decode_len: int) -> None:
        n = self._count.get(job)
        if n is None:
            if self.max_jobs and len(self._count) >= self.max_jobs:
                raise RuntimeError(f"batch-job scheduler: more than max_jobs={self.max_jobs} jobs "
                                   f"(new job {job!r}; known: {sorted(self._count)})")
            n = 0
        if self.max_samples and n >= self.max_samples:
            return
        self._count[job] = n + 1
        self._mean[job] = float(decode_len) if n == 0 else \
            self.ALPHA * decode_len + (1 - self.ALPHA) * self._mean[job]

    def get_stats(self) -> dict[str, dict]:
        return {j: {"samples": self._count[j], "predicted_decode": int(self._mean[j]),
                    "ewma": round(self._mean[j], 2)} for j in self._count}


class BlockReserve:
    """Blocks the running requests will need in the step after this one (see the module text)."""

    def __init__(self, scheduler: Scheduler, margin_blocks: int, max_blocks: int):
        self.s = scheduler
        self.margin, self.cap = int(margin_blocks), int(max_blocks)
        self._sum = 0
        self._n = -1            # running-set size the sum stands for; -1 = stale

    def invalidate(self) -> None:
        self._n = -1

    def one(self, r: Request) -> int:
        bs = self.s.block_size
        chunk = self.s.cfg.max_num_batched_tokens
        decode_step = 1 + self.s.spec_slack
        done, prompt = r.num_computed_tokens, r.num_prompt_tokens
        this_step = min(prompt - done, chunk) if done < prompt else decode_step
        after = done + this_step
        next_step = min(prompt - after, chunk) if after < prompt else decode_step
        room = (bs - after % bs) % bs           # free slots in the last block after this step
        return _cdiv(next_step - room, bs) if next_step > room else 0

    def predict(self) -> int:
        n = len(self.s.running)
        if n == self._n:
            pass
        elif self._n >= 0 and n == self._n + 1:
            self._sum += self.one(self.s.running[-1])
            self._n = n
        else:
            self._sum = sum(self.one(r) for r in self.s.running)
            self._n = n
        total = self._sum + self.margin
        return min(total, self.cap) if self.cap > 0 else total


class LengthBuckets:
    """Requests keyed by prompt length; FIFO among equal lengths."""

    def __init__(self):
        self._by_len: dict[int, "OrderedDict[str, Request]"] = {}
        self._lens: list[int] = []          # sorted, one entry per non-empty bucket
        self._n = 0

    def put(self, req: Optional[Request]) -> None:
        if req is None:
            return
        L = req.num_prompt_tokens
        b = self._by_len.get(L)
        if b is None:
            b = self._by_len[L] = OrderedDict()
            bisect.insort(self._lens, L)
        if req.request_id not in b:
            b[req.request_id] = req
            self._n += 1

    def remove(self, req: Optional[Request]) -> bool:
        if req is None:
            return False
        L = req.num_prompt_tokens
        b = self._by_len.get(L)
        if b is None or b.pop(req.request_id, None) is None:
            return False
        self._n -= 1
        if not b:
            del self._by_len[L]
            self._lens.pop(bisect.bisect_left(self._lens, L))
        return True

    def peek_best_fit(self, limit: int) -> Optional[Request]:
        """Oldest request of the greatest prompt length <= ``limit``."""
        i = bisect.bisect_right(self._lens, limit)
        if i == 0:
            return None
        return next(iter(self._by_len[self._lens[i - 1]].values()))

    def peek_shortest(self) -> Optional[Request]:
        return next(iter(self._by_len[self._lens[0]].values())) if self._lens else None

    def __len__(self) -> int:
        return self._n

    def __bool__(self) -> bool:
        return self._n > 0

    def __iter__(self) -> Iterator[Request]:
        for L in self._lens:
            yield from self._by_len[L].values()


class JobQueue:
    """Waiting queue of the batch-job scheduler (deque interface of the base scheduler)."""

    def __init__(self, scheduler: Scheduler, estimator: JobDecodeEstimator, reserve: BlockReserve,
                 parser: JobNameParser, cfg):
        self.s, self.est, self.reserve, self.parser, self.cfg = scheduler, estimator, reserve, parser, cfg
        self.jobs: dict[str, LengthBuckets] = {}
        self.front: deque[Request] = deque()                  # preempted / rotated: served in order, first
        self.cold: dict[str, "OrderedDict[str, Request]"] = {}   # first requests of each job
        self.seen: dict[str, int] = {}                         # requests ever queued per job
        self._n = 0

    # ---- deque interface
    def append(self, req: Optional[Request]) -> None:
        if req is None:
            return
        if req.status in (RequestStatus.PREEMPTED, RequestStatus.WAITING_FOR_REMOTE_KVS) or req.block_ids:
            self.front.append(req)            # holds state already: not subject to job ordering
            self._n += 1
            return
        job = self.parser.parse(req)
        b = self.jobs.get(job)
        if b is None:
            if self.cfg.max_jobs and len(self.jobs) >= self.cfg.max_jobs:
                raise RuntimeError(f"batch-job scheduler: more than max_jobs={self.cfg.max_jobs} jobs "
                                   f"(new job {job!r})")
            b = self.jobs[job] = LengthBuckets()
        before = len(b)
        b.put(req)
        if len(b) == before:
            return
        self._n += 1
        self.seen[job] = self.seen.get(job, 0) + 1
        if self.seen[job] <= self.cfg.cold_start_requests:
            self.cold.setdefault(job, OrderedDict())[req.request_id] = req

    def appendleft(self, req: Request) -> None:
        self.front.appendleft(req)
        self._n += 1

    def extendleft(self, reqs) -> None:
        for r in reqs:
            self.appendleft(r)

    def remove(self, req: Optional[Request]) -> None:
        if req is None:
            return
        try:
            self.front.remove(req)
            self._n -= 1
            return
        except ValueError:
            pass
        job = self.parser.parse(req)
        b = self.jobs.get(job)
        if b is None or not b.remove(req):
            raise ValueError("request is not queued")
        self._n -= 1
        if not b:
            del self.jobs[job]
        c = self.cold.get(job)
        if c is not None:
            c.pop(req.request_id, None)
            if not c:
                del self.cold[job]

    def popleft(self) -> Request:
        req = self.peek(force=True)
        if req is None:
            raise IndexError("pop from an empty queue")
        self.remove(req)
        return req

    def __getitem__(self, i: int) -> Request:
        if i != 0:
            raise IndexError("only the head of the job queue is addressable")
        req = self.peek(force=True)
        if req is None:
            raise IndexError("empty queue")
        return req

    def __contains__(self, req) -> bool:
        if req in self.front:
            return True
        b = self.jobs.get(self.parser.parse(req))
        return b is not None and any(r is req for r in b._by_len.get(req.num_prompt_tokens, {}).values())

    def __len__(self) -> int:
        return self._n

    def __bool__(self) -> bool:
        return self._n > 0

    def __iter__(self) -> Iterator[Request]:
        yield from self.front
        for b in self.jobs.values():
            yield from b

    # ---- policy
    def admission_budget(self) -> int:
        """Tokens of KV that may be handed to new requests right now."""
        free = self.s.pool.num_free_blocks - self.reserve.predict()
        return max(0, free * self.s.block_size)

    def cold_start_request(self) -> Optional[Request]:
        for c in self.cold.values():
            for r in c.values():
                return r
        return None

    def classify_jobs(self) -> tuple[list[tuple[str, int]], list[tuple[str, int]]]:
        long_, short = [], []
        for job, b in self.jobs.items():
            if b:
                d = self.est.predict(job)
                (long_ if d > self.cfg.short_decode_token_threshold else short).append((job, d))
        return long_, short

    def sort_jobs(self, budget: int, long_: list, short: list) -> list[tuple[str, int]]:
        prefer_long = budget > self.cfg.low_available_tokens_threshold
        if long_ and short:
            long_ = sorted(long_, key=lambda x: -x[1])
            short = sorted(short, key=lambda x: -x[1])
            return long_ + short if prefer_long else short + long_
        key = (lambda x: -x[1]) if prefer_long else (lambda x: x[1])
        return sorted(long_, key=key) + sorted(short, key=key)

    def peek(self, force: bool = False) -> Optional[Request]:
        """The request to admit next, or None when nothing fits the budget.  ``force``: the caller
        needs *some* head (an idle engine must make progress): the shortest prompt of the first job."""
        if self.front:
            return self.front[0]
        budget = self.admission_budget()
        if budget > 0 or force or not self.s.running:
            r = self.cold_start_request()
            if r is not None:
                return r
            long_, short = self.classify_jobs()
            order = self.sort_jobs(budget, long_, short)
            for job, _ in order:
                r = self.jobs[job].peek_best_fit(budget)
                if r is not None:
                    return r
            if (force or not self.s.running) and order:
                return self.jobs[order[0][0]].peek_shortest()
        return None


class BatchJobAwareScheduler(Scheduler):
    def __init__(self, sched_cfg, cache_cfg, num_blocks, kv_connector=None, engine_cfg=None):
        super().__init__(sched_cfg, cache_cfg, num_blocks, kv_connector)
        c = get_b200_config().scheduler_config.batch_job_sched_config
        self.job_cfg = c
        self.parser = JobNameParser()
        self.estimator = JobDecodeEstimator(c.max_jobs, c.max_samples_per_job)
        self.block_reserve = BlockReserve(self, c.reserve_margin_blocks, c.reserve_max_blocks)
        queued = list(self.waiting)
        self.waiting = JobQueue(self, self.estimator, self.block_reserve, self.parser, c)
        for r in queued:
            self.waiting.append(r)

    def schedule(self):
        self.block_reserve.invalidate()
        return super().schedule()

    def predicted_reserve(self) -> int:
        return self.block_reserve.predict()

    def _pick_waiting(self) -> Optional[Request]:
        return self.waiting.peek()

    def _pop_waiting(self, req: Request) -> None:
        self.waiting.remove(req)

    def _can_admit(self, req: Request, num_new_blocks: int) -> bool:
        if not super()._can_admit(req, num_new_blocks):
            return False
        if not self.running or req.block_ids:
            return True
        return self.pool.num_free_blocks - self.block_reserve.predict() >= num_new_blocks

    def _finish(self, req: Request, status) -> None:
        if status in (RequestStatus.FINISHED_STOPPED, RequestStatus.FINISHED_LENGTH):
            self.estimator.observe(self.parser.parse(req), req.num_output_tokens)
        self.parser.remove(req.request_id)
        super()._finish(req, status)

    def job_stats(self) -> dict:
        return self.estimator.get_stats()
