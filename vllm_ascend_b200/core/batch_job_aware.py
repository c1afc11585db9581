"""Batch-job-aware scheduler for offline throughput.

Behaviour of vllm_ascend/core/batch_job_aware_scheduler.py: requests carry a job
name (``Request.job_id`` or a ``#job_name[NAME]#`` prefix of the request id); the
decode length of each job is estimated with an EWMA (alpha 0.1, cold start 128);
jobs with long predicted decodes are admitted first while KV space is plentiful
(longest-processing-time first) and short ones when it is scarce; admission keeps
a reserve of KV blocks for the predicted growth of the running set so running
requests are not preempted.
"""
from __future__ import annotations

import re
from collections import defaultdict
from typing import Optional

from ..engine.request import Request, RequestStatus
from ..engine.scheduler import Scheduler
from ..platform_config import get_b200_config

_JOB_RE = re.compile(r"#job_name\[(.*?)\]#")


def parse_job_name(req: Request) -> str:
    if req.job_id:
        return req.job_id
    m = _JOB_RE.search(req.request_id)
    return m.group(1) if m else "_default"


class JobDecodeEstimator:
    COLD_START_DEFAULT = 128
    ALPHA = 0.1

    def __init__(self):
        self.ewma: dict[str, float] = {}
        self.samples: dict[str, int] = defaultdict(int)

    def predict(self, job: str) -> int:
        return int(round(self.ewma.get(job, self.COLD_START_DEFAULT)))

    def observe(self, job: str, decode_len: int) -> None:
        if job not in self.ewma:
            self.ewma[job] = float(decode_len)
        else:
            self.ewma[job] = self.ALPHA * decode_len + (1 - self.ALPHA) * self.ewma[job]
        self.samples[job] += 1


class BatchJobAwareScheduler(Scheduler):
    SHORT_DECODE_THRESHOLD = 32
    PLENTY_TOKENS_THRESHOLD = 4096
    COLD_START_SAMPLES = 2

    def __init__(self, sched_cfg, cache_cfg, num_blocks, kv_connector=None, engine_cfg=None):
        super().__init__(sched_cfg, cache_cfg, num_blocks, kv_connector)
        c = get_b200_config().scheduler_config.batch_job_sched_config
        self.max_jobs = c.max_jobs
        self.reserve_margin_blocks = c.reserve_margin_blocks
        self.reserve_max_blocks = c.reserve_max_blocks
        self.estimator = JobDecodeEstimator()
        self._inflight_cold: dict[str, int] = defaultdict(int)

    # -- reserve: blocks the running set is predicted to need before it finishes a block
    def predicted_reserve(self) -> int:
        need = 0
        bs = self.block_size
        for r in self.running:
            job = parse_job_name(r)
            remaining = max(0, min(self.estimator.predict(job), r.sampling_params.max_tokens)
                            - r.num_output_tokens)
            final_tokens = r.num_tokens + remaining
            need += max(0, (final_tokens + bs - 1) // bs - len(r.block_ids))
        need += self.reserve_margin_blocks
        if self.reserve_max_blocks > 0:
            need = min(need, self.reserve_max_blocks)
        return need

    def _can_admit(self, req: Request, num_new_blocks: int) -> bool:
        if not self.running:
            return self.pool.can_allocate(num_new_blocks)
        return self.pool.num_free_blocks - self.predicted_reserve() >= num_new_blocks

    def _pick_waiting(self) -> Optional[Request]:
        if not self.waiting:
            return None
        # preempted requests resume first
        for r in self.waiting:
            if r.status == RequestStatus.PREEMPTED:
                return r
        by_job: dict[str, list[Request]] = defaultdict(list)
        for r in self.waiting:
            by_job[parse_job_name(r)].append(r)
        # cold-start: sample every job's decode length early
        for job, rs in by_job.items():
            if self.estimator.samples[job] + self._inflight_cold[job] < self.COLD_START_SAMPLES:
                return rs[0]
        free_tokens = (self.pool.num_free_blocks - self.predicted_reserve()) * self.block_size
        jobs = sorted(by_job, key=lambda j: self.estimator.predict(j))
        long_jobs = [j for j in jobs if self.estimator.predict(j) >= self.SHORT_DECODE_THRESHOLD]
        short_jobs = [j for j in jobs if self.estimator.predict(j) < self.SHORT_DECODE_THRESHOLD]
        if free_tokens > self.PLENTY_TOKENS_THRESHOLD:
            order = list(reversed(long_jobs)) + short_jobs      # longest decode first
        else:
            order = short_jobs + long_jobs                      # shortest decode first
        job = order[0]
        # best fit by prefill length inside the job: the longest prompt that fits the budget
        budget = max(free_tokens, 0)
        fitting = [r for r in by_job[job] if r.num_prompt_tokens <= budget]
        pool = fitting or by_job[job]
        return max(pool, key=lambda r: r.num_prompt_tokens) if fitting else min(
            pool, key=lambda r: r.num_prompt_tokens)

    def _pop_waiting(self, req: Request) -> None:
        super()._pop_waiting(req)
        job = parse_job_name(req)
        if self.estimator.samples[job] < self.COLD_START_SAMPLES:
            self._inflight_cold[job] += 1

    def _finish(self, req: Request, status) -> None:
        job = parse_job_name(req)
        if status in (RequestStatus.FINISHED_STOPPED, RequestStatus.FINISHED_LENGTH):
            self.estimator.observe(job, req.num_output_tokens)
        if self._inflight_cold[job] > 0:
            self._inflight_cold[job] -= 1
        super()._finish(req, status)
