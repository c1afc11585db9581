"""Scheduler extensions (the reference's ``vllm_ascend/core``)."""
from __future__ import annotations


def make_scheduler(engine_cfg, num_blocks: int, kv_connector=None):
    """Scheduler class selection by policy name
    (vllm_ascend/platform.py:1141-1164, 1361-1378)."""
    from ..engine.scheduler import Scheduler
    policy = engine_cfg.scheduler.policy
    cls = Scheduler
    kw = {}
    if policy == "short_request_first":
        from .short_request_first import ShortRequestFirstScheduler as cls
    elif policy == "batch_job":
        from .batch_job_aware import BatchJobAwareScheduler as cls
    elif policy == "recompute":
        from .recompute import RecomputeScheduler as cls
    elif policy == "profiling_chunk":
        from .profiling_chunk import ProfilingChunkScheduler as cls
    elif policy == "balance":
        from .balance import BalanceScheduler as cls
    elif policy == "dyntra_lb":
        from .dyntra_lb import DyntraLBScheduler as cls
    elif policy != "fcfs":
        raise ValueError(f"unknown scheduler policy {policy!r}")
    if cls is not Scheduler:
        kw["engine_cfg"] = engine_cfg
    cache_cfg = engine_cfg.cache
    dcp = engine_cfg.parallel.decode_context_parallel_size
    if dcp > 1:
        # the KV of a sequence is spread over the DCP ranks: one block id covers
        # block_size * dcp tokens, block_size of them on each rank
        import copy
        cache_cfg = copy.copy(cache_cfg)
        cache_cfg.block_size = cache_cfg.block_size * dcp
    return cls(engine_cfg.scheduler, cache_cfg, num_blocks, kv_connector, **kw)
