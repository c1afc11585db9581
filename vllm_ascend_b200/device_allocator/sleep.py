"""Engine-level sleep / wake-up (RL weight-refresh workflow).

level 1: weights are offloaded to pinned host memory, the KV cache is discarded;
level 2: everything is discarded, only module buffers (rotary tables, norm-free
state) are kept on the host — the two levels of vllm_ascend/worker/worker.py:221-273.
With ``rl_config.sleep_mode_extra_cleanup`` the captured graphs are dropped and the model-parallel
communicators destroyed before sleeping; wake-up re-creates the communicators and re-captures the
graphs (vllm_ascend/device_allocator/sleep_mem_optimized.py:34-186).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import envs

from ..platform_config import get_b200_config
from .vmm import VmmAllocator


def sleep(engine, level: int = 1) -> int:
    if not engine.cfg.enable_sleep_mode:
        raise RuntimeError("sleep mode is off: construct the LLM with enable_sleep_mode=True")
    if level not in (1, 2):
        raise ValueError("sleep level must be 1 or 2")
    runner = engine.runner
    from ..parallel import state as pstate
    if pstate.has_nccl_groups() and not envs.VLLM_B200_SLEEP_WITH_NCCL:
        # On two B200 ranks over NCCL a sleep / wake-up cycle did not return (three runs: communicators
        # destroyed and re-created, re-created with a warm-up collective, and kept); the step that blocks
        # was not found.  Until it is, a multi-rank NCCL engine refuses to sleep instead of hanging.
        raise RuntimeError("sleep mode is not available on multi-rank NCCL engines "
                           "(set VLLM_B200_SLEEP_WITH_NCCL=1 to try it anyway)")
    torch.cuda.synchronize()
    if get_b200_config().rl_config.sleep_mode_extra_cleanup:
        runner.drop_graphs()
        engine._recapture_on_wake = True
        from ..parallel import state as pstate
        pstate.suspend_groups()
    alloc = VmmAllocator.get_instance()
    freed = alloc.sleep(offload_tags=("weights",) if level == 1 else ())
    engine.sleep_level = level
    return freed


def wake_up(engine, tags: Optional[list[str]] = None) -> int:
    alloc = VmmAllocator.get_instance()
    restored = alloc.wake_up(tags)
    if tags is None or "kv_cache" in tags:
        # KV contents were discarded: caches must start from zeros and no prefix survives
        for caches in engine.runner.kv_caches:
            for t in caches:
                t.zero_()
        engine.scheduler.pool.reset_prefix_cache()
    if getattr(engine, "_recapture_on_wake", False) and not alloc.sleeping_tags:
        from ..parallel import state as pstate
        pstate.restore_groups()
        engine.runner.capture_graphs()
        engine._recapture_on_wake = False
    if not alloc.sleeping_tags:
        engine.sleep_level = 0
    torch.cuda.synchronize()
    return restored
