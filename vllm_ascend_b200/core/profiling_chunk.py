"""Dynamic prefill chunk sizing from a fitted latency model.

Behaviour of vllm_ascend/core/profiling_chunk_predictor.py and
scheduler_profiling_chunk.py: prefill latency is modelled as
f(C, H) = a*C*(C+H) + b*C + c*H (C = chunk tokens, H = already computed tokens of
the sequence; without history this is the quadratic a*l^2 + b*l + c).  Given a
target latency the next chunk size solves a*x^2 + (a*H + b)*x - T = 0, smoothed
with ``smooth_factor`` and clamped to ``[min_chunk, max_num_batched_tokens]``, so
pipeline stages see equal-time chunks on very long prompts.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np

from ..engine.scheduler import Scheduler, SchedulerOutput
from ..platform_config import get_b200_config


class ChunkSizePredictor:
    MIN_FIT_POINTS = 5

    def __init__(self, smooth_factor: float = 0.8, min_chunk: int = 512, max_fit_chunk: int = 30):
        self.smooth = smooth_factor
        self.min_chunk = min_chunk
        self.max_fit_chunk = max_fit_chunk
        self.a = self.b = self.c = 0.0
        self.fitted = False
        self.target_latency: Optional[float] = None
        self.samples: list[tuple[int, int, float]] = []     # (chunk, history, seconds)
        self._last: Optional[float] = None

    def observe(self, chunk: int, history: int, seconds: float) -> None:
        self.samples.append((chunk, history, seconds))
        if len(self.samples) > self.max_fit_chunk:
            self.samples.pop(0)
        if len(self.samples) >= self.MIN_FIT_POINTS:
            self.fit()

    def fit(self) -> bool:
        C = np.array([s[0] for s in self.samples], dtype=np.float64)
        H = np.array([s[1] for s in self.samples], dtype=np.float64)
        T = np.array([s[2] for s in self.samples], dtype=np.float64)
        X = np.column_stack([C * (C + H), C, H])
        try:
            coef, *_ = np.linalg.lstsq(X, T, rcond=None)
        except np.linalg.LinAlgError:
            return False
        a, b, c = (float(x) for x in coef)
        if not all(math.isfinite(v) for v in (a, b, c)) or (a <= 0 and b <= 0):
            return False
        self.a, self.b, self.c = max(a, 0.0), b, c
        self.fitted = True
        return True

    def latency(self, chunk: int, history: int) -> float:
        return self.a * chunk * (chunk + history) + self.b * chunk + self.c * history

    def set_target(self, base_chunk: int, elapsed: float = 0.0) -> None:
        self.target_latency = elapsed if elapsed > 0 else max(self.latency(base_chunk, 0), 1e-6)

    def predict(self, history: int, max_chunk: int) -> int:
        if not self.fitted or not self.target_latency:
            return max_chunk
        a, lin, T = self.a, self.a * history + self.b, self.target_latency
        if a > 1e-18:
            disc = lin * lin + 4 * a * T
            x = (-lin + math.sqrt(max(disc, 0.0))) / (2 * a)
        elif lin > 0:
            x = T / lin
        else:
            x = max_chunk
        if self._last is not None:
            x = self.smooth * x + (1 - self.smooth) * self._last
        self._last = x
        return int(min(max(x, self.min_chunk), max_chunk))


class ProfilingChunkScheduler(Scheduler):
    def __init__(self, sched_cfg, cache_cfg, num_blocks, kv_connector=None, engine_cfg=None):
        super().__init__(sched_cfg, cache_cfg, num_blocks, kv_connector)
        c = get_b200_config().scheduler_config.profiling_chunk_config
        self.predictor = ChunkSizePredictor(c.smooth_factor, c.min_chunk, 30)
        self.base_budget = sched_cfg.max_num_batched_tokens
        self.need_timing = c.need_timing

    def record_step(self, out: SchedulerOutput, seconds: float) -> None:
        """Called by the engine with the measured duration of a prefill-only step."""
        prefills = [(r, n) for r, n in out.scheduled if n > 1]
        if len(prefills) != 1 or len(out.scheduled) != 1:
            return
        r, n = prefills[0]
        self.predictor.observe(n, r.num_computed_tokens - n if r.num_computed_tokens >= n
                               else r.num_computed_tokens, seconds)
        if self.predictor.fitted and self.predictor.target_latency is None:
            self.predictor.set_target(self.base_budget)

    def schedule(self) -> SchedulerOutput:
        # budget for this step: equal-latency chunk of the longest running prefill
        longest = None
        for r in list(self.running) + list(self.waiting)[:1]:
            if r.num_computed_tokens < r.num_prompt_tokens:
                if longest is None or r.num_computed_tokens > longest.num_computed_tokens:
                    longest = r
        saved = self.cfg.max_num_batched_tokens
        if longest is not None and self.predictor.fitted:
            self.cfg.max_num_batched_tokens = self.predictor.predict(longest.num_computed_tokens,
                                                                     self.base_budget)
        try:
            return super().schedule()
        finally:
            self.cfg.max_num_batched_tokens = saved
