"""Dynamic prefill chunk sizing from a fitted latency model.

Behaviour of vllm_ascend/core/profiling_chunk_predictor.py and
scheduler_profiling_chunk.py: prefill latency is modelled as
f(C, H) = a*C*(C+H) + b*C + c*H + d (C = chunk tokens, H = already computed tokens of
the sequence; without history this is the quadratic a*l^2 + b*l + d), summed over the requests
of a step.  The model is fitted once at start-up from timed dummy prefills of decreasing size
and refined online from the measured duration of every step that contains prefill work.  Given a
target latency the next chunk size solves a*x^2 + (a*H + b)*x - T = 0, smoothed
with ``smooth_factor`` and clamped to ``[min_chunk, max_num_batched_tokens]``, so
pipeline stages see equal-time chunks on very long prompts.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np

from ..engine.scheduler import Scheduler, SchedulerOutput
from ..logger import logger
from ..platform_config import get_b200_config


class ChunkSizePredictor:
    """Step latency T = a * sum C(C+H) + b * sum C + c * sum H + d over the requests of a step
    (C new tokens, H tokens already in the cache), least-squares fitted."""
    MIN_FIT_POINTS = 5

    def __init__(self, smooth_factor: float = 0.8, min_chunk: int = 512, max_fit_chunk: int = 30):
        self.smooth = smooth_factor
        self.min_chunk = min_chunk
        self.max_fit_chunk = max_fit_chunk
        self.a = self.b = self.c = self.d = 0.0
        self.fitted = False
        self.target_latency: Optional[float] = None
        self.samples: list[tuple[float, float, float, float]] = []     # (sum C(C+H), sum C, sum H, seconds)
        self._last: Optional[float] = None

    def observe(self, chunk: int, history: int, seconds: float) -> None:
        self.observe_batch([(chunk, history)], seconds)

    def observe_batch(self, chunks: list[tuple[int, int]], seconds: float) -> None:
        """``chunks``: (new tokens, cached tokens) of every request of one step."""
        x1 = float(sum(c * (c + h) for c, h in chunks))
        x2 = float(sum(c for c, _ in chunks))
        x3 = float(sum(h for _, h in chunks))
        self.samples.append((x1, x2, x3, float(seconds)))
        if len(self.samples) > self.max_fit_chunk:
            self.samples.pop(0)
        if len(self.samples) >= self.MIN_FIT_POINTS:
            self.fit()

    def fit(self) -> bool:
        S = np.array(self.samples, dtype=np.float64)
        cols = [S[:, 0], S[:, 1]]
        use_hist = bool(np.ptp(S[:, 2]) > 0)           # history never varied: its column is not identifiable
        if use_hist:
            cols.append(S[:, 2])
        cols.append(np.ones(len(S)))
        X = np.column_stack(cols)
        scale = np.maximum(np.abs(X).max(axis=0), 1e-30)       # columns differ by ten orders of magnitude
        try:
            coef, *_ = np.linalg.lstsq(X / scale, S[:, 3], rcond=None)
        except np.linalg.LinAlgError:
            return False
        coef = coef / scale
        a, b = float(coef[0]), float(coef[1])
        c = float(coef[2]) if use_hist else 0.0
        d = float(coef[-1])
        if not all(math.isfinite(v) for v in (a, b, c, d)) or (a <= 0 and b <= 0):
            return False
        lo, hi = float(S[:, 1].min()), float(S[:, 1].max())
        if hi > lo and a * hi * hi + b * hi <= a * lo * lo + b * lo:
            return False                    # latency must grow with the amount of work
        self.a, self.b, self.c, self.d = max(a, 0.0), max(b, 0.0), max(c, 0.0), max(d, 0.0)
        self.fitted = True
        return True

    def latency(self, chunk: int, history: int) -> float:
        return self.a * chunk * (chunk + history) + self.b * chunk + self.c * history + self.d

    def set_target(self, base_chunk: int, elapsed: float = 0.0) -> None:
        self.target_latency = elapsed if elapsed > 0 else max(self.latency(base_chunk, 0), 1e-6)

    def predict(self, history: int, max_chunk: int) -> int:
        if not self.fitted or not self.target_latency:
            return max_chunk
        a, lin = self.a, self.a * history + self.b
        T = self.target_latency - self.d - self.c * history
        if T <= 0:
            x = float(self.min_chunk)
        elif a > 1e-18:
            disc = lin * lin + 4 * a * T
            x = (-lin + math.sqrt(max(disc, 0.0))) / (2 * a)
        elif lin > 0:
            x = T / lin
        else:
            x = max_chunk
        if self._last is not None:
            x = self.smooth * x + (1 - self.smooth) * self._last
        self._last = x
        return int(round(min(max(x, self.min_chunk), max_chunk)))


class ProfilingChunkScheduler(Scheduler):
    PROFILE_SAMPLES = 16

    def __init__(self, sched_cfg, cache_cfg, num_blocks, kv_connector=None, engine_cfg=None):
        super().__init__(sched_cfg, cache_cfg, num_blocks, kv_connector)
        c = get_b200_config().scheduler_config.profiling_chunk_config
        self.predictor = ChunkSizePredictor(c.smooth_factor, c.min_chunk, 64)
        self.base_budget = sched_cfg.max_num_batched_tokens
        self.need_timing = c.need_timing
        self.profiled = False

    def run_profiling(self, profile_fn, num_samples: Optional[int] = None) -> bool:
        """Start-up profiling: ``profile_fn(num_tokens) -> seconds`` runs one prefill-shaped forward
        of that many tokens.  Chunk sizes step down from the token budget; the first call is a
        warm-up.  Fits the model without history and sets the latency target to that of a
        full-budget chunk; online samples (``record_step``) add the history terms later.  Runs once
        (vllm_ascend/core/scheduler_profiling_chunk.py:109-203)."""
        if self.profiled:
            return self.predictor.fitted
        self.profiled = True
        if profile_fn is None:
            logger.warning("profiling chunk: no executor to profile with; chunk sizes stay fixed until "
                           "online samples arrive")
            return False
        n = num_samples or self.PROFILE_SAMPLES
        got = 0
        for i in range(n + 1):
            chunk = int(self.base_budget - max(i - 1, 0) * (self.base_budget / n))
            if chunk <= 0:
                break
            try:
                sec = profile_fn(chunk)
            except Exception as e:          # a size the model cannot run (e.g. beyond its context)
                logger.debug("profiling chunk: forward of %d tokens failed: %s", chunk, e)
                continue
            if i == 0 or sec is None or sec <= 0:
                continue
            self.predictor.samples.append((float(chunk) * chunk, float(chunk), 0.0, float(sec)))
            got += 1
        if got < min(8, n) or not self.predictor.fit():
            logger.warning("profiling chunk: start-up profiling gave %d usable samples; not fitted", got)
            self.predictor.samples.clear()
            return False
        self.predictor.set_target(self.base_budget)
        logger.info("profiling chunk: fitted a=%.3e b=%.3e d=%.3e, target %.2f ms for %d tokens",
                    self.predictor.a, self.predictor.b, self.predictor.d, self.predictor.target_latency * 1e3,
                    self.base_budget)
        return True

    def record_step(self, out: SchedulerOutput, seconds: float) -> None:
        """Called by the engine with the measured duration of a step that contained prefill work."""
        chunks = []
        for r, n in out.scheduled:
            done = r.num_computed_tokens                # already advanced by this step
            chunks.append((n, max(done - n, 0)))
        if not chunks or not any(n > 1 for n, _ in chunks):
            return
        self.predictor.observe_batch(chunks, seconds)
        if self.predictor.fitted and self.predictor.target_latency is None:
            self.predictor.set_target(self.base_budget)

    def schedule(self) -> SchedulerOutput:
        # budget for this step: equal-latency chunk of the longest running prefill
        longest = None
        head = [self.waiting[0]] if self.waiting else []
        for r in list(self.running) + head:
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
