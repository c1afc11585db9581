"""Dynamic speculation length: how many draft tokens a request gets follows how many it has been
getting accepted.

Every verification updates the request's running acceptance estimate (accepted / drafted, exponential
moving average); the next draft budget is the number of leading tokens whose joint acceptance
probability stays above ``budget_threshold`` (a geometric model: p^k >= threshold), at least
``min_tokens``, at most the configured maximum.  A request whose drafts keep failing stops paying for
them; one whose drafts always pass uses the full budget.  Counterpart of the reference's dynamic
speculative-length scheduling (``dynamic_spec_config``, vllm_ascend/spec_decode/utils.py
DynamicSpecScheduler), which takes the per-token confidence from a trained head where this uses the
measured acceptance.

``VerifyBudgetAllocator`` is the batch half of that scheduling: from acceptance probabilities per
(request, draft position) it forms the survival probability of every draft prefix, keeps a shared
budget of verify tokens per request that is re-estimated every few steps (mean number of positions
whose survival exceeds the threshold, rounded up, bumped to an odd number because the verify width
includes the bonus token), and hands the batch's budget to the positions with the highest survival
anywhere in the batch; since survival falls along a request, what a request receives is a prefix
length.  Every request keeps at least ``min_verify_tokens``
(vllm_ascend/spec_decode/utils.py:211-560).  Proposers that know a confidence per draft token (the
probability of the token a draft model picked) pass it in; for the others the controller's
per-request acceptance estimate stands in for every position.
"""
from __future__ import annotations

import math

import numpy as np


class VerifyBudgetAllocator:
    def __init__(self, num_speculative_tokens: int, params: dict | None = None):
        p = dict(params or {})
        self.D = int(num_speculative_tokens)
        self.threshold = float(p.get("budget_threshold", 0.3))
        self.interval = int(p.get("budget_update_interval", 16))
        self.min_k = max(0, min(int(p.get("min_verify_tokens", p.get("min_tokens", 1))), self.D))
        self.budget_k = max(self.min_k, min(int(p.get("initial_verify_budget_per_req", 5)), self.D))
        self._steps = 0

    def _update_budget(self, survival: np.ndarray) -> None:
        self._steps += 1
        if self._steps < self.interval or survival.shape[0] == 0:
            return
        self._steps = 0
        k = math.ceil(float((survival >= self.threshold).sum()) / survival.shape[0])
        if k % 2 == 0 and k < self.D:
            k += 1
        self.budget_k = max(self.min_k, min(k, self.D))

    def allocate(self, token_probs: np.ndarray) -> np.ndarray:
        """``token_probs`` [B, D]: P(draft token i accepted | the ones before it were).  Returns the
        number of draft tokens to verify per request, [B] int."""
        probs = np.clip(np.asarray(token_probs, dtype=np.float64), 1e-6, 1.0)
        B, D = probs.shape
        survival = np.cumprod(probs, axis=1)
        self._update_budget(survival)
        lens = np.full(B, min(self.min_k, D), dtype=np.int64)
        extra = max(self.budget_k - self.min_k, 0) * B
        cand = survival[:, self.min_k:]
        if extra <= 0 or cand.size == 0:
            return lens
        extra = min(extra, cand.size)
        flat = cand.reshape(-1)
        # the `extra` largest survival values of the batch; ties go to the earlier position, so a
        # request's picks stay a prefix
        order = np.argsort(-flat, kind="stable")[:extra]
        np.add.at(lens, order // cand.shape[1], 1)
        return lens


class DynamicSpecController:
    def __init__(self, max_tokens: int, params: dict | None = None):
        p = dict(params or {})
        self.max_tokens = max_tokens
        self.min_tokens = int(p.get("min_tokens", 1))
        self.threshold = float(p.get("budget_threshold", 0.3))
        self.alpha = float(p.get("ema_alpha", 0.3))
        self.initial = float(p.get("initial_acceptance", 0.7))
        self.rate: dict[str, float] = {}
        self.allocator = VerifyBudgetAllocator(max_tokens, p) if p.get("shared_budget", False) else None

    def update(self, request_id: str, drafted: int, accepted: int) -> None:
        if drafted <= 0:
            return
        r = self.rate.get(request_id, self.initial)
        self.rate[request_id] = (1 - self.alpha) * r + self.alpha * (accepted / drafted)

    def budget(self, request_id: str) -> int:
        p = min(max(self.rate.get(request_id, self.initial), 1e-3), 0.999)
        k = int(math.floor(math.log(self.threshold) / math.log(p)))
        return max(self.min_tokens, min(self.max_tokens, k))

    def budgets(self, request_ids: list[str], token_probs=None) -> list[int]:
        """Draft budgets of one propose step.  Per request from its own estimate, or, with
        ``shared_budget``, from the batch allocation over ``token_probs`` [B, D] (the controller's
        estimates when the proposer has no confidences)."""
        if self.allocator is None:
            return [self.budget(r) for r in request_ids]
        if token_probs is None:
            rates = np.array([self.rate.get(r, self.initial) for r in request_ids], dtype=np.float64)
            token_probs = np.repeat(rates[:, None], self.max_tokens, axis=1)
        return [int(x) for x in self.allocator.allocate(token_probs)]

    def forget(self, request_id: str) -> None:
        self.rate.pop(request_id, None)
