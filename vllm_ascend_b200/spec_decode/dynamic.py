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
"""
from __future__ import annotations

import math


class DynamicSpecController:
    def __init__(self, max_tokens: int, params: dict | None = None):
        p = dict(params or {})
        self.max_tokens = max_tokens
        self.min_tokens = int(p.get("min_tokens", 1))
        self.threshold = float(p.get("budget_threshold", 0.3))
        self.alpha = float(p.get("ema_alpha", 0.3))
        self.initial = float(p.get("initial_acceptance", 0.7))
        self.rate: dict[str, float] = {}

    def update(self, request_id: str, drafted: int, accepted: int) -> None:
        if drafted <= 0:
            return
        r = self.rate.get(request_id, self.initial)
        self.rate[request_id] = (1 - self.alpha) * r + self.alpha * (accepted / drafted)

    def budget(self, request_id: str) -> int:
        p = min(max(self.rate.get(request_id, self.initial), 1e-3), 0.999)
        k = int(math.floor(math.log(self.threshold) / math.log(p)))
        return max(self.min_tokens, min(self.max_tokens, k))

    def forget(self, request_id: str) -> None:
        self.rate.pop(request_id, None)
