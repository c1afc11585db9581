"""Request-level data types of the public API (vLLM-compatible names)."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Any, Optional

import numpy as np


@dataclass
class SamplingParams:
    n: int = 1
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0                       # 0 / -1: disabled
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int = 16
    min_tokens: int = 0
    stop_token_ids: Optional[list[int]] = None
    ignore_eos: bool = False
    seed: Optional[int] = None
    logprobs: Optional[int] = None             # log-probabilities of the sampled token and the top-N tokens
    prompt_logprobs: Optional[int] = None      # log-probabilities of the prompt tokens (+ top-N); disables prefix reuse
    logit_bias: Optional[dict] = None          # token id -> additive bias
    allowed_token_ids: Optional[list[int]] = None
    bad_words_token_ids: Optional[list[list[int]]] = None   # token sequences that must not be generated
    guided_decoding: Optional[Any] = None      # sample.guided.GuidedDecodingParams (or a dict of its fields)
    extra_args: Optional[dict] = None

    def __post_init__(self):
        if isinstance(self.guided_decoding, dict):
            from ..sample.guided import GuidedDecodingParams
            self.guided_decoding = GuidedDecodingParams(**self.guided_decoding)
        if self.top_k is None or self.top_k < 0:
            self.top_k = 0
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.max_tokens is not None and self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if not (self.repetition_penalty > 0.0):
            raise ValueError("repetition_penalty must be positive")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError("min_p must be in [0, 1]")
        if self.min_tokens < 0:
            raise ValueError("min_tokens must be non-negative")
        if self.n < 1:
            raise ValueError("n must be at least 1")
        for name in ("logprobs", "prompt_logprobs"):
            v = getattr(self, name)
            if v is not None and int(v) < 0:
                raise ValueError(f"{name} must be non-negative")
        if self.allowed_token_ids is not None:
            ids = [int(t) for t in self.allowed_token_ids]
            if not ids:
                raise ValueError("allowed_token_ids must not be empty")
            if min(ids) < 0:
                raise ValueError("allowed_token_ids must be non-negative")
            self.allowed_token_ids = ids

    def validate_for_vocab(self, vocab_size: int) -> None:
        """Checks that need the model: token ids named by the request exist.  Raises ``ValueError``
        (the HTTP server answers 400) instead of letting an index fault stop the engine later."""
        if self.allowed_token_ids is not None and max(self.allowed_token_ids) >= vocab_size:
            raise ValueError(f"allowed_token_ids holds an id >= vocab size {vocab_size}")
        if self.top_k and self.top_k > vocab_size:
            self.top_k = 0
        for t in self.stop_token_ids or ():
            if not (0 <= int(t) < vocab_size):
                raise ValueError(f"stop_token_ids holds an id outside [0, {vocab_size})")

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-5

    @property
    def has_processors(self) -> bool:
        return bool(self.logit_bias or self.allowed_token_ids or self.bad_words_token_ids or self.min_tokens > 0
                    or self.guided_decoding is not None)

    @property
    def has_penalties(self) -> bool:
        return (self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
                or self.repetition_penalty != 1.0)


class RequestError(RuntimeError):
    """A failure that belongs to one request (malformed parameters discovered while a step is
    built): the serving loop aborts that request and keeps serving the others."""

    def __init__(self, request_id: str, message: str):
        super().__init__(f"request {request_id}: {message}")
        self.request_id = request_id


class RequestStatus(enum.IntEnum):
    WAITING = 0
    WAITING_FOR_REMOTE_KVS = 1
    RUNNING = 2
    PREEMPTED = 3
    FINISHED_STOPPED = 4
    FINISHED_LENGTH = 5
    FINISHED_ABORTED = 6

    @property
    def finished(self) -> bool:
        return self >= RequestStatus.FINISHED_STOPPED


@dataclass
class Request:
    request_id: str
    prompt_token_ids: np.ndarray
    sampling_params: SamplingParams
    eos_token_id: Optional[int] = None
    arrival_time: float = field(default_factory=time.monotonic)
    priority: int = 0
    kv_transfer_params: Optional[dict] = None
    lora_request: Optional[Any] = None
    # ---- engine state ----
    status: RequestStatus = RequestStatus.WAITING
    row: int = -1                         # persistent batch row
    num_computed_tokens: int = 0
    num_output_tokens: int = 0
    block_ids: list = field(default_factory=list)
    num_cached_tokens: int = 0            # prefix-cache hit length
    num_preemptions: int = 0
    output_token_ids: Optional[list[int]] = None
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    spec_token_ids: list = field(default_factory=list)
    num_inflight: int = 0                 # tokens sampled by steps still running on the GPU (async scheduling)
    job_id: Optional[str] = None
    stop_reason: Optional[str] = None      # why a stopped request stopped when it was not a stop token ("recomputed")
    # multimodal: items (placeholder run + pixels), 3-axis rotary positions of the prompt and the
    # offset decoded tokens continue from (position = index + delta)
    pooled: Optional[Any] = None          # final hidden state of the last prompt token (embedding requests)
    guided: Optional[Any] = None          # sample.guided.GuidedState of structured-output requests
    logprobs: Optional[list] = None       # per generated token: {token id: logprob} (sampled + top-N)
    prompt_logprobs: Optional[list] = None    # per prompt token (None for the first): {token id: logprob}
    mm_inputs: list = field(default_factory=list)
    mrope_positions: Optional[np.ndarray] = None
    mrope_delta: int = 0

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        return self.num_prompt_tokens + self.num_output_tokens

    @property
    def is_finished(self) -> bool:
        return self.status.finished


@dataclass
class CompletionOutput:
    index: int
    token_ids: list[int]
    text: str = ""
    finish_reason: Optional[str] = None
    logprobs: Optional[list] = None
    stop_reason: Optional[str] = None


@dataclass
class RequestMetrics:
    arrival_time: float
    first_token_time: Optional[float]
    finish_time: Optional[float]

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token_time is None else self.first_token_time - self.arrival_time

    @property
    def tpot(self) -> Optional[float]:
        return None


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: list[int]
    outputs: list[CompletionOutput]
    finished: bool
    metrics: Optional[RequestMetrics] = None
    kv_transfer_params: Optional[dict] = None
    num_cached_tokens: int = 0
    prompt_logprobs: Optional[list] = None     # [None, {token: logprob, ...}, ...] one entry per prompt token
