"""Sampler: penalties -> temperature -> top-k/top-p/min-p -> exponential race;
greedy rows take argmax.  Order and semantics follow
vllm_ascend/sample/sampler.py:47-159 (and the upstream Sampler flow it extends).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import hashlib

import numpy as np
import torch

from .. import ops


def request_seed(req, base_seed: int = 0) -> int:
    """Seed of a request's random stream.  A request that names a seed uses it; otherwise the seed is
    a digest of (engine seed, request id) that is the same in every process: tensor- and
    expert-parallel ranks sample independently from identical logits and must draw identical tokens
    (Python's ``hash`` of a string differs from process to process)."""
    sp = req.sampling_params
    if sp.seed is not None:
        return int(sp.seed) & ((1 << 62) - 1)
    s = getattr(req, "_sample_seed", None)
    if s is None:
        h = hashlib.blake2b(f"{int(base_seed)}/{req.request_id}".encode(), digest_size=8).digest()
        s = int.from_bytes(h, "little") & ((1 << 62) - 1)
        try:
            req._sample_seed = s
        except AttributeError:
            pass
    return s


def tokens_sampled_so_far(req) -> int:
    """Position of the next token in the request's random stream: tokens already received plus the
    ones sampled by steps still running on the GPU (asynchronous scheduling builds step N+1 before
    step N's token is read back)."""
    return int(req.num_output_tokens) + int(getattr(req, "num_inflight", 0))


@dataclass
class SamplingMetadata:
    all_greedy: bool
    temperature: Optional[torch.Tensor] = None     # fp32 [B]
    top_k: Optional[torch.Tensor] = None           # int32 [B]
    top_p: Optional[torch.Tensor] = None           # fp32 [B]
    min_p: Optional[torch.Tensor] = None           # fp32 [B]
    seeds: Optional[torch.Tensor] = None           # int64 [B] (bit pattern of uint64)
    offsets: Optional[torch.Tensor] = None         # int64 [B]
    has_penalties: bool = False
    prompt_ids: Optional[torch.Tensor] = None      # int64 [B, Lp] padded with vocab_size
    output_ids: Optional[torch.Tensor] = None      # int64 [B, Lo] padded with vocab_size
    repetition_penalty: Optional[torch.Tensor] = None
    frequency_penalty: Optional[torch.Tensor] = None
    presence_penalty: Optional[torch.Tensor] = None
    generator: Optional[torch.Generator] = None    # CPU path only
    allowed_mask: Optional[torch.Tensor] = None    # bool [B, V] (allowed_token_ids / guided decoding)
    bias_index: Optional[torch.Tensor] = None      # int64 [2, n] (row, token) of additive biases
    bias_values: Optional[torch.Tensor] = None     # fp32 [n]
    ban_index: Optional[torch.Tensor] = None       # int64 [2, n] (row, token) forced to -inf

    @staticmethod
    def build(reqs: list, device, vocab_size: int, base_seed: int = 0) -> "SamplingMetadata":
        sps = [r.sampling_params for r in reqs]
        proc = _build_processors(reqs, device, vocab_size) if any(sp.has_processors for sp in sps) else {}
        if all(sp.greedy and not sp.has_penalties for sp in sps):
            return SamplingMetadata(all_greedy=True, **proc)
        B = len(reqs)
        f32 = lambda xs: torch.tensor(xs, dtype=torch.float32, device=device)
        md = SamplingMetadata(
            all_greedy=False, **proc,
            temperature=f32([sp.temperature for sp in sps]),
            top_k=torch.tensor([sp.top_k for sp in sps], dtype=torch.int32, device=device),
            top_p=f32([sp.top_p for sp in sps]),
            min_p=f32([sp.min_p for sp in sps]) if any(sp.min_p > 0 for sp in sps) else None,
        )
        md.seeds = torch.tensor([request_seed(r, base_seed) for r in reqs], dtype=torch.int64, device=device)
        md.offsets = torch.tensor([tokens_sampled_so_far(r) for r in reqs], dtype=torch.int64, device=device)
        if any(sp.has_penalties for sp in sps):
            md.has_penalties = True
            Lp = max(r.num_prompt_tokens for r in reqs)
            Lo = max(1, max(r.num_output_tokens for r in reqs))
            p = np.full((B, Lp), vocab_size, dtype=np.int64)
            o = np.full((B, Lo), vocab_size, dtype=np.int64)
            for i, r in enumerate(reqs):
                p[i, :r.num_prompt_tokens] = r.prompt_token_ids
                if r.output_token_ids:
                    o[i, :len(r.output_token_ids)] = r.output_token_ids
            md.prompt_ids = torch.from_numpy(p).to(device)
            md.output_ids = torch.from_numpy(o).to(device)
            md.repetition_penalty = f32([sp.repetition_penalty for sp in sps])
            md.frequency_penalty = f32([sp.frequency_penalty for sp in sps])
            md.presence_penalty = f32([sp.presence_penalty for sp in sps])
        return md


def _build_processors(reqs: list, device, vocab_size: int) -> dict:
    """Sparse logit edits of this step: additive biases, banned tokens (bad words whose prefix
    has just been generated, EOS / stop tokens before min_tokens) and allowed-token masks.  Order of
    application follows the upstream sampler: allowed ids, bad words, min-tokens, bias, then
    penalties (the reference's v2 sampler does the same on device, worker/v2/sample/*)."""
    bias_r, bias_c, bias_v, ban_r, ban_c = [], [], [], [], []
    allowed = None
    for i, r in enumerate(reqs):
        sp = r.sampling_params
        out = r.output_token_ids or []
        if sp.allowed_token_ids:
            if allowed is None:
                allowed = torch.ones((len(reqs), vocab_size), dtype=torch.bool)
            ids = torch.as_tensor(sp.allowed_token_ids, dtype=torch.long)
            if int(ids.min()) < 0 or int(ids.max()) >= vocab_size:
                from ..engine.request import RequestError
                raise RequestError(r.request_id, f"allowed_token_ids outside [0, {vocab_size})")
            allowed[i] = False
            allowed[i, ids] = True
        g = getattr(r, "guided", None)
        if g is not None:
            # structured output: tokens that keep the text inside the request's language
            g.sync(out)
            if allowed is None:
                allowed = torch.ones((len(reqs), vocab_size), dtype=torch.bool)
            allowed[i] &= g.mask(vocab_size, "cpu")
        for seq in sp.bad_words_token_ids or ():
            seq = list(seq)
            if not seq or not (0 <= seq[-1] < vocab_size):
                continue
            k = len(seq) - 1
            if k == 0 or (len(out) >= k and list(out[-k:]) == seq[:-1]):
                ban_r.append(i)
                ban_c.append(seq[-1])
        if sp.min_tokens > 0 and tokens_sampled_so_far(r) < sp.min_tokens:
            stops = set(sp.stop_token_ids or ())
            if r.eos_token_id is not None and not sp.ignore_eos:
                stops.add(r.eos_token_id)
            for t in stops:
                if 0 <= t < vocab_size:
                    ban_r.append(i)
                    ban_c.append(int(t))
        for t, b in (sp.logit_bias or {}).items():
            if 0 <= int(t) < vocab_size:
                bias_r.append(i)
                bias_c.append(int(t))
                bias_v.append(float(b))
    kw = {}
    if allowed is not None:
        kw["allowed_mask"] = allowed.to(device)
    if bias_r:
        kw["bias_index"] = torch.tensor([bias_r, bias_c], dtype=torch.int64, device=device)
        kw["bias_values"] = torch.tensor(bias_v, dtype=torch.float32, device=device)
    if ban_r:
        kw["ban_index"] = torch.tensor([ban_r, ban_c], dtype=torch.int64, device=device)
    return kw


def compute_logprobs(logits: torch.Tensor, tokens: torch.Tensor, k: int):
    """Log-probabilities under the model's raw distribution: (sampled token [B], top-k ids [B, k],
    top-k values [B, k])."""
    lp = torch.log_softmax(logits.float(), dim=-1)
    tok_lp = lp.gather(1, tokens.view(-1, 1).long()).squeeze(1)
    if k > 0:
        vals, ids = lp.topk(k, dim=-1)
    else:
        vals, ids = lp.new_zeros((lp.shape[0], 0)), tokens.new_zeros((lp.shape[0], 0))
    return tok_lp, ids, vals


class Sampler:
    def apply_processors(self, logits: torch.Tensor, md: SamplingMetadata) -> torch.Tensor:
        """Allowed-token masks, banned tokens, additive biases and the repetition / frequency /
        presence penalties.  Returns ``logits`` itself when the step has none of them, otherwise a
        new fp32 tensor."""
        if md.allowed_mask is not None or md.ban_index is not None or md.bias_index is not None:
            logits = logits.float()
            if md.allowed_mask is not None:
                logits = logits.masked_fill(~md.allowed_mask, float("-inf"))
            else:
                logits = logits.clone()
            if md.ban_index is not None:
                logits[md.ban_index[0], md.ban_index[1]] = float("-inf")
            if md.bias_index is not None:
                logits.index_put_((md.bias_index[0], md.bias_index[1]), md.bias_values, accumulate=True)
        if md.has_penalties and not md.all_greedy:
            lf = ops.to_float_logits(logits)
            if lf is logits:
                lf = logits.clone()
            logits = ops.apply_penalties(lf, md.prompt_ids, md.output_ids, md.repetition_penalty,
                                         md.frequency_penalty, md.presence_penalty)
        return logits

    def filtered_probs(self, processed_logits: torch.Tensor, md: SamplingMetadata, rows: torch.Tensor) -> torch.Tensor:
        """Distribution the sampler draws from at the given rows (after temperature and
        top-k / top-p / min-p) of already processed logits: the target distribution of speculative
        verification (vllm_ascend/sample/rejection_sampler.py:232 filters the target logits the same
        way before rejection)."""
        from ..ops import reference as ref
        t = md.temperature[rows].clamp(min=1e-5).unsqueeze(1)
        probs = torch.softmax(processed_logits.float() / t, dim=-1)
        probs = ref.top_k_top_p_filter(probs, md.top_k[rows].to(torch.int64), md.top_p[rows],
                                       None if md.min_p is None else md.min_p[rows])
        return (probs / probs.sum(dim=-1, keepdim=True).clamp(min=1e-30)).contiguous()

    def sample_processed(self, logits: torch.Tensor, md: SamplingMetadata) -> torch.Tensor:
        """Draw from logits that already went through ``apply_processors`` (destroys them on CUDA)."""
        if md.all_greedy:
            return ops.argmax(logits)
        lf = ops.to_float_logits(logits)
        return ops.sample(lf, md.temperature, md.top_k, md.top_p, md.min_p, md.seeds, md.offsets,
                          md.generator)

    def __call__(self, logits: torch.Tensor, md: SamplingMetadata) -> torch.Tensor:
        """logits [B, V] (bf16 or fp32) -> token ids int64 [B]."""
        processed = self.apply_processors(logits, md)
        if md.all_greedy:
            return ops.argmax(processed)
        lf = ops.to_float_logits(processed)
        if lf is logits:
            lf = logits.clone()
        return ops.sample(lf, md.temperature, md.top_k, md.top_p, md.min_p, md.seeds, md.offsets,
                          md.generator)
