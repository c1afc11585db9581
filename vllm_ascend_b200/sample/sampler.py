"""Sampler: penalties -> temperature -> top-k/top-p/min-p -> exponential race;
greedy rows take argmax.  Order and semantics follow
vllm_ascend/sample/sampler.py:47-159 (and the upstream Sampler flow it extends).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .. import ops


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
    allowed_mask: Optional[torch.Tensor] = None    # bool [B, V] (guided decoding / bad words)

    @staticmethod
    def build(reqs: list, device, vocab_size: int, base_seed: int = 0) -> "SamplingMetadata":
        sps = [r.sampling_params for r in reqs]
        if all(sp.greedy and not sp.has_penalties for sp in sps):
            return SamplingMetadata(all_greedy=True)
        B = len(reqs)
        f32 = lambda xs: torch.tensor(xs, dtype=torch.float32, device=device)
        md = SamplingMetadata(
            all_greedy=False,
            temperature=f32([sp.temperature for sp in sps]),
            top_k=torch.tensor([sp.top_k for sp in sps], dtype=torch.int32, device=device),
            top_p=f32([sp.top_p for sp in sps]),
            min_p=f32([sp.min_p for sp in sps]) if any(sp.min_p > 0 for sp in sps) else None,
        )
        seeds = [(sp.seed if sp.seed is not None else (base_seed * 1000003 + hash(r.request_id)) & ((1 << 62) - 1))
                 for sp, r in zip(sps, reqs)]
        md.seeds = torch.tensor(seeds, dtype=torch.int64, device=device)
        md.offsets = torch.tensor([r.num_output_tokens for r in reqs], dtype=torch.int64, device=device)
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


class Sampler:
    def __call__(self, logits: torch.Tensor, md: SamplingMetadata) -> torch.Tensor:
        """logits [B, V] (bf16 or fp32) -> token ids int64 [B]."""
        if md.allowed_mask is not None:
            logits = logits.float().masked_fill(~md.allowed_mask, float("-inf"))
        if md.all_greedy:
            return ops.argmax(logits)
        lf = ops.to_float_logits(logits)
        if lf is logits:
            lf = logits.clone()
        if md.has_penalties:
            lf = ops.apply_penalties(lf, md.prompt_ids, md.output_ids, md.repetition_penalty,
                                     md.frequency_penalty, md.presence_penalty)
        return ops.sample(lf, md.temperature, md.top_k, md.top_p, md.min_p, md.seeds, md.offsets,
                          md.generator)
