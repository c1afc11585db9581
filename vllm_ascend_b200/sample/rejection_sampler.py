"""Rejection sampling for speculative decoding.

``rejection_sample`` takes the flattened draft token ids with per-request counts, the
target model's distribution at every draft position (+ the bonus position) and returns
``[batch, max_spec_len + 1]`` token ids padded with -1 together with the number of tokens
emitted per request.  Greedy rows accept while ``draft == argmax(target)``; random rows
accept ``x`` with probability ``min(1, p_target(x) / p_draft(x))``, emit a recovered token
drawn from ``max(p_target - p_draft, 0)`` at the first rejection, and the bonus token only
when every draft was accepted (vllm_ascend/sample/rejection_sampler.py:422-905, 1130-1310).
Two more verification rules of the reference are provided as options: block verification
(:1482-1597) and entropy-adaptive acceptance (threshold ``min(exp(-H * alpha), tau)``).
"""
from __future__ import annotations

from ctypes import c_int, c_void_p
from typing import Optional

import torch

from .. import _native

P, I = c_void_p, c_int
_native.register_signature("b200_rejection_sample", [P, P, P, P, P, P, P, P, P, P, P, I, I, I, P, P])
_native.register_signature("b200_expand_draft_inputs", [P, P, P, P, P, P, P, I, I, P])

PLACEHOLDER = -1


def rejection_sample_ref(draft_ids, cu_draft, target_argmax, bonus_ids, target_probs, draft_probs,
                         uniform, race_noise, is_greedy, max_spec: int):
    """Plain PyTorch definition (also the CPU path)."""
    B = bonus_ids.shape[0]
    out = torch.full((B, max_spec + 1), PLACEHOLDER, dtype=torch.int32)
    num = torch.zeros(B, dtype=torch.int32)
    cu = cu_draft.tolist()
    for b in range(B):
        s0, n = cu[b], cu[b + 1] - cu[b]
        greedy = bool(is_greedy[b]) or target_probs is None
        stop = n
        for i in range(n):
            x = int(draft_ids[s0 + i])
            if greedy:
                ok = x == int(target_argmax[s0 + i])
            else:
                pt = float(target_probs[s0 + i, x])
                pd = float(draft_probs[s0 + i, x]) if draft_probs is not None else 1.0
                ok = pd > 0 and float(uniform[s0 + i]) * pd < pt
            if not ok:
                stop = i
                break
            out[b, i] = x
        if stop == n:
            out[b, n] = int(bonus_ids[b])
            num[b] = n + 1
        elif greedy:
            out[b, stop] = int(target_argmax[s0 + stop])
            num[b] = stop + 1
        else:
            pt = target_probs[s0 + stop].float()
            if draft_probs is not None:
                r = (pt - draft_probs[s0 + stop].float()).clamp(min=0)
            else:
                r = pt.clone()
                r[int(draft_ids[s0 + stop])] = 0
            out[b, stop] = int((r / race_noise[b].float().clamp(min=1e-20)).argmax())
            num[b] = stop + 1
    return out, num


def rejection_sample(draft_ids: torch.Tensor, cu_draft: torch.Tensor, target_argmax: torch.Tensor,
                     bonus_ids: torch.Tensor, target_probs: Optional[torch.Tensor],
                     draft_probs: Optional[torch.Tensor], uniform: Optional[torch.Tensor],
                     race_noise: Optional[torch.Tensor], is_greedy: torch.Tensor, max_spec: int):
    if not draft_ids.is_cuda:
        return rejection_sample_ref(draft_ids, cu_draft, target_argmax, bonus_ids, target_probs, draft_probs,
                                    uniform, race_noise, is_greedy, max_spec)
    B = bonus_ids.shape[0]
    dev = draft_ids.device
    out = torch.empty((B, max_spec + 1), dtype=torch.int32, device=dev)
    num = torch.empty(B, dtype=torch.int32, device=dev)
    V = target_probs.shape[1] if target_probs is not None else 0
    rc = _native.lib().b200_rejection_sample(
        draft_ids.data_ptr(), cu_draft.data_ptr(), target_argmax.data_ptr(), bonus_ids.data_ptr(),
        _native.ptr(target_probs), _native.ptr(draft_probs), _native.ptr(uniform), _native.ptr(race_noise),
        is_greedy.data_ptr(), out.data_ptr(), num.data_ptr(), B, V, max_spec,
        _native.status_word(dev).data_ptr(), _native.stream_ptr())
    _native.check(rc, "rejection_sample")
    _native.count_launch()
    return out, num


def block_verify_accept_len(p_target_at_draft: torch.Tensor, p_draft_at_draft: torch.Tensor,
                            uniform: torch.Tensor) -> int:
    """Block verification for one request: accept the longest prefix ``i`` such that
    ``u_i <= min(1, prod_{j<=i} p_t(x_j) / p_d(x_j))`` holds jointly, which accepts at least as
    many tokens in expectation as token-by-token verification."""
    ratio = torch.cumprod(p_target_at_draft.double() / p_draft_at_draft.double().clamp(min=1e-30), 0).clamp(max=1.0)
    ok = uniform.double() <= ratio
    idx = torch.nonzero(ok).flatten()
    return int(idx[-1]) + 1 if idx.numel() else 0


def entropy_threshold(target_probs_row: torch.Tensor, alpha: float, tau: float) -> float:
    """Acceptance threshold ``min(exp(-H * alpha), tau)`` of entropy-adaptive verification: a
    confident target (low entropy H) demands a high target probability of the draft token."""
    p = target_probs_row.double().clamp(min=1e-30)
    H = float(-(p * p.log()).sum())
    return min(float(torch.exp(torch.tensor(-H * alpha))), tau)


class RejectionSampler:
    def __init__(self, method: str = "standard", entropy_alpha: float = 1.0, entropy_tau: float = 0.9):
        if method not in ("standard", "block_verify", "entropy_verify"):
            raise ValueError(f"unknown rejection sampling method {method!r}")
        self.method, self.alpha, self.tau = method, entropy_alpha, entropy_tau
        self.stats = {"drafted": 0, "accepted": 0, "steps": 0}

    def __call__(self, draft_ids, cu_draft, target_logits, bonus_ids, is_greedy, temperature, max_spec,
                 draft_probs=None, generator=None, target_probs=None, seeds=None, offsets=None):
        """target_logits: [N, V] rows of the draft positions (fp32), after the request's logit
        processors and penalties.  ``target_probs``: the distribution the sampler would draw from at
        those rows (temperature, top-k / top-p / min-p applied); softmax(logits / T) when absent.
        ``seeds`` / ``offsets`` (int64 [B]: request seed, tokens sampled so far): the acceptance
        uniforms and the recovered-token race come from the request's own counter-based stream, the
        same in every tensor-parallel process; otherwise from ``generator``."""
        target_argmax = target_logits.argmax(-1).to(torch.int32)
        all_greedy = bool(is_greedy.all())
        probs = uniform = noise = None
        if not all_greedy:
            N, V = target_logits.shape
            B = bonus_ids.shape[0]
            counts = (cu_draft[1:] - cu_draft[:-1]).long()
            if target_probs is not None:
                probs = target_probs.float().contiguous()
            else:
                t_rows = torch.repeat_interleave(temperature.float().clamp(min=1e-5), counts)
                probs = torch.softmax(target_logits.float() / t_rows[:, None], dim=-1).contiguous()
            if seeds is not None:
                from . import rng
                off = offsets if offsets is not None else torch.zeros_like(seeds)
                row_seed = torch.repeat_interleave(seeds, counts)
                within = torch.arange(N, device=probs.device) - torch.repeat_interleave(cu_draft[:-1].long(), counts)
                row_off = torch.repeat_interleave(off, counts) + within
                uniform = rng.uniform(rng.stream_keys(row_seed, row_off, rng.TAG_ACCEPT)).contiguous()
                noise = rng.exponential(rng.stream_keys(seeds, off, rng.TAG_RECOVER), V).contiguous()
            else:
                uniform = torch.rand(N, device=probs.device, generator=generator)
                noise = torch.empty(B, V, device=probs.device).exponential_(generator=generator)
            if self.method != "standard":
                uniform = self._reshape_uniform(draft_ids, cu_draft, probs, draft_probs, uniform, is_greedy)
        out, num = rejection_sample(draft_ids, cu_draft, target_argmax, bonus_ids, probs, draft_probs, uniform,
                                    noise, is_greedy.to(torch.uint8), max_spec)
        self.stats["steps"] += 1
        self.stats["drafted"] += int(draft_ids.numel())
        self.stats["accepted"] += int((num - 1).clamp(min=0).sum())
        return out, num

    def _reshape_uniform(self, draft_ids, cu_draft, probs, draft_probs, uniform, is_greedy):
        """The two alternative rules are expressed through the uniform numbers the kernel
        compares against, so one kernel serves all three methods: position i is accepted by the
        kernel iff u_i * p_d < p_t; forcing u_i to 0 accepts, to 2 rejects."""
        u = uniform.clone()
        cu = cu_draft.tolist()
        for b in range(len(cu) - 1):
            s0, n = cu[b], cu[b + 1] - cu[b]
            if n == 0 or bool(is_greedy[b]):
                continue
            x = draft_ids[s0:s0 + n].long()
            pt = probs[s0:s0 + n].gather(1, x[:, None]).squeeze(1)
            pd = draft_probs[s0:s0 + n].gather(1, x[:, None]).squeeze(1) if draft_probs is not None \
                else torch.ones_like(pt)
            if self.method == "block_verify":
                k = block_verify_accept_len(pt, pd, uniform[s0:s0 + n])
                u[s0:s0 + k] = 0.0
                if k < n:
                    u[s0 + k] = 2.0
            else:
                for i in range(n):
                    thr = entropy_threshold(probs[s0 + i], self.alpha, self.tau)
                    ok = float(pt[i]) >= thr * float(pd[i])
                    u[s0 + i] = 0.0 if ok else 2.0
        return u
