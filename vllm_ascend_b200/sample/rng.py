"""Counter-based random numbers for the parts of sampling that run as PyTorch tensor ops.

A value is a pure function of (request seed, position in the request's stream, purpose tag,
column), computed with 64-bit integer mixing (the splitmix64 finaliser) on the tensor's device.
It therefore does not depend on the batch a request happens to share, on how often a generator
was advanced before, or on the process: tensor-parallel ranks that verify the same draft tokens
draw the same numbers.  The rejection sampler of the reference reaches the same property with
per-request generators (vllm_ascend/sample/rejection_sampler.py:1130-1190)."""
from __future__ import annotations

import torch


def _s64(x: int) -> int:
    """Python int holding a uint64 bit pattern -> the int64 with the same bits."""
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >= (1 << 63) else x


_C0 = _s64(0x9E3779B97F4A7C15)
_C1 = _s64(0xBF58476D1CE4E5B9)
_C2 = _s64(0x94D049BB133111EB)
_K_OFF = _s64(0xD6E8FEB86659FD93)
_K_TAG = _s64(0xA0761D6478BD642F)

TAG_ACCEPT = 1      # uniform compared with p_target / p_draft at a draft position
TAG_RECOVER = 2     # exponential race that draws the recovered token


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    return (x >> s) & ((1 << (64 - s)) - 1)


def _mix(x: torch.Tensor) -> torch.Tensor:
    x = x + _C0
    x = (x ^ _lsr(x, 30)) * _C1
    x = (x ^ _lsr(x, 27)) * _C2
    return x ^ _lsr(x, 31)


def stream_keys(seeds: torch.Tensor, offsets: torch.Tensor, tag: int) -> torch.Tensor:
    """int64 [N]: one key per (seed, offset, tag)."""
    return _mix(_mix(seeds.to(torch.int64)) + offsets.to(torch.int64) * _K_OFF + _s64(tag * _K_TAG))


def uniform(keys: torch.Tensor, cols: int = 0) -> torch.Tensor:
    """fp32 in (0, 1): [N] for ``cols == 0`` else [N, cols]."""
    if cols:
        idx = torch.arange(cols, dtype=torch.int64, device=keys.device)
        h = _mix(keys[:, None] + idx[None, :] * _C1)
    else:
        h = _mix(keys)
    return (_lsr(h, 41).to(torch.float32) + 0.5) * (1.0 / (1 << 23))


def exponential(keys: torch.Tensor, cols: int) -> torch.Tensor:
    """fp32 Exp(1) variates [N, cols]."""
    return -torch.log(uniform(keys, cols))
