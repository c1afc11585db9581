"""Layer-shaped wrappers around the kernels with the call shape a host vLLM's ``CustomOp``
expects (``forward_oot``): what the out-of-tree op table points at
(vllm_ascend/utils.py:703-732 lists the reference's)."""
from __future__ import annotations

from typing import Optional

import torch

from . import reference as ref
from .. import ops


class SiluAndMul(torch.nn.Module):
    def forward_oot(self, x: torch.Tensor) -> torch.Tensor:
        return ops.silu_and_mul(x)

    forward = forward_oot


class RMSNorm(torch.nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, dtype=torch.bfloat16):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(hidden_size, dtype=dtype))
        self.variance_epsilon = eps
        self.gemma = False

    def forward_oot(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        y, r = ops.rms_norm(x, self.weight, self.variance_epsilon, residual, gemma=self.gemma)
        return y if residual is None else (y, r)

    forward = forward_oot


class GemmaRMSNorm(RMSNorm):
    def __init__(self, hidden_size: int, eps: float = 1e-6, dtype=torch.bfloat16):
        super().__init__(hidden_size, eps, dtype)
        self.gemma = True


class RotaryEmbedding(torch.nn.Module):
    """Neox-style rotary embedding over a cached cos/sin table."""

    def __init__(self, head_size: int, rotary_dim: int, max_position: int, base: float, is_neox_style: bool = True,
                 dtype=torch.float32):
        super().__init__()
        from ..models.layers import get_cos_sin_cache
        self.head_size, self.rotary_dim, self.is_neox_style = head_size, rotary_dim, is_neox_style
        self.register_buffer("cos_sin_cache", get_cos_sin_cache(rotary_dim, max_position, base, None, "cpu"),
                             persistent=False)

    def forward_oot(self, positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor):
        cs = self.cos_sin_cache.to(query.device)
        q = query.view(query.shape[0], -1, self.head_size)
        k = key.view(key.shape[0], -1, self.head_size)
        fn = ref.apply_rope if self.is_neox_style else ref.apply_rope_interleaved
        return (fn(q, positions, cs, self.rotary_dim).view_as(query),
                fn(k, positions, cs, self.rotary_dim).view_as(key))

    forward = forward_oot
