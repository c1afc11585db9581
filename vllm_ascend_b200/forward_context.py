"""Per-step forward context.

One object per engine step carries what layers need besides their inputs: attention
metadata, the MoE communication method chosen for the step, padded token count, whether a
graph is being captured, the running layer index.  Mirrors
vllm_ascend/ascend_forward_context.py:58-169 (context extras) and :223-343 (MoE method
selection, delegated to ``ops.moe_comm.select_moe_comm_method``).
"""
from __future__ import annotations

import contextlib
import threading
from dataclasses import dataclass, field
from typing import Any, Optional

import torch


@dataclass
class ForwardContext:
    attn_metadata: Any = None
    num_tokens: int = 0
    padded_length: int = 0
    num_tokens_across_dp: Optional[list] = None
    max_tokens_across_dp: int = 0
    moe_comm_type: Any = None
    moe_comm_method: Any = None
    fused_moe_mask: Optional[torch.Tensor] = None     # active-token mask for padded decode batches
    capturing: bool = False
    in_profile_run: bool = False
    cudagraph_runtime_mode: str = "NONE"
    batch_descriptor: Any = None
    layer_idx: int = 0
    sp_enabled: bool = False
    gemm_rs_fusion: bool = False       # row-parallel GEMM ends in a fused reduce-scatter
    prefetch_weights: bool = False
    extra: dict = field(default_factory=dict)


_TLS = threading.local()


def get_forward_context() -> ForwardContext:
    ctx = getattr(_TLS, "ctx", None)
    if ctx is None:
        raise RuntimeError("no forward context is set; wrap the model call in set_forward_context()")
    return ctx


def has_forward_context() -> bool:
    return getattr(_TLS, "ctx", None) is not None


@contextlib.contextmanager
def set_forward_context(attn_metadata=None, num_tokens: int = 0, **extras):
    prev = getattr(_TLS, "ctx", None)
    ctx = ForwardContext(attn_metadata=attn_metadata, num_tokens=num_tokens)
    for k, v in build_extra_context(num_tokens=num_tokens, **extras).items():
        if hasattr(ctx, k):
            setattr(ctx, k, v)
        else:
            ctx.extra[k] = v
    _TLS.ctx = ctx
    try:
        yield ctx
    finally:
        _TLS.ctx = prev


def build_extra_context(num_tokens: int = 0, num_tokens_across_dp=None, tp_size: int = 1, ep_size: int = 1,
                        fused_moe_available: bool = False, fused_moe_capacity: int = 512,
                        is_cuda: bool = True, sp_enabled: bool = False, capturing: bool = False,
                        in_profile_run: bool = False, moe_override: str = "", is_moe: bool = False,
                        **passthrough) -> dict:
    """The dictionary of extras for a step: padded length (a multiple of the TP size when the
    residual stream is sequence-sharded), the largest token count over the DP ranks, the
    MoE communication type, and the active-token mask of the fused MoE path."""
    out: dict = dict(passthrough)
    mx = max(num_tokens_across_dp) if num_tokens_across_dp else num_tokens
    out["num_tokens_across_dp"] = list(num_tokens_across_dp) if num_tokens_across_dp else None
    out["max_tokens_across_dp"] = mx
    out["padded_length"] = ((num_tokens + tp_size - 1) // tp_size) * tp_size if sp_enabled else num_tokens
    out["sp_enabled"] = sp_enabled
    out["gemm_rs_fusion"] = sp_enabled and tp_size <= 8
    out["capturing"] = capturing
    out["in_profile_run"] = in_profile_run
    if is_moe:
        from .ops.moe_comm import MoECommType, select_moe_comm_method
        t = select_moe_comm_method(mx, ep_size, fused_moe_available, fused_moe_capacity, is_cuda, moe_override)
        out["moe_comm_type"] = t
        if t is MoECommType.FUSED:
            # every rank pads to the same capacity; the mask marks its real tokens
            mask = torch.zeros(fused_moe_capacity, dtype=torch.bool)
            mask[:num_tokens] = True
            out["fused_moe_mask"] = mask
    return out
