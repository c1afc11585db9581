"""MoE routing and expert computation.

``gating_topk`` implements the router of the reference's fused gating op
(softmax / sigmoid scores, correction bias, group-limited top-k, renormalise,
scaling; csrc/moe/moe_gating_top_k, golden model in
tests/e2e/nightly/single_node/ops/singlecard_ops/test_npu_moe_gating_top_k.py:34-90).
``fused_experts`` is dispatch -> grouped GEMM1 -> SwiGLU -> grouped GEMM2 ->
weighted combine for the experts resident on this rank
(vllm_ascend/ops/fused_moe/moe_mlp.py:573-687).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from . import reference as ref


def gating_topk_ref(logits: torch.Tensor, k: int, scoring: str = "softmax", renorm: bool = True,
                    n_group: int = 1, topk_group: int = 1,
                    bias: Optional[torch.Tensor] = None, scale: float = 1.0):
    x = logits.float()
    scores = torch.softmax(x, dim=-1) if scoring == "softmax" else torch.sigmoid(x)
    choice = scores + bias.float() if bias is not None else scores
    T, E = scores.shape
    if n_group > 1:
        g = choice.view(T, n_group, E // n_group)
        if bias is not None:
            gscore = g.topk(2, dim=-1).values.sum(-1)       # noaux_tc: sum of the top-2 per group
        else:
            gscore = g.max(dim=-1).values
        gidx = gscore.topk(topk_group, dim=-1).indices
        gmask = torch.zeros(T, n_group, dtype=torch.bool, device=x.device)
        gmask.scatter_(1, gidx, True)
        choice = choice.masked_fill(~gmask.unsqueeze(-1).expand(T, n_group, E // n_group)
                                    .reshape(T, E), float("-inf"))
    ids = choice.topk(k, dim=-1).indices
    w = scores.gather(1, ids)
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True).clamp_min(1e-20)
    return (w * scale).float(), ids.to(torch.int32)


def gating_topk(logits: torch.Tensor, k: int, scoring: str = "softmax", renorm: bool = True,
                n_group: int = 1, topk_group: int = 1, bias: Optional[torch.Tensor] = None,
                scale: float = 1.0):
    if logits.is_cuda and _native.available() and hasattr(_native.lib(), "b200_moe_gating_topk") \
            and logits.shape[1] <= 512 and k <= 16:
        from . import moe_native
        return moe_native.gating_topk(logits, k, scoring, renorm, n_group, topk_group, bias, scale)
    return gating_topk_ref(logits, k, scoring, renorm, n_group, topk_group, bias, scale)


def fused_experts_ref(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor,
                      topk_w: torch.Tensor, topk_ids: torch.Tensor,
                      expert_map: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T,H]; w13 [E_local, 2I, H]; w2 [E_local, H, I]; ids are global expert ids,
    ``expert_map`` maps global -> local (-1: not on this rank)."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    ids = topk_ids.long()
    if expert_map is not None:
        ids = expert_map.long()[ids]
    E = w13.shape[0]
    for e in range(E):
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = x[tok] @ w13[e].to(x.dtype).t()
        a = ref.silu_and_mul(h)
        y = a @ w2[e].to(x.dtype).t()
        out.index_add_(0, tok, y.float() * topk_w[tok, slot].unsqueeze(-1).float())
    return out.to(x.dtype)


def fused_experts(x, w13, w2, topk_w, topk_ids, expert_map=None, quant=None):
    if x.is_cuda and x.dtype == torch.bfloat16 and _native.available() \
            and hasattr(_native.lib(), "b200_grouped_gemm_bf16") and quant is None:
        from . import moe_native
        return moe_native.fused_experts(x, w13, w2, topk_w, topk_ids, expert_map)
    if quant is not None:
        return quant.apply_experts(x, w13, w2, topk_w, topk_ids, expert_map)
    return fused_experts_ref(x, w13, w2, topk_w, topk_ids, expert_map)


def hash_topk(token_ids: torch.Tensor, table: torch.Tensor):
    """Hash routing: the experts of a token are a fixed function of its token id
    (``table`` [vocab, k] of expert ids), all with equal weight — the router of the first
    layers of some models (vllm_ascend/ops/fused_moe/router/fused_topk_router.py:103-141)."""
    ids = table[token_ids.long()].to(torch.int32)
    k = ids.shape[1]
    w = torch.full(ids.shape, 1.0 / k, dtype=torch.float32, device=ids.device)
    return w, ids
