"""LoRA on routed experts.

Every (adapter slot, expert) pair has its own A / B matrices for the expert's gate, up and down
projections, stacked as ``[slots * E, ...]`` so the batched LoRA kernels pick the pair of a
(token, expert) assignment by the combined index ``slot * E + expert``.  Steps that carry an
adapter on a MoE layer take the expert-by-expert path: GEMM1 (unfused, the delta has to land
before SiLU-mul), delta, SiLU-mul, GEMM2, delta, weighted sum.  Tensor-parallel experts shard
B of gate / up by rows and A of down by columns like the base weights, so the partial sums the
all-reduce adds up include the adapter's contribution.  Role of the reference's MoE LoRA for its
all-gather / all-to-all MoE paths (vllm_ascend/lora/fused_moe.py, lora/quant_moe.py); expert
parallel engines do not take expert adapters here.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from . import ops as lops


@dataclass
class MoELoRAState:
    a13: torch.Tensor          # [slots * E, 2 * r, H]     (gate rows, then up rows)
    b_gate: torch.Tensor       # [slots * E, I_local, r]
    b_up: torch.Tensor         # [slots * E, I_local, r]
    a2: torch.Tensor           # [slots * E, r, I_local]
    b2: torch.Tensor           # [slots * E, H, r]
    num_experts: int
    rank: int
    punica: object

    def zero_slot(self, slot: int) -> None:
        E = self.num_experts
        for t in (self.a13, self.b_gate, self.b_up, self.a2, self.b2):
            t[slot * E:(slot + 1) * E].zero_()


def fused_experts_lora(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor,
                       topk_ids: torch.Tensor, expert_map, st: MoELoRAState) -> torch.Tensor:
    T, H = x.shape
    E, r = st.num_experts, st.rank
    I = w13.shape[1] // 2
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    ids = topk_ids.long()
    if expert_map is not None:
        ids = expert_map.long()[ids]
    slots = st.punica.token_slots[:T]
    for e in range(w13.shape[0]):
        tok, k = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok].contiguous()
        s = slots[tok]
        idx = torch.where(s >= 0, s * E + e, torch.full_like(s, -1)).to(torch.int32)
        h = ops.linear(xe, w13[e])
        v = lops.bgmv_shrink(xe, st.a13, idx, 1.0)
        lops.bgmv_expand(v, st.b_gate, idx, h, 0, 0, add=True)
        lops.bgmv_expand(v, st.b_up, idx, h, I, r, add=True)
        a = ops.silu_and_mul(h)
        y = ops.linear(a, w2[e])
        v2 = lops.bgmv_shrink(a, st.a2, idx, 1.0)
        lops.bgmv_expand(v2, st.b2, idx, y, 0, 0, add=True)
        out.index_add_(0, tok, y.float() * topk_w[tok, k].unsqueeze(-1).float())
    return out.to(x.dtype)
