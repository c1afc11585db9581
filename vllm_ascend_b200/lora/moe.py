"""LoRA on routed experts.

Every (adapter slot, expert) pair has its own A / B matrices for the expert's gate, up and down
projections, stacked as ``[slots * E, ...]`` so the batched LoRA kernels pick the pair of a
(token, expert) assignment by the combined index ``slot * E + expert``.  Steps that carry an
adapter on a MoE layer take the expert-by-expert path: GEMM1 (unfused, the delta has to land
before SiLU-mul), delta, SiLU-mul, GEMM2, delta, weighted sum.  Tensor-parallel experts shard
B of gate / up by rows and A of down by columns like the base weights, so the partial sums the
all-reduce adds up include the adapter's contribution.  Role of the reference's MoE LoRA for its
all-gather / all-to-all MoE paths (vllm_ascend/lora/fused_moe.py, lora/quant_moe.py).

Under expert parallelism each rank stores the adapters of its own experts only (whole, not
sliced), and the adapter slot of every token travels with the token: the all-gather path gathers
the slot vector next to the activations, the all-to-all path sends it with the rows.  Steps that
carry an adapter leave the fused dispatch kernel for those two paths.
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
    num_experts: int           # experts stored here (the local ones under expert parallelism)
    rank: int
    punica: object
    expert_map: object = None  # global expert id -> local row (list, -1 = elsewhere); None = identity
    sharded: bool = True       # expert weights are TP-sliced along I (False under expert parallelism)

    def zero_slot(self, slot: int) -> None:
        E = self.num_experts
        for t in (self.a13, self.b_gate, self.b_up, self.a2, self.b2):
            t[slot * E:(slot + 1) * E].zero_()


def fused_experts_lora(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor,
                       topk_ids: torch.Tensor, expert_map, st: MoELoRAState, slots=None) -> torch.Tensor:
    """slots: adapter slot of every row of x (defaults to this step's local token slots)."""
    T, H = x.shape
    E, r = st.num_experts, st.rank
    I = w13.shape[1] // 2
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    ids = topk_ids.long()
    if expert_map is not None:
        ids = expert_map.long()[ids]
    if slots is None:
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
