"""Lightning-attention layer: linear attention with a fixed exponential decay per head
(the recurrent layers of MiniMax-Text-01; Bailing's linear layers have the same recurrence).

Per token: one projection to [q | k | v] per head followed by SiLU; S_t = r_h S_{t-1} + k_t v_t^T,
o_t = S_t^T q_t with r_h = exp(-slope_h); RMSNorm over all heads together; a sigmoid output gate
from the layer input; output projection.  The decay slopes are not learned: slope_h =
2^(-8 (h + 1) / H) scaled by 1 - layer / (L - 1) (+ 1e-5), so later layers forget more slowly.
Instead of a KV cache the layer keeps one [D x D] fp32 state per head and sequence.

Heads are sharded over TP (the checkpoint's projection rows are grouped per head, so a rank's
heads are contiguous rows); the norm's mean square is all-reduced.  Role of the reference's
linear-attention layer op for this family (``BailingMoELinearAttention`` in its
out-of-tree op table, vllm_ascend/utils.py:703-732, kernels in
vllm_ascend/ops/triton/mamba/lightning_attn.py).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops import linear_attn as la
from .layers import ColumnParallelLinear, ParamFactory, RowParallelLinear, TPComm


def lightning_slopes(num_heads: int, layer_idx: int, num_layers: int) -> torch.Tensor:
    base = 1.0 / (2.0 ** (8.0 / num_heads))
    rate = base ** (torch.arange(num_heads, dtype=torch.float32) + 1)
    return rate * (1 - layer_idx / (num_layers - 1 + 1e-5) + 1e-5)


class LightningAttention:
    is_linear_attention = True
    kind = "lightning"

    def __init__(self, pf: ParamFactory, cfg: ModelConfig, layer_idx: int, comm: TPComm):
        tp = comm.size
        self.cfg, self.comm = cfg, comm
        self.H_total = cfg.num_attention_heads
        self.H = self.H_total // tp
        self.D = cfg.head_dim
        p = f"model.layers.{layer_idx}.self_attn"
        full = self.H_total * self.D
        self.qkv_proj = ColumnParallelLinear(pf, f"{p}.qkv_proj", cfg.hidden_size, [3 * full], comm)
        self.output_gate = ColumnParallelLinear(pf, f"{p}.output_gate", cfg.hidden_size, [full], comm)
        self.out_proj = RowParallelLinear(pf, f"{p}.out_proj", full, cfg.hidden_size, comm)
        self.norm_weight = pf.ones((self.H * self.D,))
        slopes = lightning_slopes(self.H_total, layer_idx, cfg.num_hidden_layers)
        self.log_decay = (-slopes[comm.rank * self.H:(comm.rank + 1) * self.H]).to(pf.device)
        self.chunk = int(cfg.lightning_block_size or 64)

    def state_shapes(self, num_slots: int):
        """(unused convolution slot, recurrent state) shapes: the runner allocates a pair per layer."""
        return (num_slots, 1, 1), (num_slots, self.H, self.D, self.D)

    def __call__(self, x: torch.Tensor, meta, cache) -> torch.Tensor:
        _, state = cache
        T = x.shape[0]
        qkv = F.silu(self.qkv_proj(x)).view(T, self.H, 3 * self.D)
        q, k, v = qkv[..., :self.D], qkv[..., self.D:2 * self.D], qkv[..., 2 * self.D:]
        o = la.lightning_attention(q, k, v, self.log_decay, state, meta.query_start_loc, meta.state_slots,
                                   meta.has_initial_state, cu_cpu=meta.query_start_loc_cpu,
                                   chunk=self.chunk).reshape(T, self.H * self.D)
        # RMSNorm over all heads together; this rank holds H of them
        of = o.float()
        ss = (of * of).sum(-1, keepdim=True)
        if self.comm.size > 1:
            ss = self.comm.group.all_reduce(ss)
        o = (of * torch.rsqrt(ss / (self.H_total * self.D) + self.cfg.rms_norm_eps)).to(x.dtype) * self.norm_weight
        o = torch.sigmoid(self.output_gate(x)) * o
        return self.out_proj(o)

    def named_tensors(self):
        for attr in ("qkv_proj", "output_gate", "out_proj"):
            for n, t in getattr(self, attr).named_tensors():
                yield f"{attr}.{n}", t
        yield "norm.weight", self.norm_weight
