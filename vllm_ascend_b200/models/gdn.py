"""Gated DeltaNet linear-attention layer (the recurrent layers of Qwen3-Next style hybrids).

Per token: projections to q, k, v, an output gate z and two per-head scalars (b -> write
strength beta, a -> decay g); a short causal convolution + SiLU over [q | k | v]; the gated
delta-rule recurrence on a [key_dim x value_dim] state per value head; gated RMSNorm with z; output
projection.  Instead of a KV cache the layer keeps, per sequence, the last K-1 convolution
inputs and the recurrent state.  Role of vllm_ascend/ops/gdn.py (GatedDeltaNetAttention).
Heads are sharded over TP; projections use one [q | k | v | z] layout (checkpoints with the
interleaved per-group layout are re-ordered at load time).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from ..ops import linear_attn as la
from .layers import ColumnParallelLinear, ParamFactory, RowParallelLinear, TPComm


class GatedDeltaNet:
    is_linear_attention = True

    def __init__(self, pf: ParamFactory, cfg: ModelConfig, layer_idx: int, comm: TPComm):
        tp = comm.size
        self.cfg = cfg
        self.Hk, self.Hv = cfg.linear_num_key_heads // tp, cfg.linear_num_value_heads // tp
        self.Dk, self.Dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.K = cfg.linear_conv_kernel_dim
        self.key_dim, self.value_dim = self.Hk * self.Dk, self.Hv * self.Dv
        self.conv_dim = 2 * self.key_dim + self.value_dim
        p = f"model.layers.{layer_idx}.linear_attn"
        kd, vd = cfg.linear_num_key_heads * self.Dk, cfg.linear_num_value_heads * self.Dv
        self.in_proj_qkvz = ColumnParallelLinear(pf, f"{p}.in_proj_qkvz", cfg.hidden_size, [kd, kd, vd, vd], comm)
        self.in_proj_ba = ColumnParallelLinear(pf, f"{p}.in_proj_ba", cfg.hidden_size,
                                               [cfg.linear_num_value_heads, cfg.linear_num_value_heads], comm)
        r = comm.rank
        self.conv_weight = torch.cat([
            pf.normal(f"{p}.conv1d.q", (kd, self.K), 0, r, tp, std=0.3),
            pf.normal(f"{p}.conv1d.k", (kd, self.K), 0, r, tp, std=0.3),
            pf.normal(f"{p}.conv1d.v", (vd, self.K), 0, r, tp, std=0.3)], dim=0).contiguous()
        self.dt_bias = pf.normal(f"{p}.dt_bias", (cfg.linear_num_value_heads,), 0, r, tp, std=0.5, dtype=torch.float32)
        self.A_log = pf.normal(f"{p}.A_log", (cfg.linear_num_value_heads,), 0, r, tp, std=0.5, dtype=torch.float32)
        self.norm_weight = pf.ones((self.Dv,))
        self.out_proj = RowParallelLinear(pf, f"{p}.out_proj", vd, cfg.hidden_size, comm)
        self.scale = self.Dk ** -0.5

    def state_shapes(self, num_slots: int):
        """(conv state, recurrent state) shapes for ``num_slots`` sequences."""
        return (num_slots, self.K - 1, self.conv_dim), (num_slots, self.Hv, self.Dk, self.Dv)

    def __call__(self, x: torch.Tensor, meta, cache) -> torch.Tensor:
        conv_state, ssm_state = cache
        T = x.shape[0]
        qkvz = self.in_proj_qkvz(x)
        ba = self.in_proj_ba(x)
        kd, vd = self.key_dim, self.value_dim
        mixed = qkvz[:, :2 * kd + vd]
        z = qkvz[:, 2 * kd + vd:]
        cu, slots, has_init = meta.query_start_loc, meta.state_slots, meta.has_initial_state
        mixed = la.causal_conv1d(mixed, self.conv_weight, None, conv_state, cu, slots, has_init, act=True)
        q = mixed[:, :kd].reshape(T, self.Hk, self.Dk)
        k = mixed[:, kd:2 * kd].reshape(T, self.Hk, self.Dk)
        v = mixed[:, 2 * kd:].reshape(T, self.Hv, self.Dv)
        beta = torch.sigmoid(ba[:, :self.Hv].float())
        g = -torch.exp(self.A_log) * F.softplus(ba[:, self.Hv:].float() + self.dt_bias)
        o = la.gated_delta_rule(q, k, v, g, beta, ssm_state, cu, slots, has_init, self.scale, l2norm=True,
                                cu_cpu=None if meta.max_query_len <= 1 else meta.query_start_loc_cpu)
        o = ops.rms_norm_gated(o.reshape(T, vd), z.contiguous(), self.norm_weight, self.cfg.rms_norm_eps,
                               group=self.Dv, norm_before_gate=True)
        return self.out_proj(o)

    def load_hf(self, suffix: str, w: torch.Tensor, tp: int, r: int) -> bool:
        """One tensor of a published checkpoint (name relative to ``linear_attn.``).  The checkpoint
        groups the projection rows by key head ([q, k, v-heads of the group, z-heads of the group] and
        [b, a] per group); here the layout is [q | k | v | z] and [b | a], sliced per TP rank."""
        cfg = self.cfg
        Hk, Hv, Dk, Dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, self.Dk, self.Dv
        ratio = Hv // Hk

        def shard(parts):          # every part is split over TP along dim 0
            return torch.cat([p_[r * p_.shape[0] // tp:(r + 1) * p_.shape[0] // tp] for p_ in parts], dim=0)
        if suffix == "in_proj_qkvz.weight":
            g = w.view(Hk, 2 * Dk + 2 * ratio * Dv, -1)
            q, k = g[:, :Dk].reshape(Hk * Dk, -1), g[:, Dk:2 * Dk].reshape(Hk * Dk, -1)
            v = g[:, 2 * Dk:2 * Dk + ratio * Dv].reshape(Hv * Dv, -1)
            z = g[:, 2 * Dk + ratio * Dv:].reshape(Hv * Dv, -1)
            self.in_proj_qkvz.weight.copy_(shard([q, k, v, z]))
        elif suffix == "in_proj_ba.weight":
            g = w.view(Hk, 2 * ratio, -1)
            self.in_proj_ba.weight.copy_(shard([g[:, :ratio].reshape(Hv, -1), g[:, ratio:].reshape(Hv, -1)]))
        elif suffix == "conv1d.weight":
            c = w.reshape(w.shape[0], -1)                                   # [conv_dim, K]
            kd, vd = Hk * Dk, Hv * Dv
            self.conv_weight.copy_(shard([c[:kd], c[kd:2 * kd], c[2 * kd:2 * kd + vd]]))
        elif suffix in ("dt_bias", "A_log"):
            getattr(self, suffix).copy_(w[r * Hv // tp:(r + 1) * Hv // tp].to(torch.float32))
        elif suffix == "norm.weight":
            self.norm_weight.copy_(w)
        elif suffix == "out_proj.weight":
            n = w.shape[1] // tp
            self.out_proj.weight.copy_(w[:, r * n:(r + 1) * n])
        else:
            return False
        return True

    def named_tensors(self):
        yield "conv1d.weight", self.conv_weight
        yield "dt_bias", self.dt_bias
        yield "A_log", self.A_log
        yield "norm.weight", self.norm_weight
