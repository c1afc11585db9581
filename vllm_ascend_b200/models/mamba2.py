"""Mamba-2 mixer (selective state-space layer of Bamba / Granite-4 / Nemotron-H style hybrids).

Per token: one input projection to [z | x | B | C | dt]; a short causal convolution + SiLU over
[x | B | C]; the state-space recurrence per head h (P channels, N state dimensions)

    S_t = exp(dt_t A_h) S_{t-1} + B_t (dt_t x_t)^T          y_t = S_t^T C_t + D_h x_t

with dt = softplus(dt + dt_bias) clamped to the configured limits, A_h = -exp(A_log_h), and B, C
shared by the heads of a group; RMSNorm of y * silu(z) over the whole inner width; output projection.
The recurrence is gated linear attention with q = C, k = B, v = dt x and log-decay dt A
(state-space duality), so prefill chunks run in the chunk-parallel form and decode rows in one
batched state update (``ops.linear_attn.gated_linear_attention``).  Instead of a KV cache the
layer keeps, per sequence, the last K-1 convolution inputs and the [N x P] state per head.

Heads are sharded over TP.  Groups are sharded when there are at least as many as ranks, otherwise
each rank keeps the one group its heads belong to (its B / C columns are computed redundantly).
The mean square of the gated norm is all-reduced.  Role of the Mamba layers the reference runs
through vLLM's hybrid models (vllm_ascend/patch/platform/patch_mamba_config.py: state page sizing;
vllm_ascend/ops/triton/mamba/causal_conv1d.py: the convolution; hybrid KV + state transfer in
vllm_ascend/distributed/kv_transfer/kv_p2p/mooncake_hybrid_connector.py).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops import linear_attn as la
from .layers import ColumnParallelLinear, ParamFactory, RowParallelLinear, TPComm


class Mamba2Mixer:
    is_linear_attention = True
    kind = "mamba2"

    def __init__(self, pf: ParamFactory, cfg: ModelConfig, layer_idx: int, comm: TPComm):
        m = cfg.mamba_config
        tp, r = comm.size, comm.rank
        self.cfg, self.comm = cfg, comm
        self.H_total, self.P, self.N = int(m["n_heads"]), int(m["d_head"]), int(m["d_state"])
        self.G_total, self.K = int(m["n_groups"]), int(m["d_conv"])
        self.I_total = self.H_total * self.P
        if self.H_total % tp or (self.G_total % tp and tp % self.G_total):
            raise ValueError(f"Mamba-2 layer: {self.H_total} heads / {self.G_total} groups do not divide over {tp} ranks")
        self.H = self.H_total // tp
        self.I = self.H * self.P
        self.G = max(1, self.G_total // tp)                     # groups held by this rank
        # first group of this rank in the checkpoint's numbering
        self.g0 = r * self.G if self.G_total >= tp else r // (tp // self.G_total)
        self.conv_dim = self.I + 2 * self.G * self.N
        self.dt_limit = tuple(float(x) for x in m.get("time_step_limit", (0.0, float("inf"))))
        self.eps = cfg.rms_norm_eps
        p = f"model.layers.{layer_idx}.mamba"
        gn_virtual = self.G * self.N * tp                        # so that a rank's share is its G groups
        self.in_proj = ColumnParallelLinear(pf, f"{p}.in_proj", cfg.hidden_size,
                                            [self.I_total, self.I_total, gn_virtual, gn_virtual, self.H_total], comm,
                                            bias=bool(m.get("proj_bias", False)))
        self.out_proj = RowParallelLinear(pf, f"{p}.out_proj", self.I_total, cfg.hidden_size, comm,
                                          bias=bool(m.get("proj_bias", False)))
        self.conv_weight = pf.normal(f"{p}.conv1d.w", (self.conv_dim, self.K), std=0.3).contiguous()
        self.conv_bias = pf.zeros((self.conv_dim,)) if m.get("conv_bias", True) else None
        self.dt_bias = pf.normal(f"{p}.dt_bias", (self.H_total,), 0, r, tp, std=0.5, dtype=torch.float32)
        self.A_log = pf.normal(f"{p}.A_log", (self.H_total,), 0, r, tp, std=0.5, dtype=torch.float32)
        self.D = pf.ones((self.H,), dtype=torch.float32)
        self.norm_weight = pf.ones((self.I,))
        self.chunk = int(m.get("chunk_size", 64)) if int(m.get("chunk_size", 64)) <= 128 else 64

    def state_shapes(self, num_slots: int):
        """(conv state, recurrent state) shapes for ``num_slots`` sequences."""
        return (num_slots, self.K - 1, self.conv_dim), (num_slots, self.H, self.N, self.P)

    def __call__(self, x: torch.Tensor, meta, cache) -> torch.Tensor:
        conv_state, ssm_state = cache
        T = x.shape[0]
        proj = self.in_proj(x)
        I, GN = self.I, self.G * self.N
        z = proj[:, :I]
        xbc = proj[:, I:I + self.conv_dim]
        dt = proj[:, I + self.conv_dim:]
        cu, slots, has_init = meta.query_start_loc, meta.state_slots, meta.has_initial_state
        xbc = la.causal_conv1d(xbc.contiguous(), self.conv_weight, self.conv_bias, conv_state, cu, slots, has_init,
                               act=True)
        xs = xbc[:, :I].reshape(T, self.H, self.P)
        B = xbc[:, I:I + GN].reshape(T, self.G, self.N)
        C = xbc[:, I + GN:].reshape(T, self.G, self.N)
        dt = F.softplus(dt.float() + self.dt_bias)
        dt = torch.clamp(dt, self.dt_limit[0], self.dt_limit[1])
        g = dt * (-torch.exp(self.A_log))                                   # [T, H] log-decay
        v = xs.float() * dt.unsqueeze(-1)
        y = la.gated_linear_attention(C, B, v, g, ssm_state, cu, slots, has_init,
                                      cu_cpu=meta.query_start_loc_cpu, chunk=self.chunk)
        y = y + self.D.view(1, self.H, 1) * xs.float()
        # gated RMSNorm over the whole inner width (all ranks' heads)
        h = y.reshape(T, I) * F.silu(z.float())
        ss = (h * h).sum(-1, keepdim=True)
        if self.comm.size > 1:
            ss = self.comm.group.all_reduce(ss)
        h = (h * torch.rsqrt(ss / self.I_total + self.eps)).to(x.dtype) * self.norm_weight
        return self.out_proj(h)

    # ------------------------------------------------------------------ checkpoints
    def _rows(self, tp: int, r: int):
        """Row ranges of the checkpoint's [z | x | B | C | dt] projection this rank holds."""
        It, GNt, Ht = self.I_total, self.G_total * self.N, self.H_total
        gn = self.G * self.N
        return [(r * self.I, self.I), (It + r * self.I, self.I),
                (2 * It + self.g0 * self.N, gn), (2 * It + GNt + self.g0 * self.N, gn),
                (2 * It + 2 * GNt + r * self.H, self.H)]

    def load_hf(self, suffix: str, w: torch.Tensor, tp: int, r: int) -> bool:
        """One tensor of a published checkpoint (name relative to ``mamba.``)."""
        It, GNt = self.I_total, self.G_total * self.N
        if suffix in ("in_proj.weight", "in_proj.bias"):
            dst = self.in_proj.weight if suffix.endswith("weight") else self.in_proj.bias
            dst.copy_(torch.cat([w[a:a + n] for a, n in self._rows(tp, r)], dim=0))
        elif suffix in ("conv1d.weight", "conv1d.bias"):
            c = w.reshape(w.shape[0], -1) if suffix.endswith("weight") else w
            gn = self.G * self.N
            parts = [c[r * self.I:(r + 1) * self.I], c[It + self.g0 * self.N:It + self.g0 * self.N + gn],
                     c[It + GNt + self.g0 * self.N:It + GNt + self.g0 * self.N + gn]]
            (self.conv_weight if suffix.endswith("weight") else self.conv_bias).copy_(torch.cat(parts, dim=0))
        elif suffix in ("dt_bias", "A_log", "D"):
            getattr(self, suffix).copy_(w[r * self.H:(r + 1) * self.H].to(torch.float32))
        elif suffix == "norm.weight":
            self.norm_weight.copy_(w[r * self.I:(r + 1) * self.I])
        elif suffix == "out_proj.weight":
            self.out_proj.weight.copy_(w[:, r * self.I:(r + 1) * self.I])
        elif suffix == "out_proj.bias":
            self.out_proj.bias.copy_(w)
        else:
            return False
        return True

    def named_tensors(self):
        for attr in ("in_proj", "out_proj"):
            for n, t in getattr(self, attr).named_tensors():
                yield f"{attr}.{n}", t
        yield "conv1d.weight", self.conv_weight
        if self.conv_bias is not None:
            yield "conv1d.bias", self.conv_bias
        yield "dt_bias", self.dt_bias
        yield "A_log", self.A_log
        yield "D", self.D
        yield "norm.weight", self.norm_weight
