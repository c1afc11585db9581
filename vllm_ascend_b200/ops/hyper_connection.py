"""Manifold-constrained hyper-connections: the residual stream of a decoder is widened to ``m``
parallel streams [T, m, H]; every sub-layer reads a learned mixture of them and writes its output
back through learned, input-dependent weights.

``hc_pre``  (before a sub-layer): the flattened streams are RMS-normalised and projected to
(2 + m) m mixing logits.  From them: read weights ``pre`` [m] = sigmoid(.) + eps (the sub-layer's
input is sum_i pre_i x_i), write weights ``post`` [m] = 2 sigmoid(.), and a stream-mixing matrix
``comb`` [m, m] that is made (approximately) doubly stochastic by a softmax followed by Sinkhorn
iterations (alternating row / column normalisation), so that mixing neither amplifies nor loses the
residual signal.
``hc_post`` (after it):  out_i = post_i f(x) + sum_j comb[j, i] x_j.
``hc_head`` (after the last layer): the streams are merged by read weights only.

Semantics of the reference's fused ops ``npu_hc_pre_v2`` / ``npu_hc_post`` and of ``hc_head`` as
its DeepSeek-V4 model uses them (vllm_ascend/models/deepseek_v4/model.py:692-726, 837-844;
csrc/moe/hc_post/op_kernel/hc_post_bfloat16.h; golden definition in
tests/e2e/nightly/single_node/ops/singlecard_ops/test_npu_hc_pre.py).  Plain PyTorch on either
device: m is 2..4, the work is a skinny fp32 GEMM and a handful of element-wise passes.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def sinkhorn(comb: torch.Tensor, iters: int, eps: float) -> torch.Tensor:
    """[..., m, m] logits -> approximately doubly stochastic matrix."""
    c = comb.softmax(-1) + eps
    c = c / (c.sum(-2, keepdim=True) + eps)
    for _ in range(max(iters - 1, 0)):
        c = c / (c.sum(-1, keepdim=True) + eps)
        c = c / (c.sum(-2, keepdim=True) + eps)
    return c


def hc_pre(x: torch.Tensor, hc_fn: torch.Tensor, hc_scale: torch.Tensor, hc_base: torch.Tensor, m: int,
           sinkhorn_iters: int = 20, norm_eps: float = 1e-6, hc_eps: float = 1e-6):
    """x [T, m, H]; hc_fn [(2 + m) m, m H] fp32; hc_scale [3]; hc_base [(2 + m) m].
    Returns (y [T, H] in x's dtype, post [T, m] fp32, comb [T, m, m] fp32)."""
    xf = x.float()
    flat = xf.flatten(-2)
    inv_rms = torch.rsqrt(flat.square().mean(-1, keepdim=True) + norm_eps)
    mixes = F.linear(flat, hc_fn.float()) * inv_rms
    pre, post, comb = mixes.split([m, m, m * m], dim=-1)
    pre = torch.sigmoid(pre * hc_scale[0] + hc_base[:m]) + hc_eps
    post = 2 * torch.sigmoid(post * hc_scale[1] + hc_base[m:2 * m])
    comb = comb.unflatten(-1, (m, m)) * hc_scale[2] + hc_base[2 * m:].view(m, m)
    comb = sinkhorn(comb, sinkhorn_iters, hc_eps)
    y = (pre.unsqueeze(-1) * xf).sum(dim=-2).to(x.dtype)
    return y, post, comb


def hc_post(y: torch.Tensor, residual: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """y [T, H] (sub-layer output), residual [T, m, H] (the streams the sub-layer read),
    post [T, m], comb [T, m, m] -> new streams [T, m, H]."""
    out = post.unsqueeze(-1) * y.float().unsqueeze(-2) + comb.transpose(-1, -2) @ residual.float()
    return out.to(residual.dtype)


def hc_head(x: torch.Tensor, hc_fn: torch.Tensor, hc_scale: torch.Tensor, hc_base: torch.Tensor,
            norm_eps: float = 1e-6, hc_eps: float = 1e-6) -> torch.Tensor:
    """x [T, m, H]; hc_fn [m, m H]; hc_scale [1]; hc_base [m] -> [T, H]."""
    xf = x.float()
    flat = xf.flatten(-2)
    inv_rms = torch.rsqrt(flat.square().mean(-1, keepdim=True) + norm_eps)
    pre = torch.sigmoid(F.linear(flat, hc_fn.float()) * inv_rms * hc_scale + hc_base) + hc_eps
    return (pre.unsqueeze(-1) * xf).sum(dim=-2).to(x.dtype)


class HyperConnection:
    """Parameters of one sub-layer's hyper-connection and the two calls around the sub-layer."""

    def __init__(self, pf, name: str, hidden: int, m: int, sinkhorn_iters: int, norm_eps: float, hc_eps: float = 1e-6):
        self.m, self.iters, self.norm_eps, self.hc_eps = m, sinkhorn_iters, norm_eps, hc_eps
        mix = (2 + m) * m
        self.fn = pf.normal(f"{name}_fn", (mix, m * hidden), std=1.0 / (m * hidden) ** 0.5, dtype=torch.float32)
        self.base = pf.zeros((mix,), dtype=torch.float32)
        self.scale = pf.ones((3,), dtype=torch.float32)

    def pre(self, streams: torch.Tensor):
        return hc_pre(streams, self.fn, self.scale, self.base, self.m, self.iters, self.norm_eps, self.hc_eps)

    @staticmethod
    def post(y, streams, post, comb):
        return hc_post(y, streams, post, comb)

    def named_tensors(self, name: str):
        yield f"{name}_fn", self.fn
        yield f"{name}_base", self.base
        yield f"{name}_scale", self.scale
