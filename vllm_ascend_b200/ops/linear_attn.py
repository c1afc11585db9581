"""Linear-attention ops (Gated DeltaNet): causal short convolution with state, and the gated
delta-rule recurrence; CUDA kernels on GPU tensors, PyTorch definitions otherwise
(vllm_ascend/ops/gdn.py, ops/triton/fla/*, csrc/moe/causal_conv1d*,
csrc/attention/recurrent_gated_delta_rule*)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_void_p

import torch
import torch.nn.functional as F

from .. import _native

P, I, L, Fl = c_void_p, c_int, c_long, c_float
_native.register_signature("b200_causal_conv1d", [P, L, P, P, P, P, P, P, P, L, I, I, I, I, L, P, P])
_native.register_signature("b200_gated_delta_rule", [P, P, P, L, L, P, P, P, P, P, P, P, L, I, I, I, I, I, Fl, I,
                                                     L, P, P])


def causal_conv1d_ref(x, weight, bias, state, cu, slots, has_init, act=True):
    """x [T, C], weight [C, K], state [slots, K-1, C] (updated in place) -> y [T, C]."""
    K = weight.shape[1]
    y = torch.empty_like(x)
    cu_l = cu.tolist()
    for b in range(len(cu_l) - 1):
        t0, t1 = cu_l[b], cu_l[b + 1]
        s = int(slots[b])
        hist = state[s].float() if bool(has_init[b]) else torch.zeros(K - 1, x.shape[1], device=x.device)
        seq = torch.cat([hist, x[t0:t1].float()], dim=0)                     # [K-1+n, C]
        win = seq.unfold(0, K, 1)                                           # [n, C, K]
        out = (win * weight.float().unsqueeze(0)).sum(-1)
        if bias is not None:
            out = out + bias.float()
        y[t0:t1] = (F.silu(out) if act else out).to(x.dtype)
        state[s] = seq[-(K - 1):].to(state.dtype)
    return y


def causal_conv1d(x, weight, bias, state, cu, slots, has_init, act=True):
    if not (x.is_cuda and x.dtype == torch.bfloat16):
        return causal_conv1d_ref(x, weight, bias, state, cu, slots, has_init, act)
    T, C = x.shape
    y = torch.empty((T, C), dtype=x.dtype, device=x.device)
    rc = _native.lib().b200_causal_conv1d(
        x.data_ptr(), x.stride(0), weight.data_ptr(), _native.ptr(bias), state.data_ptr(), cu.data_ptr(),
        slots.data_ptr(), has_init.data_ptr(), y.data_ptr(), y.stride(0), cu.numel() - 1, C, weight.shape[1],
        int(act), state.shape[0], _native.status_word(x.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "causal_conv1d")
    _native.count_launch()
    return y


def gated_delta_rule_ref(q, k, v, g, beta, state, cu, slots, has_init, scale, l2norm=True):
    """q, k [T, Hk, DK]; v [T, Hv, DV]; g, beta [T, Hv]; state [slots, Hv, DK, DV] fp32 (in place)."""
    T, Hv, DV = v.shape
    Hk = q.shape[1]
    rep = Hv // Hk
    out = torch.empty((T, Hv, DV), dtype=v.dtype, device=v.device)
    qf, kf = q.float(), k.float()
    if l2norm:
        qf = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6)
        kf = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
    qf = qf.repeat_interleave(rep, dim=1) * scale
    kf = kf.repeat_interleave(rep, dim=1)
    cu_l = cu.tolist()
    for b in range(len(cu_l) - 1):
        s = int(slots[b])
        S = state[s].clone() if bool(has_init[b]) else torch.zeros_like(state[s])
        for t in range(cu_l[b], cu_l[b + 1]):
            S = S * torch.exp(g[t].float())[:, None, None]
            mem = torch.einsum("hkv,hk->hv", S, kf[t])
            delta = (v[t].float() - mem) * beta[t].float()[:, None]
            S = S + kf[t][:, :, None] * delta[:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, qf[t]).to(out.dtype)
        state[s] = S
    return out


def gated_delta_rule(q, k, v, g, beta, state, cu, slots, has_init, scale, l2norm=True):
    if not (q.is_cuda and q.dtype == torch.bfloat16):
        return gated_delta_rule_ref(q, k, v, g, beta, state, cu, slots, has_init, scale, l2norm)
    T, Hv, DV = v.shape
    Hk, DK = q.shape[1], q.shape[2]
    assert q.stride(0) == k.stride(0) and q.stride(2) == 1 and q.stride(1) == DK and v.stride(1) == DV
    out = torch.empty((T, Hv, DV), dtype=v.dtype, device=v.device)
    g = g.float().contiguous()
    beta = beta.float().contiguous()
    rc = _native.lib().b200_gated_delta_rule(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), v.stride(0), g.data_ptr(), beta.data_ptr(),
        state.data_ptr(), cu.data_ptr(), slots.data_ptr(), has_init.data_ptr(), out.data_ptr(), out.stride(0),
        cu.numel() - 1, Hk, Hv, DK, DV, scale, int(l2norm), state.shape[0],
        _native.status_word(q.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "gated_delta_rule")
    _native.count_launch()
    return out
