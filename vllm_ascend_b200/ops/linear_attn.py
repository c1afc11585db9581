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


def gated_delta_rule_chunked(q, k, v, g, beta, state, cu_cpu, slots, has_init, scale, l2norm=True,
                             chunk=64, seqs=None, out=None):
    """The gated delta rule in its chunk-parallel form (same contract as ``gated_delta_rule_ref``;
    ``cu_cpu``: host sequence boundaries, ``seqs``: indices of the sequences to process, default all;
    rows of other sequences in ``out`` are left alone).

    A chunk of C tokens with log-decays g, cumulative gamma_i = sum_{j<=i} g_j, entered with state S0:

        u_j = beta_j (v_j - e^{gamma_j} S0^T k_j - sum_{m<j} e^{gamma_j - gamma_m} (k_m . k_j) u_m)
        o_i = e^{gamma_i} S0^T q_i + sum_{j<=i} e^{gamma_i - gamma_j} (k_j . q_i) u_j
        S_C = e^{gamma_C} S0 + sum_j e^{gamma_C - gamma_j} k_j u_j^T

    The first line is a unit-lower-triangular system (I + A) U = beta (V - e^gamma K S0) with
    A = strict_lower(beta (K K^T) * Gamma), so U = U' - W S0 with U' and W solved once per chunk,
    for every chunk of every sequence at once.  What stays sequential is three small matrix
    products per chunk position (all sequences that have such a chunk batched together), instead
    of one state update per token: the form the reference uses for prefill
    (vllm_ascend/ops/triton/fla/chunk.py:259, chunk_gated_delta_rule)."""
    import numpy as np
    T, Hv, DV = v.shape
    Hk, DK = q.shape[1], q.shape[2]
    rep = Hv // Hk
    dev = q.device
    cu_cpu = np.asarray(cu_cpu, dtype=np.int64)
    seqs = np.arange(len(cu_cpu) - 1) if seqs is None else np.asarray(seqs, dtype=np.int64)
    if out is None:
        out = torch.empty((T, Hv, DV), dtype=v.dtype, device=dev)
    lens = cu_cpu[seqs + 1] - cu_cpu[seqs]
    keep = lens > 0
    seqs, lens = seqs[keep], lens[keep]
    if seqs.size == 0:
        return out
    order = np.argsort(-lens, kind="stable")          # longest first: the scan's live set is a prefix
    seqs, lens = seqs[order], lens[order]
    C = int(chunk)
    nch = (lens + C - 1) // C
    first = np.concatenate([[0], np.cumsum(nch)[:-1]])           # first chunk id of each sequence
    Nc = int(nch.sum())
    tok = np.full((Nc, C), -1, dtype=np.int64)
    for b, (sq, n) in enumerate(zip(seqs, lens)):
        ids = np.arange(cu_cpu[sq], cu_cpu[sq] + n)
        flat = tok[first[b]:first[b] + nch[b]].reshape(-1)
        flat[:n] = ids
    tok_t = torch.from_numpy(tok).to(dev)
    valid = tok_t >= 0
    gather = tok_t.clamp(min=0).reshape(-1)
    vmask = valid.reshape(-1, 1, 1).float()

    qf, kf = q.float(), k.float()
    if l2norm:
        qf = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6)
        kf = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)

    def chunks(x, heads, dim):          # [T, heads, dim] -> [Nc, heads, C, dim], padding rows zero
        return (x[gather] * vmask).reshape(Nc, C, heads, dim).permute(0, 2, 1, 3)
    Qc = chunks(qf * scale, Hk, DK)
    Kc = chunks(kf, Hk, DK)
    Vc = chunks(v.float(), Hv, DV)
    vm2 = valid.reshape(-1, 1).float()
    gc = (g.float()[gather] * vm2).reshape(Nc, C, Hv).permute(0, 2, 1)          # [Nc, Hv, C]
    bc = (beta.float()[gather] * vm2).reshape(Nc, C, Hv).permute(0, 2, 1)
    gamma = gc.cumsum(-1)
    tri = torch.ones(C, C, dtype=torch.bool, device=dev).tril()                 # j >= m
    diff = gamma.unsqueeze(-1) - gamma.unsqueeze(-2)                            # gamma_j - gamma_m
    Gam = torch.where(tri, diff, torch.full_like(diff, float("-inf"))).exp()    # 0 above the diagonal
    KK = (Kc @ Kc.transpose(-1, -2)).repeat_interleave(rep, dim=1)              # [Nc, Hv, C, C]
    QK = (Qc @ Kc.transpose(-1, -2)).repeat_interleave(rep, dim=1)
    A = (bc.unsqueeze(-1) * KK * Gam).tril(-1)
    Kv = Kc.repeat_interleave(rep, dim=1)                                       # [Nc, Hv, C, DK]
    eg = gamma.exp().unsqueeze(-1)
    rhs = torch.cat([bc.unsqueeze(-1) * Vc, (bc.unsqueeze(-1) * eg) * Kv], dim=-1)
    eye = torch.eye(C, device=dev, dtype=torch.float32)
    sol = torch.linalg.solve_triangular(A + eye, rhs, upper=False, unitriangular=True)
    Up, W = sol[..., :DV], sol[..., DV:]                                        # U', W
    Aqk = QK * Gam                                                              # lower incl. diagonal
    Qg = Qc.repeat_interleave(rep, dim=1) * eg
    g_last = gamma[..., -1:]
    Kd = Kv * (g_last - gamma).exp().unsqueeze(-1)
    decay = g_last.exp().unsqueeze(-1)                                          # [Nc, Hv, 1, 1]

    sl = slots[torch.from_numpy(seqs).to(dev)].long()
    init = has_init[torch.from_numpy(seqs).to(dev)].reshape(-1, 1, 1, 1).to(torch.float32)
    S = state[sl].float() * (init != 0).float()                                 # [ns, Hv, DK, DV]
    O = torch.empty((Nc, Hv, C, DV), dtype=torch.float32, device=dev)
    first_t = torch.from_numpy(first).to(dev)
    for i in range(int(nch.max())):
        live = int((nch > i).sum())                 # sequences 0..live-1 have an i-th chunk
        ids = first_t[:live] + i
        Si = S[:live]
        U = Up[ids] - W[ids] @ Si
        O[ids] = Qg[ids] @ Si + Aqk[ids] @ U
        S[:live] = decay[ids] * Si + Kd[ids].transpose(-1, -2) @ U
    state[sl] = S.to(state.dtype)
    rows = O.permute(0, 2, 1, 3).reshape(Nc * C, Hv, DV)
    sel = valid.reshape(-1)
    out[gather[sel]] = rows[sel].to(out.dtype)
    return out


def _chunk_min(on_cuda: bool = False) -> int:
    """Fewest new tokens of a sequence that take the chunk-parallel form; 0 = never.  Unset, the
    form serves host tensors only: on a B200 the recurrence kernel runs 4 x 2048 tokens of 32 heads in
    3.3 ms, the chunk-parallel form built from fp32 matrix products in 10.3 ms."""
    import os
    from .. import envs
    if "VLLM_B200_GDN_CHUNK_MIN" not in os.environ and on_cuda:
        return 0
    return int(envs.VLLM_B200_GDN_CHUNK_MIN)


def gated_delta_rule(q, k, v, g, beta, state, cu, slots, has_init, scale, l2norm=True, cu_cpu=None):
    """``cu_cpu`` (host copy of ``cu``) lets long sequences (>= ``VLLM_B200_GDN_CHUNK_MIN`` new tokens:
    prefill chunks) take the chunk-parallel form while decode and verification rows stay on the
    per-token recurrence."""
    cmin = _chunk_min(q.is_cuda) if cu_cpu is not None else 0
    if cmin > 0:
        import numpy as np
        cu_h = np.asarray(cu_cpu, dtype=np.int64)[:cu.numel()]
        lens = np.diff(cu_h)
        long_ = np.nonzero(lens >= cmin)[0]
        if long_.size:
            out = torch.empty(v.shape, dtype=v.dtype, device=v.device)
            gated_delta_rule_chunked(q, k, v, g, beta, state, cu_h, slots, has_init, scale, l2norm,
                                     seqs=long_, out=out)
            short = np.nonzero((lens < cmin) & (lens > 0))[0]
            if short.size:
                rows = np.concatenate([np.arange(cu_h[b], cu_h[b + 1]) for b in short])
                rows_t = torch.from_numpy(rows).to(q.device)
                sel = torch.from_numpy(short).to(q.device)
                cu_s = torch.from_numpy(np.concatenate([[0], np.cumsum(lens[short])]).astype(np.int32)).to(q.device)
                out[rows_t] = gated_delta_rule(q[rows_t].contiguous(), k[rows_t].contiguous(), v[rows_t].contiguous(),
                                               g[rows_t], beta[rows_t], state, cu_s, slots[sel].contiguous(),
                                               has_init[sel].contiguous(), scale, l2norm)
            return out
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


# ---------------------------------------------------------------------------- lightning attention
def lightning_attention_ref(q, k, v, log_decay, state, cu, slots, has_init):
    """Linear attention with a fixed per-head decay (MiniMax-Text-01, Bailing linear layers):

        S_t = e^{-lambda_h} S_{t-1} + k_t v_t^T          o_t = S_t^T q_t

    q, k, v [T, H, D]; ``log_decay`` [H] = -lambda_h; state [slots, H, D, D] fp32 (in place).
    Token by token: the definition the other forms are tested against."""
    T, H, D = q.shape
    out = torch.empty((T, H, v.shape[-1]), dtype=v.dtype, device=v.device)
    ratio = torch.exp(log_decay.float()).view(H, 1, 1)
    cu_l = cu.tolist()
    for b in range(len(cu_l) - 1):
        s = int(slots[b])
        S = state[s].clone() if bool(has_init[b]) else torch.zeros_like(state[s])
        for t in range(cu_l[b], cu_l[b + 1]):
            S = ratio * S + k[t].float()[:, :, None] * v[t].float()[:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, q[t].float()).to(out.dtype)
        if cu_l[b + 1] > cu_l[b]:
            state[s] = S
    return out


def gated_linear_attention_ref(q, k, v, g, state, cu, slots, has_init):
    """S_t = e^{g_t} S_{t-1} + k_t v_t^T, o_t = S_t^T q_t with a scalar log-decay per token and head.
    q, k [T, Hk, N] (Hk divides H: grouped keys / queries), v [T, H, P], g [T, H];
    state [slots, H, N, P] fp32 (in place).  Token by token."""
    T, H, P = v.shape
    rep = H // q.shape[1]
    out = torch.empty((T, H, P), dtype=v.dtype, device=v.device)
    qf = q.float().repeat_interleave(rep, dim=1)
    kf = k.float().repeat_interleave(rep, dim=1)
    cu_l = cu.tolist()
    for b in range(len(cu_l) - 1):
        s = int(slots[b])
        S = state[s].clone() if bool(has_init[b]) else torch.zeros_like(state[s])
        for t in range(cu_l[b], cu_l[b + 1]):
            S = torch.exp(g[t].float()).view(H, 1, 1) * S + kf[t][:, :, None] * v[t].float()[:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, qf[t]).to(out.dtype)
        if cu_l[b + 1] > cu_l[b]:
            state[s] = S
    return out


def gated_linear_attention(q, k, v, g, state, cu, slots, has_init, cu_cpu, chunk=64):
    """Same contract as ``gated_linear_attention_ref``, two batched forms chosen per sequence from
    the host copy of ``cu``:

    * one new token (decode): every such sequence in one batched update
      S = e^g S + k v^T, o = S^T q (no per-sequence work on the host);
    * more tokens (prefill chunks, verification): chunks of ``chunk`` tokens with cumulative
      log-decay gamma_i inside the chunk,
      O = (Q K^T * e^{gamma_i - gamma_j} [j <= i]) V + diag(e^{gamma_i}) Q S0 and
      S_C = e^{gamma_C} S0 + (e^{gamma_C - gamma_j} K)^T V,
      all chunks' local products at once and one small update per chunk position.

    This is the state-space-duality form of Mamba-2 (q = C, k = B, v = dt x, g = dt A) and, with a
    constant g per head, lightning attention.  The reference's kernels for these layers are its
    Triton lightning-attention prefill / decode pair and vLLM's Mamba-2 kernels
    (vllm_ascend/ops/triton/mamba/lightning_attn.py, vllm_ascend/ops/triton/mamba/causal_conv1d.py)."""
    import numpy as np
    T, H, DV = v.shape
    Hk, D = q.shape[1], q.shape[2]
    rep = H // Hk
    dev = q.device
    cu_h = np.asarray(cu_cpu, dtype=np.int64)[:cu.numel()]
    lens = np.diff(cu_h)
    out = torch.empty((T, H, DV), dtype=v.dtype, device=dev)
    gf = g.float()
    ones = np.nonzero(lens == 1)[0]
    if ones.size:
        rows = torch.from_numpy(cu_h[ones]).to(dev)
        sel = torch.from_numpy(ones).to(dev)
        sl = slots[sel].long()
        init = (has_init[sel] != 0).float().view(-1, 1, 1, 1)
        S = state[sl].float() * init
        kr = k[rows].float().repeat_interleave(rep, dim=1)
        S = torch.exp(gf[rows]).view(-1, H, 1, 1) * S + kr.unsqueeze(-1) * v[rows].float().unsqueeze(-2)
        out[rows] = torch.einsum("bhkv,bhk->bhv", S, q[rows].float().repeat_interleave(rep, dim=1)).to(out.dtype)
        state[sl] = S.to(state.dtype)
    many = np.nonzero(lens > 1)[0]
    if many.size == 0:
        return out
    order = np.argsort(-lens[many], kind="stable")
    seqs, ln = many[order], lens[many][order]
    C = int(chunk)
    nch = (ln + C - 1) // C
    first = np.concatenate([[0], np.cumsum(nch)[:-1]])
    Nc = int(nch.sum())
    tok = np.full((Nc, C), -1, dtype=np.int64)
    for b, (sq, n) in enumerate(zip(seqs, ln)):
        tok[first[b]:first[b] + nch[b]].reshape(-1)[:n] = np.arange(cu_h[sq], cu_h[sq] + n)
    tok_t = torch.from_numpy(tok).to(dev)
    valid = tok_t >= 0
    gather = tok_t.clamp(min=0).reshape(-1)
    vmask = valid.reshape(-1, 1, 1).float()

    def chunks(x, heads, dim):
        return (x.float()[gather] * vmask).reshape(Nc, C, heads, dim).permute(0, 2, 1, 3)      # [Nc, heads, C, dim]
    Qc, Kc, Vc = chunks(q, Hk, D), chunks(k, Hk, D), chunks(v, H, DV)
    gc = (gf[gather] * valid.reshape(-1, 1).float()).reshape(Nc, C, H).permute(0, 2, 1)         # padding: no decay
    gamma = gc.cumsum(-1)                                                                       # [Nc, H, C]
    tri = torch.ones(C, C, dtype=torch.bool, device=dev).tril()
    diff = gamma.unsqueeze(-1) - gamma.unsqueeze(-2)
    Gam = torch.where(tri, diff, torch.full_like(diff, float("-inf"))).exp()                    # 0 above the diagonal
    QK = (Qc @ Kc.transpose(-1, -2)).repeat_interleave(rep, dim=1)                              # [Nc, H, C, C]
    intra = (QK * Gam) @ Vc
    Qd = Qc.repeat_interleave(rep, dim=1) * gamma.exp().unsqueeze(-1)
    g_last = gamma[..., -1:]
    Kd = Kc.repeat_interleave(rep, dim=1) * (g_last - gamma).exp().unsqueeze(-1)
    KV = Kd.transpose(-1, -2) @ Vc                                                              # [Nc, H, D, DV]
    block = g_last.exp().unsqueeze(-1)                                                          # [Nc, H, 1, 1]

    sel = torch.from_numpy(seqs).to(dev)
    sl = slots[sel].long()
    S = state[sl].float() * (has_init[sel] != 0).float().view(-1, 1, 1, 1)
    O = torch.empty((Nc, H, C, DV), dtype=torch.float32, device=dev)
    first_t = torch.from_numpy(first).to(dev)
    for i in range(int(nch.max())):
        live = int((nch > i).sum())
        ids = first_t[:live] + i
        Si = S[:live]
        O[ids] = intra[ids] + Qd[ids] @ Si
        S[:live] = block[ids] * Si + KV[ids]
    state[sl] = S.to(state.dtype)
    rows = O.permute(0, 2, 1, 3).reshape(Nc * C, H, DV)
    keep = valid.reshape(-1)
    out[gather[keep]] = rows[keep].to(out.dtype)
    return out


def lightning_attention(q, k, v, log_decay, state, cu, slots, has_init, cu_cpu, chunk=64):
    """Lightning attention through the batched forms of ``gated_linear_attention``: the log-decay
    of a token is its head's constant."""
    g = log_decay.float().to(q.device).view(1, -1).expand(q.shape[0], -1)
    return gated_linear_attention(q, k, v, g, state, cu, slots, has_init, cu_cpu, chunk)


# ---------------------------------------------------------------------------- KDA (delta rule, per-channel decay)
def kda_recurrent_ref(q, k, v, g, beta, state, cu, slots, has_init, scale, l2norm=True):
    """Delta rule whose decay is a vector over the key channels (Kimi delta attention):

        S_t = diag(e^{g_t}) S_{t-1};  u_t = beta_t (v_t - S_t^T k_t);  S_t += k_t u_t^T;  o_t = S_t^T q_t

    q, k [T, H, DK]; v [T, H, DV]; g [T, H, DK] (log-decay per key channel); beta [T, H];
    state [slots, H, DK, DV] fp32 (in place).  Token by token
    (vllm_ascend/ops/triton/kda/fused_recurrent_kda.py:98-136 is the same recurrence as a kernel)."""
    T, H, DV = v.shape
    out = torch.empty((T, H, DV), dtype=v.dtype, device=v.device)
    qf, kf = q.float(), k.float()
    if l2norm:
        qf = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6)
        kf = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
    qf = qf * scale
    cu_l = cu.tolist()
    for b in range(len(cu_l) - 1):
        s = int(slots[b])
        S = state[s].clone() if bool(has_init[b]) else torch.zeros_like(state[s])
        for t in range(cu_l[b], cu_l[b + 1]):
            S = S * torch.exp(g[t].float())[:, :, None]
            u = (v[t].float() - torch.einsum("hkv,hk->hv", S, kf[t])) * beta[t].float()[:, None]
            S = S + kf[t][:, :, None] * u[:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, qf[t]).to(out.dtype)
        if cu_l[b + 1] > cu_l[b]:
            state[s] = S
    return out


def kda_chunked(q, k, v, g, beta, state, cu_cpu, slots, has_init, scale, l2norm=True, chunk=16):
    """Chunk-parallel form of ``kda_recurrent_ref`` for one step's sequences (host boundaries
    ``cu_cpu``).  As for the scalar-gated rule, U solves a unit-lower-triangular system per chunk; the
    pairwise decays e^{gamma_j - gamma_m} differ per key channel, so the chunk-local products are
    contractions over (channel) of k_j k_m e^{gamma_j - gamma_m}, formed exactly (only non-positive
    exponents are ever exponentiated) for a short chunk
    (vllm_ascend/ops/triton/kda/kda.py, chunk_delta_h.py, solve_tril.py are the reference's kernels)."""
    import numpy as np
    T, H, DV = v.shape
    DK = q.shape[2]
    dev = q.device
    cu_h = np.asarray(cu_cpu, dtype=np.int64)
    out = torch.empty((T, H, DV), dtype=v.dtype, device=dev)
    qf, kf = q.float(), k.float()
    if l2norm:
        qf = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6)
        kf = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
    qf = qf * scale
    C = int(chunk)
    tri = torch.ones(C, C, dtype=torch.bool, device=dev).tril()
    eye = torch.eye(C, device=dev)
    for b in range(len(cu_h) - 1):
        t0, t1 = int(cu_h[b]), int(cu_h[b + 1])
        if t1 <= t0:
            continue
        s = int(slots[b])
        S = state[s].float().clone() if bool(has_init[b]) else torch.zeros_like(state[s], dtype=torch.float32)
        for c0 in range(t0, t1, C):
            c1 = min(c0 + C, t1)
            n = c1 - c0
            Q, K, V = (x[c0:c1].permute(1, 0, 2) for x in (qf, kf, v.float()))            # [H, n, *]
            G = g[c0:c1].float().permute(1, 0, 2).cumsum(1)                               # gamma [H, n, DK]
            Bt = beta[c0:c1].float().t()                                                  # [H, n]
            diff = G.unsqueeze(2) - G.unsqueeze(1)                                        # gamma_j - gamma_m [H, n, n, DK]
            dec = torch.where(tri[:n, :n, None], diff, torch.full_like(diff, float("-inf"))).exp()
            KK = torch.einsum("hjd,hmd,hjmd->hjm", K, K, dec)
            QK = torch.einsum("hjd,hmd,hjmd->hjm", Q, K, dec)
            A = (Bt.unsqueeze(-1) * KK).tril(-1)
            eG = G.exp()                                                                   # e^{gamma_j}, per channel
            rhs = torch.cat([Bt.unsqueeze(-1) * V, Bt.unsqueeze(-1) * (K * eG)], dim=-1)
            sol = torch.linalg.solve_triangular(A + eye[:n, :n], rhs, upper=False, unitriangular=True)
            U = sol[..., :DV] - sol[..., DV:] @ S                                          # [H, n, DV]
            O = (Q * eG) @ S + QK @ U
            out[c0:c1] = O.permute(1, 0, 2).to(out.dtype)
            last = G[:, -1:, :]
            S = last.transpose(1, 2).exp() * S + (K * (last - G).exp()).transpose(1, 2) @ U
        state[s] = S.to(state.dtype)
    return out
