"""Plain PyTorch restatements of every op.

They are (a) the execution path for CPU tensors (the tiny fp32 correctness
config runs entirely through them) and (b) the fp32 oracle the GPU kernel tests
compare against — the same role numpy goldens play in the reference's op tests
(tests/e2e/nightly/single_node/ops/singlecard_ops/*).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float,
             residual: Optional[torch.Tensor] = None, gemma: bool = False):
    orig = x.dtype
    if residual is not None:
        z = (x.float() + residual.float()).to(orig)
        residual = z
        xf = z.float()
    else:
        xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    w = weight.float() + 1.0 if gemma else weight.float()
    out = (xf * torch.rsqrt(var + eps) * w).to(orig)
    return out, residual


def silu_and_mul(x: torch.Tensor, limit: float = 0.0) -> torch.Tensor:
    d = x.shape[-1] // 2
    g, u = x[..., :d].float(), x[..., d:].float()
    if limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    return (F.silu(g) * u).to(x.dtype)


def embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0,
              vocab_end: Optional[int] = None) -> torch.Tensor:
    if vocab_end is None:
        vocab_end = vocab_start + weight.shape[0]
    mask = (ids >= vocab_start) & (ids < vocab_end)
    local = torch.where(mask, ids - vocab_start, torch.zeros_like(ids))
    out = F.embedding(local, weight)
    return out * mask.unsqueeze(-1).to(out.dtype)


def build_cos_sin_cache(rot_dim: int, max_pos: int, theta: float,
                        rope_scaling: Optional[dict] = None,
                        device="cpu") -> torch.Tensor:
    """fp32 [max_pos, rot_dim]: cos in the first half, sin in the second.

    Supports plain RoPE, linear and YaRN scaling (the variants of
    vllm_ascend/ops/rotary_embedding.py:233-578 that change only the table).
    """
    half = rot_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2 / rot_dim))
    mscale = 1.0
    if rope_scaling:
        kind = rope_scaling.get("rope_type", rope_scaling.get("type", "default"))
        factor = float(rope_scaling.get("factor", 1.0))
        if kind == "linear":
            inv_freq = inv_freq / factor
        elif kind in ("yarn", "deepseek_yarn"):
            orig = rope_scaling.get("original_max_position_embeddings", max_pos)
            beta_fast = rope_scaling.get("beta_fast", 32)
            beta_slow = rope_scaling.get("beta_slow", 1)

            def corr_dim(n_rot):
                return (rot_dim * math.log(orig / (n_rot * 2 * math.pi))) / (2 * math.log(theta))

            low = max(math.floor(corr_dim(beta_fast)), 0)
            high = min(math.ceil(corr_dim(beta_slow)), rot_dim - 1)
            if low == high:
                high += 0.001
            ramp = ((torch.arange(half, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
            mask = 1 - ramp
            inv_freq = inv_freq / factor * (1 - mask) + inv_freq * mask

            def yarn_mscale(scale, m=1.0):
                return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

            if kind == "deepseek_yarn":
                mscale = (yarn_mscale(factor, rope_scaling.get("mscale", 1.0)) /
                          yarn_mscale(factor, rope_scaling.get("mscale_all_dim", 0.0) or 1.0)
                          if rope_scaling.get("mscale_all_dim") else
                          yarn_mscale(factor, rope_scaling.get("mscale", 1.0)))
            else:
                mscale = yarn_mscale(factor)
        elif kind == "llama3":
            lo_f = rope_scaling.get("low_freq_factor", 1.0)
            hi_f = rope_scaling.get("high_freq_factor", 4.0)
            orig = rope_scaling.get("original_max_position_embeddings", 8192)
            wavelen = 2 * math.pi / inv_freq
            smooth = ((orig / wavelen) - lo_f) / (hi_f - lo_f)
            scaled = torch.where(wavelen > orig / lo_f, inv_freq / factor, inv_freq)
            mid = (1 - smooth) * inv_freq / factor + smooth * inv_freq
            is_mid = (wavelen <= orig / lo_f) & (wavelen >= orig / hi_f)
            inv_freq = torch.where(is_mid, mid, scaled)
    t = torch.arange(max_pos, dtype=torch.float64)
    freqs = torch.outer(t, inv_freq)
    cache = torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1)
    return cache.float().to(device)


def apply_rope_neox(x: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                    rot_dim: int) -> torch.Tensor:
    """x: [T, H, D]; rotates the first rot_dim dims pairing j with j + rot_dim/2."""
    half = rot_dim // 2
    cs = cos_sin[positions]                       # [T, rot_dim]
    cos, sin = cs[:, :half].unsqueeze(1), cs[:, half:].unsqueeze(1)
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:rot_dim]
    out = xf.clone()
    out[..., :half] = x1 * cos - x2 * sin
    out[..., half:rot_dim] = x2 * cos + x1 * sin
    return out.to(x.dtype)


def mrope_axis_table(sections, interleaved: bool = False) -> torch.Tensor:
    """int32 [sum(sections)]: which position axis (0 temporal, 1 height, 2 width) each rotary
    pair follows.  Sectioned layout: the first sections[0] pairs are temporal, then height, then
    width (Qwen2-VL); interleaved layout: t h w t h w ... with the temporal axis taking what is
    left once height / width are used up (Qwen3-VL).  Follows the index arithmetic of
    vllm_ascend/ops/rotary_embedding.py:582-672 (the mrope paths)."""
    half = int(sum(sections))
    axis = torch.zeros(half, dtype=torch.int32)
    if interleaved:
        for a in (1, 2):
            idx = torch.arange(a, sections[a] * 3, 3)
            axis[idx[idx < half]] = a
    else:
        axis[sections[0]:sections[0] + sections[1]] = 1
        axis[sections[0] + sections[1]:] = 2
    return axis


def apply_mrope_neox(x: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                     rot_dim: int, axis: torch.Tensor) -> torch.Tensor:
    """x: [T, H, D]; positions int64 [3, >=T]; pair e rotates by the angle at positions[axis[e]]."""
    T = x.shape[0]
    half = rot_dim // 2
    pos = positions[:, :T][axis.long()]                      # [half, T]
    e = torch.arange(half, device=x.device).unsqueeze(1)
    cos = cos_sin[pos, e].t().unsqueeze(1)                   # [T, 1, half]
    sin = cos_sin[pos, e + half].t().unsqueeze(1)
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:rot_dim]
    out = xf.clone()
    out[..., :half] = x1 * cos - x2 * sin
    out[..., half:rot_dim] = x2 * cos + x1 * sin
    return out.to(x.dtype)


def apply_rope_interleaved(x: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                           rot_dim: int) -> torch.Tensor:
    """GPT-J style: pairs (2j, 2j+1); used by DeepSeek's rope slice."""
    half = rot_dim // 2
    cs = cos_sin[positions]
    cos, sin = cs[:, :half].unsqueeze(1), cs[:, half:].unsqueeze(1)
    xf = x.float()
    xr = xf[..., :rot_dim]
    x1, x2 = xr[..., 0::2], xr[..., 1::2]
    o1 = x1 * cos - x2 * sin
    o2 = x2 * cos + x1 * sin
    out = xf.clone()
    out[..., :rot_dim] = torch.stack([o1, o2], dim=-1).flatten(-2)
    return out.to(x.dtype)


def qknorm_rope_kvwrite(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                        rot_dim: int, q_norm_w, k_norm_w, eps: float,
                        k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                        slot_mapping: Optional[torch.Tensor], Hq: int, Hkv: int, D: int,
                        mrope_axis: Optional[torch.Tensor] = None) -> None:
    """In place on qkv [T, (Hq+2Hkv)*D]; scatters k, v into the paged caches."""
    T = qkv.shape[0]
    q = qkv[:, :Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    if q_norm_w is not None:
        q.copy_(rms_norm(q, q_norm_w, eps)[0])
    if k_norm_w is not None:
        k.copy_(rms_norm(k, k_norm_w, eps)[0])
    if rot_dim > 0 and mrope_axis is not None:
        q.copy_(apply_mrope_neox(q, positions, cos_sin, rot_dim, mrope_axis))
        k.copy_(apply_mrope_neox(k, positions, cos_sin, rot_dim, mrope_axis))
    elif rot_dim > 0:
        q.copy_(apply_rope_neox(q, positions, cos_sin, rot_dim))
        k.copy_(apply_rope_neox(k, positions, cos_sin, rot_dim))
    if k_cache is not None and slot_mapping is not None:
        valid = slot_mapping >= 0
        slots = slot_mapping[valid]
        bs = k_cache.shape[1]                      # works for any physical layout of the cache
        blk, off = slots // bs, slots % bs
        k_cache[blk, off] = k[valid].to(k_cache.dtype)
        v_cache[blk, off] = v[valid].to(v_cache.dtype)


def gather_kv(cache: torch.Tensor, block_table_row: torch.Tensor, seq_len: int) -> torch.Tensor:
    """cache [NB, BS, H, D] -> [seq_len, H, D] for one sequence."""
    bs = cache.shape[1]
    nblk = (seq_len + bs - 1) // bs
    blocks = block_table_row[:nblk].long()
    return cache[blocks].reshape(nblk * bs, *cache.shape[2:])[:seq_len]


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    query_start_loc, seq_lens, block_table: torch.Tensor, scale: float,
                    causal: bool = True, window: int = 0,
                    out: Optional[torch.Tensor] = None, return_lse: bool = False):
    """q: [T, Hq, D]; every query attends to keys [0, ctx + own_pos] of its sequence."""
    T, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    Dv = v_cache.shape[3]
    G = Hq // Hkv
    if out is None:
        out = torch.empty(T, Hq, Dv, dtype=q.dtype, device=q.device)
    lse_out = torch.full((T, Hq), float("-inf"), dtype=torch.float32, device=q.device)
    qsl = [int(x) for x in query_start_loc]
    sls = [int(x) for x in seq_lens]
    for b in range(len(sls)):
        qs, qe = qsl[b], qsl[b + 1]
        ql = qe - qs
        if ql <= 0:
            continue
        sl = sls[b]
        ctx = sl - ql
        k = gather_kv(k_cache, block_table[b], sl).float()       # [sl, Hkv, D]
        v = gather_kv(v_cache, block_table[b], sl).float()
        qq = q[qs:qe].float()                                     # [ql, Hq, D]
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
        s = torch.einsum("qhd,khd->hqk", qq, k) * scale
        kpos = torch.arange(sl, device=q.device)
        qpos = ctx + torch.arange(ql, device=q.device)
        mask = torch.ones(ql, sl, dtype=torch.bool, device=q.device)
        if causal:
            mask &= kpos[None, :] <= qpos[:, None]
        if window and window > 0:
            mask &= kpos[None, :] > (qpos[:, None] - window)
        s = s.masked_fill(~mask[None], float("-inf"))
        lse = torch.logsumexp(s, dim=-1)                          # [Hq, ql]
        p = torch.exp(s - lse.unsqueeze(-1))
        p = torch.nan_to_num(p, nan=0.0)
        o = torch.einsum("hqk,khd->qhd", p, v)
        out[qs:qe] = o.to(out.dtype)
        lse_out[qs:qe] = lse.transpose(0, 1)
    if return_lse:
        return out, lse_out
    return out


def merge_attn_states(o1, lse1, o2, lse2):
    """LSE merge of two partial attention results ([T,H,D], [T,H])."""
    m = torch.maximum(lse1, lse2)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w1, w2 = torch.exp(lse1 - m), torch.exp(lse2 - m)
    den = (w1 + w2).clamp_min(1e-30)
    o = (o1.float() * (w1 / den).unsqueeze(-1) + o2.float() * (w2 / den).unsqueeze(-1))
    return o.to(o1.dtype), m + torch.log(den)


# ---------------------------------------------------------------- sampling
def apply_penalties(logits: torch.Tensor, prompt_ids: torch.Tensor, output_ids: torch.Tensor,
                    rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> torch.Tensor:
    """logits fp32 [B, V]; id tensors padded with values >= V."""
    B, V = logits.shape
    out_counts = torch.zeros(B, V + 1, dtype=torch.float32, device=logits.device)
    out_counts.scatter_add_(1, output_ids.clamp(min=0, max=V),
                            torch.ones_like(output_ids, dtype=torch.float32))
    out_counts = out_counts[:, :V]
    prompt_mask = torch.zeros(B, V + 1, dtype=torch.bool, device=logits.device)
    prompt_mask.scatter_(1, prompt_ids.clamp(min=0, max=V), True)
    seen = prompt_mask[:, :V] | (out_counts > 0)
    r = rep.unsqueeze(1)
    scaled = torch.where(logits > 0, logits / r, logits * r)
    logits = torch.where(seen, scaled, logits)
    logits = logits - freq.unsqueeze(1) * out_counts - pres.unsqueeze(1) * (out_counts > 0).float()
    return logits


def top_k_top_p_filter(probs: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                       min_p: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sort-based reference: returns the filtered (unnormalised) probabilities."""
    B, V = probs.shape
    sp, si = probs.sort(dim=-1, descending=True)
    ranks = torch.arange(V, device=probs.device).unsqueeze(0)
    k = torch.where((top_k <= 0) | (top_k >= V), torch.full_like(top_k, V), top_k).unsqueeze(1)
    keep = ranks < k
    # ties with the k-th value stay (the radix select keeps them too)
    kth = sp.gather(1, (k - 1).clamp(min=0))
    keep |= sp >= kth
    spk = sp * keep
    mass = spk.sum(-1, keepdim=True)
    cum = spk.cumsum(-1)
    p = top_p.unsqueeze(1)
    keep_p = (cum - spk) < p * mass          # smallest prefix whose mass reaches p
    keep_p[:, 0] = True
    keep &= torch.where(p >= 1.0, torch.ones_like(keep_p), keep_p)
    if min_p is not None:
        keep &= sp >= (min_p.unsqueeze(1) * sp[:, :1])
    out = torch.zeros_like(probs)
    out.scatter_(1, si, sp * keep)
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, min_p: Optional[torch.Tensor] = None,
           generator: Optional[torch.Generator] = None, seeds: Optional[torch.Tensor] = None,
           offsets: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy rows (temperature < 1e-5) take argmax; others the exponential race.  With ``seeds`` /
    ``offsets`` every row draws from its own stream (request seed, number of tokens generated so
    far), so a request's samples do not depend on what else is in the batch."""
    greedy = temperature < 1e-5
    t = torch.where(greedy, torch.ones_like(temperature), temperature).unsqueeze(1)
    probs = torch.softmax(logits.float() / t, dim=-1)
    probs = top_k_top_p_filter(probs, top_k, top_p, min_p)
    if seeds is not None:
        e = torch.empty_like(probs)
        off = offsets if offsets is not None else torch.zeros_like(seeds)
        for i in range(probs.shape[0]):
            g = torch.Generator(device="cpu").manual_seed((int(seeds[i]) * 1000003 + int(off[i])) & ((1 << 63) - 1))
            e[i].exponential_(1.0, generator=g)
    else:
        e = torch.empty_like(probs).exponential_(1.0, generator=generator)
    sampled = (probs / e).argmax(dim=-1)
    return torch.where(greedy, logits.argmax(dim=-1), sampled)


# ---------------------------------------------------------------- quantization
def quant_fp8_group128(x: torch.Tensor, pow2_scale: bool = False):
    """Per-token groups of 128 columns (the last group may be shorter)."""
    T, H = x.shape
    G = (H + 127) // 128
    xp = torch.zeros(T, G * 128, dtype=torch.float32, device=x.device)
    xp[:, :H] = x.float()
    xg = xp.view(T, G, 128)
    amax = xg.abs().amax(dim=-1).clamp_min(1e-10)
    scale = amax / 448.0
    if pow2_scale:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = (xg / scale.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.view(T, G * 128)[:, :H].contiguous(), scale


def dequant_block_fp8_weight(w: torch.Tensor, scale: torch.Tensor, block=(128, 128)):
    N, K = w.shape
    bn, bk = block
    s = scale.repeat_interleave(bn, dim=0)[:N].repeat_interleave(bk, dim=1)[:, :K]
    return w.float() * s


def block_fp8_linear(x: torch.Tensor, w: torch.Tensor, w_scale: torch.Tensor, block=(128, 128),
                     out_dtype=torch.bfloat16) -> torch.Tensor:
    xq, xs = quant_fp8_group128(x)
    K = x.shape[1]
    xd = xq.float() * xs.repeat_interleave(128, dim=1)[:, :K]
    wd = dequant_block_fp8_weight(w, w_scale, block)
    return (xd @ wd.t()).to(out_dtype)


# ---------------------------------------------------------------- more activations / gated norm
def quant_fp8_per_token(x: torch.Tensor):
    xf = x.float()
    scale = (xf.abs().amax(dim=-1) / 448.0).clamp_min(1e-10)
    return (xf / scale.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn), scale


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias, eps: float) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(),
                        eps).to(x.dtype)


def activation(x: torch.Tensor, kind: str, gated: bool = False, alpha: float = 1.702, limit: float = 7.0):
    """kind: gelu | gelu_tanh | quick_gelu | swiglu_oai.  gated: x = [gate | up]."""
    if gated:
        d = x.shape[-1] // 2
        g, u = x[..., :d].float(), x[..., d:].float()
    else:
        g, u = x.float(), None
    if kind == "swiglu_oai":
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
        return (g * torch.sigmoid(alpha * g) * (u + 1)).to(x.dtype)
    if kind == "gelu":
        y = F.gelu(g)
    elif kind == "gelu_tanh":
        y = F.gelu(g, approximate="tanh")
    elif kind == "quick_gelu":
        y = g * torch.sigmoid(1.702 * g)
    else:
        raise ValueError(f"unknown activation {kind!r}")
    return (y * u if u is not None else y).to(x.dtype)


def rms_norm_gated(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float, group: int = 0,
                   norm_before_gate: bool = True) -> torch.Tensor:
    """rmsnorm(x) * w * silu(z) (or rmsnorm(x * silu(z)) * w), optionally per group of columns."""
    H = x.shape[-1]
    g = group or H
    xf, zf = x.float().reshape(-1, g), z.float().reshape(-1, g)
    gate = F.silu(zf)
    if not norm_before_gate:
        xf = xf * gate
    y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * w.float()[:g]
    if norm_before_gate:
        y = y * gate
    return y.reshape(x.shape).to(x.dtype)
