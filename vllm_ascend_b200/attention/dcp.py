"""Decode context parallelism (DCP): the KV cache of a sequence is sharded along the sequence
over the ranks of the DCP group (a sub-group of the TP group whose ranks would otherwise
hold identical KV, e.g. the MLA latent cache), interleaved in runs of ``interleave`` tokens.

  * layout: the scheduler works with virtual blocks of ``block_size * dcp`` tokens; of each
    virtual block a rank stores ``block_size`` tokens (vllm_ascend/worker/block_table.py:231-276)
  * attention: Q heads are all-gathered over the group, every rank attends over its local
    tokens and returns (out, lse), an all-to-all brings each head's partial results to the
    rank that owns the head, and the partials are merged by log-sum-exp
    (vllm_ascend/attention/context_parallel/attention_cp.py:278-393, common_cp.py:139-195)
"""
from __future__ import annotations

import numpy as np
import torch


def owner_and_offset(within: np.ndarray, block_size: int, dcp: int, interleave: int):
    """For token offsets inside a virtual block: (owning rank, offset inside the rank's block)."""
    owner = (within // interleave) % dcp
    local = (within // (interleave * dcp)) * interleave + within % interleave
    return owner, local


def local_slot_mapping(pos: np.ndarray, blocks: np.ndarray, block_size: int, dcp: int, rank: int,
                       interleave: int) -> np.ndarray:
    """Cache slot of each token on this rank, -1 for tokens another rank stores.  ``blocks``
    holds the (virtual = physical) block id of every token."""
    owner, local = owner_and_offset(pos % (block_size * dcp), block_size, dcp, interleave)
    return np.where(owner == rank, blocks.astype(np.int64) * block_size + local, -1)


def local_tokens(seq_len: int, block_table_row: torch.Tensor, block_size: int, dcp: int, rank: int,
                 interleave: int):
    """(cache slots [n], global positions [n]) of the tokens of one sequence held by ``rank``."""
    pos = np.arange(seq_len, dtype=np.int64)
    vb = block_size * dcp
    owner, local = owner_and_offset(pos % vb, block_size, dcp, interleave)
    mine = owner == rank
    gp = pos[mine]
    blocks = block_table_row.cpu().numpy().astype(np.int64)[gp // vb]
    return blocks * block_size + local[mine], gp


def merge_partials(outs: torch.Tensor, lses: torch.Tensor) -> torch.Tensor:
    """outs [R, T, H, D] (each normalised by its own denominator), lses [R, T, H] -> [T, H, D]."""
    m = lses.max(dim=0).values
    w = torch.exp(lses - m.clamp(min=-1e30))
    w = torch.where(torch.isfinite(lses), w, torch.zeros_like(w))
    den = w.sum(0).clamp(min=1e-30)
    return (outs * w.unsqueeze(-1)).sum(0) / den.unsqueeze(-1)


def _mla_local_partials(q_all, lat_cache, pe_cache, meta, scale, d, rank, interleave, dc):
    """PyTorch definition of one rank's partial MLA attention: (out fp32 [T, HH, dc] normalised over the
    local keys, lse fp32 [T, HH]).  Serves prefill / mixed steps and the host tests."""
    T, HH, _ = q_all.shape
    bs = lat_cache.shape[1]
    out = torch.zeros(T, HH, dc, dtype=torch.float32, device=q_all.device)
    lse = torch.full((T, HH), float("-inf"), dtype=torch.float32, device=q_all.device)
    lat_flat = lat_cache.reshape(-1, lat_cache.shape[-1])
    pe_flat = pe_cache.reshape(-1, pe_cache.shape[-1])
    qsl, sls = meta.query_start_loc_cpu, meta.seq_lens_cpu
    for b in range(meta.num_reqs):
        qs, qe = int(qsl[b]), int(qsl[b + 1])
        ql, sl = qe - qs, int(sls[b])
        if ql <= 0:
            continue
        slots, gpos = local_tokens(sl, meta.block_table[b], bs, d, rank, interleave)
        if len(slots) == 0:
            continue
        st = torch.from_numpy(slots).to(q_all.device)
        kl, kp = lat_flat[st].float(), pe_flat[st].float()
        s = (torch.einsum("qhc,kc->qhk", q_all[qs:qe, :, :dc].float(), kl) +
             torch.einsum("qhr,kr->qhk", q_all[qs:qe, :, dc:].float(), kp)) * scale
        qpos = (sl - ql) + torch.arange(ql, device=q_all.device)
        vis = torch.from_numpy(gpos).to(q_all.device)[None, :] <= qpos[:, None]           # [ql, n]
        s = s.masked_fill(~vis[:, None, :], float("-inf"))
        l = torch.logsumexp(s, dim=-1)                                                 # [ql, HH]
        p = torch.exp(s - l.clamp(min=-1e30).unsqueeze(-1))
        p = torch.where(torch.isfinite(s), p, torch.zeros_like(p))
        out[qs:qe] = torch.einsum("qhk,kc->qhc", p, kl)
        lse[qs:qe] = l
    return out, lse


def mla_attention_dcp(q_lat: torch.Tensor, q_pe: torch.Tensor, lat_cache: torch.Tensor, pe_cache: torch.Tensor,
                      meta, scale: float, group, interleave: int) -> torch.Tensor:
    """MLA attention with the latent cache sharded over ``group``.  q_* hold this rank's heads."""
    d, rank = group.world_size, group.rank_in_group
    T, H, dc = q_lat.shape
    bs = lat_cache.shape[1]
    # every rank needs every head of the group to attend over its slice of the sequence
    q = torch.cat([q_lat, q_pe], dim=-1)
    q_all = group.all_gather(q.contiguous(), dim=1)                        # [T, d*H, dc+dr]
    HH = q_all.shape[1]
    local_sl = getattr(meta, "dcp_seq_lens", None)
    from .. import envs
    kernel_ok = (q.is_cuda and q.dtype == torch.bfloat16 and dc == 512 and q_pe.shape[-1] == 64 and HH % 16 == 0
                 and meta.max_query_len == 1 and T == meta.num_reqs and local_sl is not None
                 and envs.VLLM_B200_MLA_ATTN == "tcgen05" and bs in (16, 32, 64, 128, 256, 512) and T <= 65535)
    if kernel_ok:
        # decode step: a rank's tokens of a sequence are an ordinary paged sequence of local_seq_lens keys,
        # all visible to the new token: the tcgen05 MLA kernel runs on it and its split merge returns
        # the log-sum-exp
        from .mla import mla_decode_native
        row_seq = torch.arange(T, dtype=torch.int32, device=q.device)
        lse = torch.empty((T, HH), dtype=torch.float32, device=q.device)
        out = mla_decode_native(q_all, lat_cache, pe_cache, row_seq, local_sl, meta.block_table, scale,
                                max_kv_len=max(1, (meta.max_seq_len + d - 1) // d), lse_out=lse).float()
    else:
        out, lse = _mla_local_partials(q_all, lat_cache, pe_cache, meta, scale, d, rank, interleave, dc)
    # partial results of head block j go to rank j: all-to-all of (out ‖ lse)
    packed = torch.cat([out, lse.unsqueeze(-1)], dim=-1).view(T, d, H, dc + 1).permute(1, 0, 2, 3).contiguous()
    recv = group.all_to_all_single(packed.view(d * T, H, dc + 1))                      # [d(src) * T, H, dc+1]
    recv = recv.view(d, T, H, dc + 1)
    return merge_partials(recv[..., :dc], recv[..., dc]).to(q_lat.dtype)


def local_seq_lens(seq_lens: np.ndarray, block_size: int, dcp: int, rank: int, interleave: int) -> np.ndarray:
    """Number of tokens of each sequence that ``rank`` stores.  A rank's tokens of one sequence
    fill its blocks densely and in global order, so the local cache of a sequence is an ordinary
    paged sequence of this length under the same block table."""
    sl = np.asarray(seq_lens, dtype=np.int64)
    vb = block_size * dcp
    rem = sl % vb
    cyc = interleave * dcp
    cnt = (rem // cyc) * interleave + np.clip(rem % cyc - rank * interleave, 0, interleave)
    return ((sl // vb) * block_size + cnt).astype(np.int32)


def _gqa_local_partials(q_all: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, meta, scale: float,
                        d: int, rank: int, interleave: int):
    """PyTorch definition of one rank's partial attention: (out fp32 [T, HH, D] normalised over the local
    keys, lse fp32 [T, HH]).  Serves prefill / mixed steps and the host tests."""
    T, HH, D = q_all.shape
    bs, Hkv = k_cache.shape[1], k_cache.shape[2]
    G = HH // Hkv
    out = torch.zeros(T, HH, D, dtype=torch.float32, device=q_all.device)
    lse = torch.full((T, HH), float("-inf"), dtype=torch.float32, device=q_all.device)
    k_flat = k_cache.reshape(-1, Hkv, D)
    v_flat = v_cache.reshape(-1, Hkv, D)
    qsl, sls = meta.query_start_loc_cpu, meta.seq_lens_cpu
    for b in range(meta.num_reqs):
        qs, qe = int(qsl[b]), int(qsl[b + 1])
        ql, sl = qe - qs, int(sls[b])
        if ql <= 0:
            continue
        slots, gpos = local_tokens(sl, meta.block_table[b], bs, d, rank, interleave)
        if len(slots) == 0:
            continue
        st = torch.from_numpy(slots).to(q_all.device)
        k = k_flat[st].float().repeat_interleave(G, dim=1)          # [n, HH, D]
        v = v_flat[st].float().repeat_interleave(G, dim=1)
        s = torch.einsum("qhd,khd->qhk", q_all[qs:qe].float(), k) * scale
        qpos = (sl - ql) + torch.arange(ql, device=q_all.device)
        vis = torch.from_numpy(gpos).to(q_all.device)[None, :] <= qpos[:, None]
        s = s.masked_fill(~vis[:, None, :], float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l.clamp(min=-1e30).unsqueeze(-1))
        p = torch.where(torch.isfinite(s), p, torch.zeros_like(p))
        out[qs:qe] = torch.einsum("qhk,khd->qhd", p, v)
        lse[qs:qe] = l
    return out, lse


def gqa_attention_dcp(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, meta, scale: float,
                      group, interleave: int) -> torch.Tensor:
    """Grouped-query attention with the KV cache sharded along the sequence over ``group`` (ranks that
    hold the same KV heads).  q [T, H, D] holds this rank's query heads; returns [T, H, D].

    Every rank gathers the group's query heads, attends over the keys it stores and keeps the
    log-sum-exp; an all-to-all returns each head's partial results to the rank that owns the head,
    which merges them (vllm_ascend/attention/context_parallel/attention_cp.py:173-393).  Decode steps
    run the tcgen05 flash-decode kernel on the local cache (the rank's tokens of a sequence form an
    ordinary paged sequence of ``local_seq_lens`` keys, all of them visible to the new token) and the
    merge kernel; steps with longer queries take the PyTorch definition."""
    from .. import ops
    d, rank = group.world_size, group.rank_in_group
    T, H, D = q.shape
    q_all = group.all_gather(q.contiguous(), dim=1)                  # [T, d*H, D]
    HH = q_all.shape[1]
    Hkv = k_cache.shape[2]
    G = HH // Hkv
    local_sl = getattr(meta, "dcp_seq_lens", None)
    kernel_ok = (q.is_cuda and q.dtype == torch.bfloat16 and D == 128 and v_cache.shape[-1] == D
                 and meta.max_query_len == 1 and G <= 16 and 16 % G == 0 and local_sl is not None)
    if kernel_ok:
        out = torch.empty((T, HH, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((T, HH), dtype=torch.float32, device=q.device)
        ops.paged_attention_decode_tc(q_all, k_cache, v_cache, meta, scale, out, 0, num_splits=1, max_q_len=1,
                                      lse_out=lse, seq_lens=local_sl)
        out = out.float()
    else:
        out, lse = _gqa_local_partials(q_all, k_cache, v_cache, meta, scale, d, rank, interleave)
    # head block j of every rank's partials goes to rank j
    packed = torch.cat([out, lse.unsqueeze(-1)], dim=-1).view(T, d, H, D + 1).permute(1, 0, 2, 3).contiguous()
    recv = group.all_to_all_single(packed.view(d * T, H, D + 1)).view(d, T, H, D + 1)
    po = recv[..., :D].permute(1, 2, 0, 3).contiguous()              # [T, H, d, D]
    pl = recv[..., D].permute(1, 2, 0).contiguous()                  # [T, H, d]
    return ops.merge_attn_partials(po, pl, out_dtype=q.dtype).to(q.dtype)
