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
    out = torch.zeros(T, HH, dc, dtype=torch.float32, device=q.device)
    lse = torch.full((T, HH), float("-inf"), dtype=torch.float32, device=q.device)
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
        st = torch.from_numpy(slots).to(q.device)
        kl, kp = lat_flat[st].float(), pe_flat[st].float()
        s = (torch.einsum("qhc,kc->qhk", q_all[qs:qe, :, :dc].float(), kl) +
             torch.einsum("qhr,kr->qhk", q_all[qs:qe, :, dc:].float(), kp)) * scale
        qpos = (sl - ql) + torch.arange(ql, device=q.device)
        vis = torch.from_numpy(gpos).to(q.device)[None, :] <= qpos[:, None]           # [ql, n]
        s = s.masked_fill(~vis[:, None, :], float("-inf"))
        l = torch.logsumexp(s, dim=-1)                                                 # [ql, HH]
        p = torch.exp(s - l.clamp(min=-1e30).unsqueeze(-1))
        p = torch.where(torch.isfinite(s), p, torch.zeros_like(p))
        out[qs:qe] = torch.einsum("qhk,kc->qhc", p, kl)
        lse[qs:qe] = l
    # partial results of head block j go to rank j: all-to-all of (out ‖ lse)
    packed = torch.cat([out, lse.unsqueeze(-1)], dim=-1).view(T, d, H, dc + 1).permute(1, 0, 2, 3).contiguous()
    recv = group.all_to_all_single(packed.view(d * T, H, dc + 1))                      # [d(src) * T, H, dc+1]
    recv = recv.view(d, T, H, dc + 1)
    return merge_partials(recv[..., :dc], recv[..., dc]).to(q_lat.dtype)
