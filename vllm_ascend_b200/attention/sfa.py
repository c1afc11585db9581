"""Sparse attention for MLA models with a "lightning indexer" (DeepSeek-V3.2 style).

Per query token the indexer scores every cached key with a small multi-head dot product,
``score(t, s) = sum_g w[t, g] * relu(q_idx[t, g] . k_idx[s])``, keeps the top-k keys, and MLA
attention then runs over the selected keys only (vllm_ascend/attention/sfa_v1.py; indexer
math csrc/attention/lightning_indexer/README.md).  This module is the numerical definition
used on every device; the dense MLA path stays the default until top-k is smaller than the
context.
"""
from __future__ import annotations

import torch

from ..ops import reference as ref


def lightning_indexer(q_idx: torch.Tensor, w: torch.Tensor, k_idx_cache: torch.Tensor, meta,
                      topk: int) -> torch.Tensor:
    """q_idx [T, G, d], w [T, G], k_idx_cache [blocks, bs, 1, d] -> indices [T, topk] (int32,
    -1 padded) into each token's own sequence positions, causal."""
    T = q_idx.shape[0]
    out = torch.full((T, topk), -1, dtype=torch.int32, device=q_idx.device)
    qsl, sls = meta.query_start_loc_cpu, meta.seq_lens_cpu
    for b in range(meta.num_reqs):
        qs, qe = int(qsl[b]), int(qsl[b + 1])
        ql, sl = qe - qs, int(sls[b])
        if ql <= 0:
            continue
        k = ref.gather_kv(k_idx_cache, meta.block_table[b], sl)[:, 0].float()          # [sl, d]
        s = torch.einsum("tgd,sd->tgs", q_idx[qs:qe].float(), k).relu()
        s = (s * w[qs:qe].float().unsqueeze(-1)).sum(1)                                   # [ql, sl]
        qpos = (sl - ql) + torch.arange(ql, device=s.device)
        s = s.masked_fill(torch.arange(sl, device=s.device)[None, :] > qpos[:, None], float("-inf"))
        kk = min(topk, sl)
        vals, idx = s.topk(kk, dim=-1)
        idx = idx.to(torch.int32).masked_fill(vals == float("-inf"), -1)
        out[qs:qe, :kk] = idx
    return out


def sparse_mla_attention(q_lat: torch.Tensor, q_pe: torch.Tensor, lat_cache: torch.Tensor,
                         pe_cache: torch.Tensor, meta, indices: torch.Tensor, scale: float) -> torch.Tensor:
    """MLA attention over the selected keys: q_lat [T,H,dc], q_pe [T,H,dr], indices [T, topk]."""
    T, H, dc = q_lat.shape
    out = torch.zeros(T, H, dc, dtype=q_lat.dtype, device=q_lat.device)
    qsl, sls = meta.query_start_loc_cpu, meta.seq_lens_cpu
    for b in range(meta.num_reqs):
        qs, qe = int(qsl[b]), int(qsl[b + 1])
        if qe <= qs:
            continue
        sl = int(sls[b])
        lat = ref.gather_kv(lat_cache, meta.block_table[b], sl)[:, 0].float()
        pe = ref.gather_kv(pe_cache, meta.block_table[b], sl)[:, 0].float()
        idx = indices[qs:qe].long()
        valid = idx >= 0
        idx = idx.clamp(min=0)
        kl, kp = lat[idx], pe[idx]                                                       # [ql, topk, *]
        s = (torch.einsum("qhc,qkc->qhk", q_lat[qs:qe].float(), kl) +
             torch.einsum("qhr,qkr->qhk", q_pe[qs:qe].float(), kp)) * scale
        s = s.masked_fill(~valid[:, None, :], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[qs:qe] = torch.einsum("qhk,qkc->qhc", p, kl).to(out.dtype)
    return out


class B200SFABackend:
    @staticmethod
    def get_name() -> str:
        return "B200_SFA"

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int) -> tuple:
        return (num_blocks, block_size, 1, head_size)

    @staticmethod
    def get_supported_block_size() -> list[int]:
        return [128]

    indexer = staticmethod(lightning_indexer)
    attention = staticmethod(sparse_mla_attention)
