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

from ctypes import c_int, c_long, c_void_p

from .. import _native
from ..ops import reference as ref

_P, _I, _L = c_void_p, c_int, c_long
_native.register_signature("b200_lightning_indexer", [_P, _L, _L, _I, _P, _P, _L, _I, _P, _P, _P, _I, _I, _P, _L,
                                                      _P, _P])
_native.register_signature("b200_gather_paged_rows", [_P, _P, _P, _P, _I, _I, _L, _I, _I, _L, _P, _P, _P])


def _rows(meta, T: int, device):
    """(row_seq, row_kv_len) of every query token: its sequence and how many keys it may see."""
    B = meta.num_reqs
    if meta.max_query_len == 1 and T == B:
        row_seq = torch.arange(T, dtype=torch.int32, device=device)
    else:
        q_lens = (meta.query_start_loc[1:B + 1] - meta.query_start_loc[:B]).long()
        row_seq = torch.repeat_interleave(torch.arange(B, device=device), q_lens, output_size=T).to(torch.int32)
    return row_seq, (meta.positions[:T] + 1).to(torch.int32)


def lightning_indexer_native(q_idx: torch.Tensor, w: torch.Tensor, k_idx_cache: torch.Tensor, meta,
                             topk: int) -> torch.Tensor:
    """tcgen05 indexer scores + top-k.  Same contract as ``lightning_indexer``."""
    T, G, d = q_idx.shape
    dev = q_idx.device
    row_seq, row_kv = _rows(meta, T, dev)
    S = (meta.max_seq_len + 127) // 128 * 128
    scores = torch.full((T, max(S, topk)), float("-inf"), dtype=torch.float32, device=dev)
    q = q_idx.contiguous()
    rc = _native.lib().b200_lightning_indexer(
        q.data_ptr(), q.stride(0), T, G, w.float().contiguous().data_ptr(), k_idx_cache.data_ptr(),
        k_idx_cache.shape[0], k_idx_cache.shape[1], row_seq.data_ptr(), row_kv.data_ptr(),
        meta.block_table.data_ptr(), meta.block_table.stride(0), meta.max_seq_len, scores.data_ptr(),
        scores.stride(0), _native.status_word(dev).data_ptr(), _native.stream_ptr())
    _native.check(rc, "lightning_indexer")
    _native.count_launch()
    vals, idx = scores.topk(topk, dim=-1)
    return idx.to(torch.int32).masked_fill(vals == float("-inf"), -1)


def sparse_mla_attention_native(q_lat: torch.Tensor, q_pe: torch.Tensor, lat_cache: torch.Tensor,
                                pe_cache: torch.Tensor, meta, indices: torch.Tensor, scale: float) -> torch.Tensor:
    """Sparse MLA attention on the GPU: the selected latent / rope rows of every query token are
    gathered into a dense per-token mini cache, then the MLA tensor-core kernel attends over it.
    ``indices`` must list the valid entries first (as top-k does)."""
    from .mla import mla_decode_native
    T, H, dc = q_lat.shape
    dev = q_lat.device
    topk = indices.shape[1]
    tk = (topk + 127) // 128 * 128
    row_seq, _ = _rows(meta, T, dev)
    idx = indices if tk == topk else torch.nn.functional.pad(indices, (0, tk - topk), value=-1)
    idx = idx.contiguous()
    lib = _native.lib()
    st = _native.status_word(dev).data_ptr()
    lat_g = torch.empty((T * tk // 128, 128, dc), dtype=lat_cache.dtype, device=dev)
    pe_g = torch.empty((T * tk // 128, 128, pe_cache.shape[-1]), dtype=pe_cache.dtype, device=dev)
    for cache, out in ((lat_cache, lat_g), (pe_cache, pe_g)):
        rc = lib.b200_gather_paged_rows(cache.data_ptr(), idx.data_ptr(), row_seq.data_ptr(),
                                        meta.block_table.data_ptr(), meta.block_table.stride(0), cache.shape[1], T, tk,
                                        cache.shape[-1] * cache.element_size(), cache.shape[0], out.data_ptr(), st,
                                        _native.stream_ptr())
        _native.check(rc, "gather_paged_rows")
    _native.count_launch(2)
    nb = tk // 128
    bt = torch.arange(T * nb, dtype=torch.int32, device=dev).view(T, nb)
    kv_len = (indices >= 0).sum(dim=1).to(torch.int32)
    rows = torch.arange(T, dtype=torch.int32, device=dev)
    q_cat = torch.cat([q_lat, q_pe], dim=-1)
    out = mla_decode_native(q_cat, lat_g, pe_g, rows, kv_len, bt, scale, max_kv_len=tk)
    return torch.where((kv_len > 0)[:, None, None], out, torch.zeros_like(out))


def lightning_indexer(q_idx: torch.Tensor, w: torch.Tensor, k_idx_cache: torch.Tensor, meta,
                      topk: int) -> torch.Tensor:
    """q_idx [T, G, d], w [T, G], k_idx_cache [blocks, bs, 1, d] -> indices [T, topk] (int32,
    -1 padded) into each token's own sequence positions, causal."""
    T = q_idx.shape[0]
    if q_idx.is_cuda and q_idx.dtype == torch.bfloat16 and q_idx.shape[-1] == 128 and q_idx.shape[1] <= 64 \
            and k_idx_cache.shape[-1] == 128 and T <= 65535:
        return lightning_indexer_native(q_idx, w, k_idx_cache, meta, topk)
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
    if q_lat.is_cuda and q_lat.dtype == torch.bfloat16 and dc == 512 and q_pe.shape[-1] == 64 and H % 16 == 0 \
            and T * ((indices.shape[1] + 127) // 128) <= 1 << 22 and T <= 65535:
        return sparse_mla_attention_native(q_lat, q_pe, lat_cache, pe_cache, meta, indices, scale)
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
