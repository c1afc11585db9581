"""MLA (multi-head latent attention) cache write and absorbed-weight attention.

Cache layout contract: two paged tensors per layer, latent
``[num_blocks, block_size, 1, kv_lora_rank]`` and rope
``[num_blocks, block_size, 1, qk_rope_head_dim]``
(vllm_ascend/worker/model_runner_v1.py:3994-4069).  Attention is MQA over the
576-wide (latent ‖ rope) key with the latent as value
(vllm_ascend/attention/mla_v1.py:1373-1577).
"""
from __future__ import annotations

from typing import Optional

import torch

from ctypes import c_float, c_int, c_long, c_void_p

from .. import _native
from ..ops import reference as ref

_P, _I, _L, _F = c_void_p, c_int, c_long, c_float
_native.register_signature("b200_mla_decode", [_P, _L, _L, _I, _P, _P, _L, _I, _P, _P, _P, _I, _F, _I, _P, _L, _P,
                                               _P, _P])
_native.register_signature("b200_mla_decode_lse", [_P, _L, _L, _I, _P, _P, _L, _I, _P, _P, _P, _I, _F, _I, _P, _L, _P,
                                                   _P, _P, _P])
_scratch: dict = {}


def mla_decode_native(q_cat: torch.Tensor, lat_cache: torch.Tensor, pe_cache: torch.Tensor,
                      row_seq: torch.Tensor, row_kv_len: torch.Tensor, block_table: torch.Tensor,
                      scale: float, num_splits: int = 0, max_kv_len: int = 0,
                      lse_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """tcgen05 MLA attention over query rows.  q_cat [R, H, 576] = absorbed q_nope ‖ q_pe;
    every row r attends to the first ``row_kv_len[r]`` tokens of sequence ``row_seq[r]``.
    Returns o_lat [R, H, 512].  ``lse_out`` (fp32 [R, H]) receives the log-sum-exp over the keys
    seen (-inf for a row without keys), for merging the results of context-parallel ranks."""
    R, H, dk = q_cat.shape
    assert dk == 576 and q_cat.dtype == torch.bfloat16 and q_cat.stride(2) == 1 and q_cat.stride(1) == dk
    dev = q_cat.device
    out = torch.empty((R, H, 512), dtype=torch.bfloat16, device=dev)
    if num_splits <= 0:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        nq = 32 if H % 32 == 0 else 16
        ctas = max(1, R * (H // nq))
        tiles = max(1, (max_kv_len + 127) // 128) if max_kv_len else 8
        num_splits = max(1, min(tiles, (2 * sms + ctas - 1) // ctas, 32))
    if lse_out is not None:
        num_splits = max(2, num_splits)          # the split merge produces the log-sum-exp
    scratch = None
    if num_splits > 1:
        need = R * H * num_splits * 513
        key = dev.index
        scratch = _scratch.get(key)
        if scratch is None or scratch.numel() < need:
            scratch = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=dev)
            _scratch[key] = scratch
    rc = _native.lib().b200_mla_decode_lse(
        q_cat.data_ptr(), q_cat.stride(0), R, H, lat_cache.data_ptr(), pe_cache.data_ptr(), lat_cache.shape[0],
        lat_cache.shape[1], row_seq.data_ptr(), row_kv_len.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), scale, num_splits, out.data_ptr(), out.stride(0), _native.ptr(scratch),
        _native.ptr(lse_out), _native.status_word(dev).data_ptr(), _native.stream_ptr())
    _native.check(rc, "mla_decode")
    _native.count_launch(2 if num_splits > 1 else 1)
    return out


def reserve_mla_scratch(device, rows: int, heads: int, max_splits: int = 32) -> None:
    """Allocate the split-KV scratch up front (before graph capture)."""
    need = rows * heads * max_splits * 513
    cur = _scratch.get(device.index)
    if cur is None or cur.numel() < need:
        _scratch[device.index] = torch.empty(need, dtype=torch.float32, device=device)


def write_latent_cache(latent: torch.Tensor, k_pe: torch.Tensor, lat_cache: torch.Tensor,
                       pe_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """Scatter the step's latents / rope keys into their cache slots; slot -1 = not stored.
    Written without data-dependent shapes so it can be captured into a CUDA graph: skipped
    tokens rewrite slot 0 with the value it already holds."""
    valid = (slot_mapping >= 0).unsqueeze(-1)
    idx = slot_mapping.clamp(min=0)
    lat_flat = lat_cache.view(-1, lat_cache.shape[-1])
    pe_flat = pe_cache.view(-1, pe_cache.shape[-1])
    lat_flat.index_copy_(0, idx, torch.where(valid, latent.to(lat_cache.dtype), lat_flat[idx]))
    pe_flat.index_copy_(0, idx, torch.where(valid, k_pe.to(pe_cache.dtype), pe_flat[idx]))


def mla_paged_attention(q_lat: torch.Tensor, q_pe: torch.Tensor, lat_cache: torch.Tensor,
                        pe_cache: torch.Tensor, meta, scale: float) -> torch.Tensor:
    """q_lat [T,H,dc], q_pe [T,H,dr] -> o_lat [T,H,dc] (softmax over latent‖rope keys)."""
    T, H, dc = q_lat.shape
    from .. import envs
    if envs.VLLM_B200_MLA_ATTN == "tcgen05" and q_lat.is_cuda and q_lat.dtype == torch.bfloat16 and dc == 512 and q_pe.shape[-1] == 64 and H % 16 == 0 \
            and lat_cache.shape[1] in (16, 32, 64, 128, 256, 512) and T <= 65535:
        q_cat = torch.cat([q_lat, q_pe], dim=-1)
        B = meta.num_reqs
        if meta.max_query_len == 1 and T == B:
            row_seq = torch.arange(T, dtype=torch.int32, device=q_lat.device)
        else:
            q_lens = (meta.query_start_loc[1:B + 1] - meta.query_start_loc[:B]).long()
            row_seq = torch.repeat_interleave(torch.arange(B, device=q_lat.device), q_lens,
                                              output_size=T).to(torch.int32)
        row_kv = (meta.positions[:T] + 1).to(torch.int32)
        # a captured graph must carry a split count that suits any later sequence length
        max_kv = meta.block_table.shape[1] * lat_cache.shape[1] if torch.cuda.is_current_stream_capturing() \
            else meta.max_seq_len
        return mla_decode_native(q_cat, lat_cache, pe_cache, row_seq, row_kv, meta.block_table, scale,
                                 max_kv_len=max_kv)
    out = torch.empty(T, H, dc, dtype=q_lat.dtype, device=q_lat.device)
    qsl, sls = meta.query_start_loc_cpu, meta.seq_lens_cpu
    for b in range(meta.num_reqs):
        qs, qe = int(qsl[b]), int(qsl[b + 1])
        ql = qe - qs
        if ql <= 0:
            continue
        sl = int(sls[b])
        ctx = sl - ql
        lat = ref.gather_kv(lat_cache, meta.block_table[b], sl)[:, 0].float()   # [sl, dc]
        pe = ref.gather_kv(pe_cache, meta.block_table[b], sl)[:, 0].float()     # [sl, dr]
        s = (torch.einsum("qhc,kc->hqk", q_lat[qs:qe].float(), lat) +
             torch.einsum("qhr,kr->hqk", q_pe[qs:qe].float(), pe)) * scale
        kpos = torch.arange(sl, device=s.device)
        qpos = ctx + torch.arange(ql, device=s.device)
        s = s.masked_fill(~(kpos[None, :] <= qpos[:, None])[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[qs:qe] = torch.einsum("hqk,kc->qhc", p, lat).to(out.dtype)
    return out


class B200MLABackend:
    """Descriptor of the MLA backend (vllm_ascend/attention/mla_v1.py: cache of a 512-wide
    normalised latent plus a 64-wide RoPE key per token, MQA with absorbed up-projections)."""

    @staticmethod
    def get_name() -> str:
        return "B200_MLA"

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int) -> tuple:
        return (num_blocks, block_size, 1, head_size)

    @staticmethod
    def get_supported_block_size() -> list[int]:
        return [128]

    @staticmethod
    def get_impl_cls():
        from ..models.transformer import MLAAttention
        return MLAAttention
