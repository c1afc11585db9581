"""MLA (multi-head latent attention) cache write and absorbed-weight attention.

Cache layout contract: two paged tensors per layer, latent
``[num_blocks, block_size, 1, kv_lora_rank]`` and rope
``[num_blocks, block_size, 1, qk_rope_head_dim]``
(vllm_ascend/worker/model_runner_v1.py:3994-4069).  Attention is MQA over the
576-wide (latent ‖ rope) key with the latent as value
(vllm_ascend/attention/mla_v1.py:1373-1577).
"""
from __future__ import annotations

import torch

from ..ops import reference as ref


def write_latent_cache(latent: torch.Tensor, k_pe: torch.Tensor, lat_cache: torch.Tensor,
                       pe_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    valid = slot_mapping >= 0
    slots = slot_mapping[valid]
    lat_cache.view(-1, lat_cache.shape[-1])[slots] = latent[valid].to(lat_cache.dtype)
    pe_cache.view(-1, pe_cache.shape[-1])[slots] = k_pe[valid].to(pe_cache.dtype)


def mla_paged_attention(q_lat: torch.Tensor, q_pe: torch.Tensor, lat_cache: torch.Tensor,
                        pe_cache: torch.Tensor, meta, scale: float) -> torch.Tensor:
    """q_lat [T,H,dc], q_pe [T,H,dr] -> o_lat [T,H,dc] (softmax over latent‖rope keys)."""
    T, H, dc = q_lat.shape
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
