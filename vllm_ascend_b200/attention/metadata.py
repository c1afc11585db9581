"""Per-step attention metadata.

Field set follows the contract of ``AscendCommonAttentionMetadata``
(vllm_ascend/attention/utils.py:214-320): query_start_loc / seq_lens on host and
device, block table, slot mapping, positions, attention state and the
decodes-first split.  Device tensors are views of persistent buffers so captured
CUDA graphs replay without host-side patching.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch


class AttentionState(enum.IntEnum):
    """States of vllm_ascend/attention/attention_v1.py:152-157."""
    PrefillNoCache = 0
    PrefillCacheHit = 1
    DecodeOnly = 2
    ChunkedPrefill = 3
    SpecDecoding = 4


@dataclass
class AttentionMetadata:
    num_reqs: int
    num_actual_tokens: int
    max_query_len: int
    max_seq_len: int
    query_start_loc: torch.Tensor          # int32 [B+1] device
    seq_lens: torch.Tensor                 # int32 [B] device
    block_table: torch.Tensor              # int32 [B, max_blocks] device
    slot_mapping: torch.Tensor             # int64 [T] device
    positions: torch.Tensor                # int64 [T] device
    query_start_loc_cpu: np.ndarray
    seq_lens_cpu: np.ndarray
    attn_state: AttentionState = AttentionState.ChunkedPrefill
    num_decodes: int = 0
    num_decode_tokens: int = 0
    num_prefills: int = 0
    # work list of the tensor-core attention kernel (one entry per 128-row tile)
    tile_seq: Optional[torch.Tensor] = None
    tile_qoff: Optional[torch.Tensor] = None
    num_tiles: int = 0
    num_splits: int = 1
    num_input_tokens: int = 0              # padded token count (graph replay)
    # linear-attention layers: per-sequence state row and whether it holds earlier tokens
    state_slots: Optional[torch.Tensor] = None          # int32 [B] device
    has_initial_state: Optional[torch.Tensor] = None    # int32 [B] device
    # multimodal rotary embedding: int64 [3, num_input_tokens] (temporal, height, width)
    mrope_positions: Optional[torch.Tensor] = None
    pcp: object = None                      # attention.pcp.PCPMeta on split prefill steps
    deepstack: object = None                # (rows [n], features [L, n, H]) added after the first L layers
    # decode-context-parallel / extras
    dcp_world_size: int = 1
    dcp_rank: int = 0
    extra: Optional[dict] = None


def split_decodes_and_prefills(query_lens: np.ndarray, decode_threshold: int = 1) -> tuple[int, int, int, int]:
    """Batches are ordered decodes-first; split at the first request whose query
    is longer than the threshold (vllm_ascend/attention/utils.py:346-435).
    Returns (num_decodes, num_prefills, num_decode_tokens, num_prefill_tokens)."""
    n = len(query_lens)
    if n == 0:
        return 0, 0, 0, 0
    is_prefill = query_lens > decode_threshold
    if not is_prefill.any():
        return n, 0, int(query_lens.sum()), 0
    first = int(np.argmax(is_prefill))
    nd_tokens = int(query_lens[:first].sum())
    return first, n - first, nd_tokens, int(query_lens.sum()) - nd_tokens


def build_tile_worklist(query_lens: np.ndarray, tok_per_tile: int,
                        seq_lens: Optional[np.ndarray] = None) -> tuple[np.ndarray, np.ndarray]:
    """(tile_seq, tile_qoff) for the tensor-core kernel.  Tiles of long-context
    sequences are placed first so the heaviest CTAs start early."""
    n_tiles = (query_lens + tok_per_tile - 1) // tok_per_tile
    total = int(n_tiles.sum())
    tile_seq = np.repeat(np.arange(len(query_lens), dtype=np.int32), n_tiles)
    starts = np.cumsum(n_tiles) - n_tiles
    tile_idx = np.arange(total, dtype=np.int32) - np.repeat(starts, n_tiles).astype(np.int32)
    tile_qoff = (tile_idx * tok_per_tile).astype(np.int32)
    if seq_lens is not None and total > 1:
        ctx = (seq_lens - query_lens)[tile_seq]
        work = ctx + tile_qoff                      # keys visible to the tile's first row
        order = np.argsort(-work, kind="stable")
        tile_seq, tile_qoff = tile_seq[order], tile_qoff[order]
    return np.ascontiguousarray(tile_seq), np.ascontiguousarray(tile_qoff)


def metadata_from_tensors(query_start_loc: torch.Tensor, seq_lens: torch.Tensor, block_table: torch.Tensor,
                          max_query_len: int, max_seq_len: int, num_q_heads: int, num_kv_heads: int,
                          head_dim: int, decode_kernel: bool = True) -> AttentionMetadata:
    """Metadata for one attention call from device tensors alone (callers that reach the attention op
    through its dispatcher schema have no runner to prepare the host-side views): copies the two
    length vectors to the host once, orders nothing (the batch must already be decodes-first) and
    builds the tile work list of the tensor-core kernel."""
    qsl = query_start_loc.detach().cpu().numpy().astype(np.int32)
    sl = seq_lens.detach().cpu().numpy().astype(np.int32)
    q_lens = qsl[1:] - qsl[:-1]
    B = int(sl.shape[0])
    nd, npf, ndt, _ = split_decodes_and_prefills(q_lens)
    T = int(qsl[-1])
    meta = AttentionMetadata(
        num_reqs=B, num_actual_tokens=T, max_query_len=int(max_query_len), max_seq_len=int(max_seq_len),
        query_start_loc=query_start_loc, seq_lens=seq_lens, block_table=block_table, slot_mapping=None,
        positions=None, query_start_loc_cpu=qsl, seq_lens_cpu=sl, num_decodes=nd, num_decode_tokens=ndt,
        num_prefills=npf, num_input_tokens=T)
    if query_start_loc.is_cuda and max_query_len > 1:
        G = max(1, num_q_heads // num_kv_heads)
        skip = nd if (decode_kernel and head_dim == 128 and 16 % G == 0) else 0
        ts, tq = build_tile_worklist(q_lens[skip:], max(1, 128 // G), sl[skip:])
        if skip == 0:
            meta.num_decodes = meta.num_decode_tokens = 0
        dev = query_start_loc.device
        meta.tile_seq = torch.from_numpy(ts + np.int32(skip)).to(dev)
        meta.tile_qoff = torch.from_numpy(tq).to(dev)
        meta.num_tiles = len(ts)
    return meta
