"""Attention backend descriptors: what a host framework asks a backend about (name, KV-cache
shape, block-size support, implementation and metadata-builder classes, block copy).

GQA/MHA backend contract of vllm_ascend/attention/attention_v1.py:82-157: KV cache
``(2, num_blocks, block_size, kv_heads, head_dim)`` logical shape, kernel block size 128,
states PrefillNoCache / PrefillCacheHit / DecodeOnly / ChunkedPrefill / SpecDecoding,
``swap_blocks`` / ``copy_blocks`` (attention_v1.py:119-145).
"""
from __future__ import annotations

import torch

from .. import _native, ops
from .metadata import AttentionMetadata, AttentionState  # noqa: F401  (re-exported)


class B200AttentionImpl:
    """Paged GQA attention: writes the step's K/V into the cache (done by the fused
    q/k-norm + RoPE + KV-write kernel upstream of this call) and attends over it."""

    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int,
                 sliding_window=None, **_):
        self.num_heads, self.head_size, self.scale = num_heads, head_size, scale
        self.num_kv_heads, self.sliding_window = num_kv_heads, sliding_window

    def forward(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                meta: AttentionMetadata, out: torch.Tensor = None) -> torch.Tensor:
        """q [T, Hq, D] -> [T, Hq, D]; ``out`` (optional) receives the result."""
        return ops.paged_attention(q, k_cache, v_cache, meta, self.scale, out=out, causal=True,
                                   window=self.sliding_window or 0)


class B200MetadataBuilder:
    """Builds ``AttentionMetadata`` from per-request query lengths and context lengths."""

    def __init__(self, block_size: int, device):
        self.block_size, self.device = block_size, torch.device(device)

    def build(self, query_lens, seq_lens, block_table: torch.Tensor, slot_mapping: torch.Tensor,
              positions: torch.Tensor) -> AttentionMetadata:
        import numpy as np
        q = np.asarray(query_lens, dtype=np.int32)
        s = np.asarray(seq_lens, dtype=np.int32)
        cu = np.zeros(len(q) + 1, dtype=np.int32)
        np.cumsum(q, out=cu[1:])
        if (q == 1).all():
            state = AttentionState.DecodeOnly
        elif (s == q).all():
            state = AttentionState.PrefillNoCache
        else:
            state = AttentionState.ChunkedPrefill
        return AttentionMetadata(
            num_reqs=len(q), num_actual_tokens=int(q.sum()), max_query_len=int(q.max()), max_seq_len=int(s.max()),
            query_start_loc=torch.from_numpy(cu).to(self.device), seq_lens=torch.from_numpy(s).to(self.device),
            block_table=block_table, slot_mapping=slot_mapping, positions=positions,
            query_start_loc_cpu=cu, seq_lens_cpu=s, attn_state=state)


class B200AttentionBackend:
    accept_output_buffer = True

    @staticmethod
    def get_name() -> str:
        return "B200_TCGEN05"

    @staticmethod
    def get_impl_cls():
        return B200AttentionImpl

    @staticmethod
    def get_builder_cls():
        return B200MetadataBuilder

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int) -> tuple:
        return (2, num_blocks, block_size, num_kv_heads, head_size)

    @staticmethod
    def get_supported_block_size() -> list[int]:
        return [128]

    @staticmethod
    def get_supported_head_sizes() -> list[int]:
        return [64, 128]

    @staticmethod
    def copy_blocks(kv_caches: list, src_to_dst: torch.Tensor) -> None:
        """src_to_dst [n, 2] int64 pairs; every cache tensor of every layer is updated."""
        pairs = src_to_dst.to(torch.int64).contiguous()
        for cache in kv_caches:
            for t in (cache if isinstance(cache, (tuple, list)) else (cache,)):
                _copy_blocks(t, pairs)

    @staticmethod
    def swap_blocks(src: torch.Tensor, dst: torch.Tensor, src_to_dst: torch.Tensor) -> None:
        """Copies whole blocks between two caches (device<->device or device<->pinned host) with one
        launch of the block copy kernel on the current stream; caches the kernel cannot address
        (pageable host memory, other layouts) take the indexing form."""
        _swap_blocks(src, dst, src_to_dst)


def _swap_blocks(src: torch.Tensor, dst: torch.Tensor, src_to_dst: torch.Tensor) -> None:
    def addressable(t):
        return t.is_cuda or t.is_pinned()

    dev = src.device if src.is_cuda else dst.device
    ok = (dev.type == "cuda" and addressable(src) and addressable(dst) and src.dim() == 4 and dst.dim() == 4
          and src.shape[1:] == dst.shape[1:] and src.dtype == dst.dtype and src.stride(3) == 1 and dst.stride(3) == 1
          and (src.shape[3] * src.element_size()) % 16 == 0 and src_to_dst.numel() > 0)
    if not ok:
        s = src_to_dst[:, 0].long()
        d = src_to_dst[:, 1].long()
        dst[d.to(dst.device)] = src[s.to(src.device)].to(dst.device, non_blocking=True)
        return
    import vllm_ascend_b200.distributed.kv_transfer.nvlink_connector  # noqa: F401  (signatures)
    e = src.element_size()
    pairs = src_to_dst.to(torch.int32)
    sb = pairs[:, 0].contiguous().to(dev, non_blocking=True)
    db = pairs[:, 1].contiguous().to(dev, non_blocking=True)
    ptrs = torch.tensor([src.data_ptr(), dst.data_ptr()], dtype=torch.int64).to(dev, non_blocking=True)
    rc = _native.lib().b200_kv_block_copy(
        ptrs[0:1].data_ptr(), ptrs[1:2].data_ptr(), sb.data_ptr(), db.data_ptr(), pairs.shape[0], 1,
        src.shape[1], src.shape[3] * e, src.shape[2], 0, 0,
        src.stride(0) * e, src.stride(1) * e, src.stride(2) * e,
        dst.stride(0) * e, dst.stride(1) * e, dst.stride(2) * e,
        src.shape[0], dst.shape[0], _native.status_word(dev).data_ptr(), _native.stream_ptr())
    _native.check(rc, "swap_blocks")
    _native.count_launch()


_TRAINING_CONSISTENT = False


def set_training_consistent_attention(on: bool) -> None:
    global _TRAINING_CONSISTENT
    _TRAINING_CONSISTENT = bool(on)


def training_consistent_attention() -> bool:
    return _TRAINING_CONSISTENT


class B200FAImpl(B200AttentionImpl):
    """One attention kernel for every batch shape: prefill, chunked prefill, mixed batches and
    decode all run the tcgen05 tile kernel with a single KV split, so the value computed for a
    token does not depend on whether it was scheduled alone, in a chunk, or next to decodes — the
    kernel an RL trainer's forward pass runs (full-sequence causal attention) and the rollout
    engine then agree.  Role of the reference's FA3 backend for training-inference consistency
    (vllm_ascend/attention/fa3_v1.py:44-144, selected by platform.py:1247-1272); like it, the
    mode has no sliding-window support and is slower for decode."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        if self.sliding_window:
            raise ValueError("the training-consistent attention backend does not support sliding windows")

    def forward(self, q, k_cache, v_cache, meta, out=None):
        if out is None:
            out = torch.empty_like(q)
        if not q.is_cuda:
            return super().forward(q, k_cache, v_cache, meta, out)
        return ops.paged_attention_consistent(q, k_cache, v_cache, meta, self.scale, out)


class B200FABackend(B200AttentionBackend):
    @staticmethod
    def get_name() -> str:
        return "B200_TCGEN05_CONSISTENT"

    @staticmethod
    def get_impl_cls():
        return B200FAImpl


def _copy_blocks(t: torch.Tensor, pairs: torch.Tensor) -> None:
    base = t
    # the HND cache is a permuted view; copy on its dense storage
    if not base.is_contiguous():
        base = base.permute(0, 2, 1, 3)
    if base.is_cuda and base.is_contiguous():
        block_bytes = base[0].numel() * base.element_size()
        import vllm_ascend_b200.distributed.kv_transfer.nvlink_connector  # noqa: F401  (signatures)
        p = pairs.to(base.device)
        _native.check(_native.lib().b200_copy_blocks(base.data_ptr(), p.data_ptr(), p.shape[0], block_bytes,
                                                     _native.stream_ptr()), "copy_blocks")
        _native.count_launch()
        return
    src = pairs[:, 0].to(t.device)
    dst = pairs[:, 1].to(t.device)
    t[dst] = t[src]


_ATTN_BACKENDS = {
    # (use_mla, use_sparse, use_compress) -> backend class path (the reference's table:
    # vllm_ascend/platform.py:216-242)
    (False, False, False): "vllm_ascend_b200.attention.backend.B200AttentionBackend",
    (True, False, False): "vllm_ascend_b200.attention.mla.B200MLABackend",
    (True, True, False): "vllm_ascend_b200.attention.sfa.B200SFABackend",
}


def attn_backend_path(use_mla: bool = False, use_sparse: bool = False, use_compress: bool = False) -> str:
    """Dotted path of the backend class for a layer kind.  One table for the platform hook a host
    vLLM queries (``B200Platform.get_attn_backend_cls``) and for this package's own model code."""
    key = (bool(use_mla), bool(use_sparse), bool(use_compress))
    from ..platform_config import get_b200_config
    rl = get_b200_config().rl_config
    if rl.enabled and rl.enable_training_consistency:
        if key != (False, False, False):
            raise ValueError("the training-consistent attention backend supports neither MLA nor sparse attention")
        return "vllm_ascend_b200.attention.backend.B200FABackend"
    if key not in _ATTN_BACKENDS:
        raise ValueError(f"no attention backend for use_mla={key[0]} use_sparse={key[1]} use_compress={key[2]}")
    return _ATTN_BACKENDS[key]


def get_attn_backend(use_mla: bool = False, use_sparse: bool = False, use_compress: bool = False):
    import importlib
    mod, cls = attn_backend_path(use_mla, use_sparse, use_compress).rsplit(".", 1)
    return getattr(importlib.import_module(mod), cls)
