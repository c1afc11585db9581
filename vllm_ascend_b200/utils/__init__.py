"""Small shared helpers: cached side streams, feature predicates, the table of out-of-tree ops
registered with a host vLLM, weak tensor references.

Counterparts in the reference: cached side streams (vllm_ascend/utils.py:480-526), feature
predicates ``enable_sp`` / ``lmhead_tp_enable`` / ``oproj_tp_enable`` / ``mlp_tp_enable`` /
``is_moe_model`` (utils.py:787-833), the OOT custom-op table (utils.py:656-784), weak-ref
tensors for graph outputs (utils.py:910-946), ``refresh_block_size`` (utils.py:1162-1212).
"""
from __future__ import annotations

import weakref
from typing import Any, Optional

import torch

_STREAMS: dict[tuple, "torch.cuda.Stream"] = {}


def side_stream(name: str, device: Optional[torch.device] = None) -> "torch.cuda.Stream":
    """One long-lived stream per (purpose, device): "prefetch", "shared_expert", "kv_transfer", ..."""
    dev = device or torch.device("cuda", torch.cuda.current_device())
    key = (name, dev.index)
    s = _STREAMS.get(key)
    if s is None:
        s = _STREAMS[key] = torch.cuda.Stream(device=dev)
    return s


# ---------------------------------------------------------------- feature predicates
def enable_sp(engine_cfg) -> bool:
    """Sequence-parallel residual stream (token-sharded between TP ranks)."""
    return bool(engine_cfg.parallel.enable_sequence_parallel) and engine_cfg.parallel.tensor_parallel_size > 1


def is_moe_model(engine_cfg) -> bool:
    return bool(engine_cfg.model.is_moe)


def _fg(engine_cfg, name: str) -> int:
    from ..platform_config import finegrained_sizes
    return int(finegrained_sizes(engine_cfg.additional_config).get(name, 0) or 0)


def lmhead_tp_enable(engine_cfg) -> bool:
    return _fg(engine_cfg, "lmtp") > 1


def oproj_tp_enable(engine_cfg) -> bool:
    return _fg(engine_cfg, "otp") > 1


def mlp_tp_enable(engine_cfg) -> bool:
    return _fg(engine_cfg, "mlp_tp") > 1


def embedding_tp_enable(engine_cfg) -> bool:
    return _fg(engine_cfg, "embed_tp") > 1


def refresh_block_size(cache_cfg, default: int = 128) -> int:
    """KV block size defaults to the attention kernels' tile height."""
    if not getattr(cache_cfg, "block_size", None):
        cache_cfg.block_size = default
    return cache_cfg.block_size


def should_skip_allreduce_across_dp_group(engine_cfg, is_decode_only: bool) -> bool:
    """The per-step DP all-reduce of (num_tokens, graph mode) is only needed when the ranks
    must agree on padding: MoE models with expert parallelism.  Dense DP replicas are
    independent (vllm_ascend/utils.py:1099-1149)."""
    pc = engine_cfg.parallel
    if pc.data_parallel_size <= 1:
        return True
    return not (engine_cfg.model.is_moe and pc.enable_expert_parallel)


# ---------------------------------------------------------------- weak tensor references
def weak_ref_tensor(t: Any) -> Any:
    """A view that does not keep the storage's allocation alive in the caching allocator's
    bookkeeping: graph outputs are held this way so the graph pool can reuse their memory."""
    if isinstance(t, torch.Tensor):
        return torch.as_strided(t.detach(), t.shape, t.stride(), t.storage_offset()) if not t.is_cuda else \
            _cuda_alias(t)
    if isinstance(t, (list, tuple)):
        return type(t)(weak_ref_tensor(x) for x in t)
    return t


def _cuda_alias(t: torch.Tensor) -> torch.Tensor:
    from ..parallel.symm_mem import _RawCudaBuffer
    nbytes = t.untyped_storage().nbytes() - t.storage_offset() * t.element_size()
    raw = torch.as_tensor(_RawCudaBuffer(t.data_ptr(), nbytes), device=t.device)
    return torch.as_strided(raw.view(t.dtype), t.shape, t.stride(), 0)


class TensorTracker:
    """Debug aid: remembers tensors weakly and reports which are still alive."""

    def __init__(self):
        self._refs: list = []

    def track(self, name: str, t: torch.Tensor) -> None:
        self._refs.append((name, weakref.ref(t)))

    def alive(self) -> list[str]:
        return [n for n, r in self._refs if r() is not None]
