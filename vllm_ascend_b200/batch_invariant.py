"""Batch-invariant (run-to-run and batch-size independent) execution mode.

What changes a result with the batch composition here is the reduction order, and only two
places choose it from the batch: the split-KV factor of decode attention and the collective
algorithm.  The GEMM kernels accumulate every output element over K in one fixed order
whatever the tile shape, the norm/activation kernels reduce per row.  So the mode pins the
split factor to 1 and the collectives to a fixed algorithm; the reference reaches the same
goal by swapping aten matmul/softmax/mean/rmsnorm for batch-invariant kernels and setting
deterministic collective variables (vllm_ascend/batch_invariant.py:76-162).
"""
from __future__ import annotations

import os

_enabled = False


def is_batch_invariant() -> bool:
    return _enabled or os.getenv("VLLM_B200_BATCH_INVARIANT", "0") == "1"


def enable_batch_invariant_mode() -> None:
    global _enabled
    _enabled = True
    os.environ["VLLM_B200_BATCH_INVARIANT"] = "1"
    # fixed NCCL algorithm/protocol: reduction order no longer depends on message size heuristics
    os.environ.setdefault("NCCL_ALGO", "Ring")
    os.environ.setdefault("NCCL_PROTO", "Simple")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    try:
        import torch
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.deterministic = True
    except Exception:
        pass


def disable_batch_invariant_mode() -> None:
    global _enabled
    _enabled = False
    os.environ["VLLM_B200_BATCH_INVARIANT"] = "0"
