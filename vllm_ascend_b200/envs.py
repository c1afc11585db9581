"""Lazily evaluated environment-variable table.

Every variable is read at attribute access time (not import time) so tests can
monkeypatch ``os.environ``.  Parity: vllm_ascend/envs.py:30-108 (same lazy
``__getattr__`` contract, B200-relevant names).
"""
from __future__ import annotations

import os
from typing import Any, Callable


def _bool(name: str, default: str = "0") -> Callable[[], bool]:
    return lambda: os.getenv(name, default).strip().lower() in ("1", "true", "yes", "on")


def _int(name: str, default: int) -> Callable[[], int]:
    return lambda: int(os.getenv(name, str(default)))


def _str(name: str, default: str | None = None) -> Callable[[], str | None]:
    return lambda: os.getenv(name, default)


env_variables: dict[str, Callable[[], Any]] = {
    # ---- build ----
    "MAX_JOBS": _int("MAX_JOBS", 8),
    "CMAKE_BUILD_TYPE": _str("CMAKE_BUILD_TYPE", "Release"),
    "COMPILE_CUSTOM_KERNELS": _bool("COMPILE_CUSTOM_KERNELS", "1"),
    # ---- kernel selection (one native path per op; these only exist to fall
    # back to the library path while a kernel is being validated) ----
    # bf16 GEMM: "tcgen05" (hand-written) or "cublas" (plain library GEMM)
    "VLLM_B200_GEMM": _str("VLLM_B200_GEMM", "tcgen05"),
    # paired-CTA (cta_group::2) GEMM for M >= this many rows; 0 disables it
    "VLLM_B200_GEMM_2CTA_MIN_M": _int("VLLM_B200_GEMM_2CTA_MIN_M", 256),
    # prefill attention: "tcgen05" or "sdpa" (torch fallback/oracle)
    "VLLM_B200_PREFILL_ATTN": _str("VLLM_B200_PREFILL_ATTN", "tcgen05"),
    "VLLM_B200_DECODE_ATTN": _str("VLLM_B200_DECODE_ATTN", "native"),
    # MLA attention: "tcgen05" (absorbed-weight kernel) or "torch" (oracle)
    "VLLM_B200_MLA_ATTN": _str("VLLM_B200_MLA_ATTN", "tcgen05"),
    # TP collectives of the linear layers: "fused" (inside the GEMM kernels over peer memory),
    # "nccl" (all-reduce), or "auto" (both are timed at start-up, per step class, the faster one serves)
    "VLLM_B200_TP_COMM": _str("VLLM_B200_TP_COMM", "fused"),
    # "1" (default): dense bf16 decoders on one GPU fold RMSNorm into the neighbouring GEMMs; "0": off
    "VLLM_B200_FOLD_NORM": _str("VLLM_B200_FOLD_NORM", "1"),
    # 128-key tiles the decode-attention kernel requests into L2 ahead of its staged K / V loads (0 = off)
    "VLLM_B200_DECODE_L2_PREFETCH": _int("VLLM_B200_DECODE_L2_PREFETCH", 0),
    # "1": let a multi-rank NCCL engine enter sleep mode (off: such a cycle has not completed on this hardware)
    "VLLM_B200_SLEEP_WITH_NCCL": _bool("VLLM_B200_SLEEP_WITH_NCCL", "0"),
    # gated delta rule: sequences with at least this many new tokens in a step (prefill chunks) take the
    # chunk-parallel form (matrix products per 64-token chunk) instead of the per-token recurrence; 0 = never.
    # Unset: 64 for host tensors, never on the GPU (the recurrence kernel is faster there)
    "VLLM_B200_GDN_CHUNK_MIN": _int("VLLM_B200_GDN_CHUNK_MIN", 64),
    # "1": the slot of every token is computed on the device from the block table (one small kernel per
    # step) instead of on the host; "0" (default): host numpy + copy
    "VLLM_B200_DEVICE_SLOT_MAPPING": _str("VLLM_B200_DEVICE_SLOT_MAPPING", "0"),
    # fused TP path and NVSwitch multicast memory: "auto" pushes the all-gather rows with multimem.st
    # when the platform offers multicast, "full" also sums the partials in the switch
    # (multimem.ld_reduce), "push" forces the multicast push at any group size, "0" uses peer loads /
    # stores only
    "VLLM_B200_NVLS": _str("VLLM_B200_NVLS", "auto"),
    # "auto" uses multicast up to this many ranks per TP group ("push" / "full" force it at any size)
    "VLLM_B200_NVLS_AUTO_MAX_RANKS": _int("VLLM_B200_NVLS_AUTO_MAX_RANKS", 2),
    # MoE path override: "", "allgather", "alltoall", "fused"
    "VLLM_B200_MOE_COMM": _str("VLLM_B200_MOE_COMM", ""),
    "VLLM_B200_ENABLE_NVLS": _bool("VLLM_B200_ENABLE_NVLS", "0"),
    # device-side bounded wait, in microseconds of globaltimer
    "VLLM_B200_WAIT_TIMEOUT_US": _int("VLLM_B200_WAIT_TIMEOUT_US", 1_000_000),
    # ---- runtime features (names follow the reference where they make sense) ----
    "DYNAMIC_EPLB": _bool("DYNAMIC_EPLB", "0"),
    "VLLM_B200_ENABLE_FUSED_MOE_COMM": _bool("VLLM_B200_ENABLE_FUSED_MOE_COMM", "1"),
    "VLLM_B200_BALANCE_SCHEDULING": _bool("VLLM_B200_BALANCE_SCHEDULING", "0"),
    "VLLM_B200_ENABLE_BATCH_MEMCPY": _bool("VLLM_B200_ENABLE_BATCH_MEMCPY", "1"),
    "VLLM_B200_TRANSPOSE_KV_CACHE_BY_BLOCK": _bool("VLLM_B200_TRANSPOSE_KV_CACHE_BY_BLOCK", "1"),
    "VLLM_B200_KV_ABORT_REQUEST_TIMEOUT": _int("VLLM_B200_KV_ABORT_REQUEST_TIMEOUT", 480),
    "VLLM_B200_LOG_PATH": _str("VLLM_B200_LOG_PATH", None),
    "VLLM_B200_ENABLE_CPU_BINDING": _bool("VLLM_B200_ENABLE_CPU_BINDING", "1"),
    "VLLM_B200_CUDA_GRAPH": _bool("VLLM_B200_CUDA_GRAPH", "1"),
    # NVTX ranges around the engine's hook points: 0 off, 1 step level (prepare / forward / sample),
    # 2 also one range per decoder layer
    "VLLM_B200_NVTX": _int("VLLM_B200_NVTX", 0),
}


def __getattr__(name: str) -> Any:
    if name in env_variables:
        return env_variables[name]()
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__() -> list[str]:
    return list(env_variables.keys())
