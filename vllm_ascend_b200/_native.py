"""ctypes binding of the in-tree native library ``_C.so`` (plain C ABI).

The library is built by ``vllm_ascend_b200.build`` (sm_100a only).  On a machine
with a GPU a missing library is a hard error: ops never fall back to PyTorch
silently on CUDA tensors.  The role matches the reference's lazy custom-op
loader ``enable_custom_op`` (vllm_ascend/utils.py:397-456).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_uint, c_void_p
from typing import Optional

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_C.so")
_lib: Optional[ctypes.CDLL] = None
_load_error: Optional[str] = None

P, I, L, F, U = c_void_p, c_int, c_long, c_float, c_uint

_SIGNATURES = {
    "b200_gemm_bf16": [P, P, P, P, P, I, I, I, I, I, I, I, P, I, P],
    "b200_gemm_bf16_2cta": [P, P, P, P, P, I, I, I, I, I, I, I, P, P],
    "b200_gemm_bf16_2cta_norm": [P, P, P, P, P, I, I, I, I, I, I, I, P, I, ctypes.c_float, P, L, I, P, P],
    "b200_gemm_swiglu_bf16": [P, P, P, I, I, I, I, I, I, P, P],
    "b200_grouped_gemm_bf16": [P, P, P, P, I, L, I, I, I, I, I, I, P, P],
    "b200_rms_norm": [P, P, P, P, L, I, F, I, L, L, P],
    "b200_silu_and_mul": [P, P, L, I, F, P],
    "b200_embedding": [P, P, P, L, I, L, L, P],
    "b200_qknorm_rope_kvwrite": [P, L, P, P, I, P, P, F, P, P, P, I, I, I, I, L, I, I, P, P],
    "b200_rope_table": [P, L, P, P, L, I, I, I, P],
    "b200_layer_norm": [P, P, P, P, L, I, F, L, L, P],
    "b200_qknorm_mrope_kvwrite": [P, L, P, L, P, P, I, P, P, F, P, P, P, I, I, I, I, L, I, I, P, P],
    "b200_quant_fp8_group128": [P, P, P, L, I, I, P],
    "b200_quant_fp8_per_token": [P, L, P, P, L, I, P],
    "b200_activation": [P, P, L, I, I, I, F, F, P],
    "b200_rms_norm_gated": [P, P, P, P, L, I, F, I, P],
    "b200_rms_norm_quant_fp8": [P, P, P, P, P, L, I, F, I, L, P],
    "b200_silu_mul_quant_fp8": [P, P, P, L, I, F, P],
    "b200_paged_decode": [P, L, P, P, P, I, P, I, I, I, I, I, F, I, I, P, L, P, L, P, P],
    "b200_attn_fwd_tc": [P, L, L, P, P, L, I, P, P, P, I, P, P, I, I, I, I, F, I, I, I, P, L, P,
                         F, U, U, I, P, P],
    "b200_attn_decode_tc": [P, L, L, P, P, L, I, P, P, P, I, I, I, I, I, F, I, I, I, P, L, P, I, P, P, P],
    "b200_attn_decode_tc_lse": [P, L, L, P, P, L, I, P, P, P, I, I, I, I, I, F, I, I, I, P, L, P, I, P, P, P, P],
    "b200_merge_attn_partials": [P, P, L, I, I, I, P, L, P, P],
    "b200_attn_decode_set_l2_prefetch": [I],
    "b200_mla_preprocess": [P, L, I, I, I, I, P, L, I, P, F, P, P, L, P, P, P, L, P, P, P, P],
    "b200_argmax": [P, I, L, I, I, P, P],
    "b200_cast_bf16_f32": [P, L, P, L, I, I, P],
    "b200_apply_penalties": [P, L, I, I, P, I, P, I, P, P, P, P],
    "b200_sample": [P, L, I, I, P, P, P, P, P, P, P, P],
}
_LONG_RET = {"b200_paged_decode_scratch_bytes": [I, I, I, I],
             "b200_attn_scratch_bytes": [L, I, I, I]}


_RESTYPES: dict = {}


def _declare(lib: ctypes.CDLL) -> None:
    for name, argtypes in _SIGNATURES.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, c_int)
    for name, argtypes in _LONG_RET.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_long


def register_signature(name: str, argtypes: list, restype=c_int) -> None:
    """Used by sub-modules that own additional entry points (comm, moe, vmm...)."""
    _SIGNATURES[name] = argtypes
    if restype is not c_int:
        _RESTYPES[name] = restype
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = restype


def load(required: bool = False) -> Optional[ctypes.CDLL]:
    global _lib, _load_error
    if _lib is not None:
        return _lib
    if _load_error is None:
        try:
            _lib = ctypes.CDLL(_LIB_PATH, mode=ctypes.RTLD_GLOBAL)
            _declare(_lib)
        except OSError as e:  # not built
            _load_error = str(e)
    if _lib is None and required:
        raise RuntimeError(
            f"native library {_LIB_PATH} is not available ({_load_error}); "
            "run `python -m vllm_ascend_b200.build`")
    return _lib


def available() -> bool:
    return load() is not None


def lib() -> ctypes.CDLL:
    return load(required=True)  # type: ignore[return-value]


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class NativeError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")


# ---------------------------------------------------------------- status word
_status_words: dict[int, torch.Tensor] = {}

# launches of this package's own kernels (shared list object: ``ops.launch_counter`` aliases it)
launch_counter = [0]


def count_launch(n: int = 1) -> None:
    launch_counter[0] += n


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels set on bounded-wait timeouts or bad
    indices.  The engine reads it between steps (``check_status``)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[idx] = t
    return t


STATUS_NAMES = {0: "OK", 1: "TIMEOUT", 2: "BAD_INDEX", 3: "OVERFLOW"}


def check_status(device: torch.device) -> None:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        return
    v = int(t.item())
    if v != 0:
        t.zero_()
        raise NativeError(f"device kernel reported status {STATUS_NAMES.get(v, v)}")
