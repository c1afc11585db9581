"""Native (sm_100a) MoE path on one rank: gating kernel, expert-major permutation,
grouped tcgen05 GEMMs (bf16 with fused SwiGLU, or block-scaled fp8), weighted combine.

Pipeline parity: ``moe_init_routing`` -> grouped GEMM1 + SwiGLU (+ requant) -> grouped
GEMM2 -> ``moe_token_unpermute`` (vllm_ascend/ops/fused_moe/token_dispatcher.py:367-461,
moe_mlp.py:174-687).
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from .. import _native
from . import launch_counter, quant_fp8_group128, silu_and_mul

P, I, L, F = c_void_p, c_int, c_long, c_float
_native.register_signature("b200_moe_gating_topk", [P, P, P, P, I, I, I, I, I, I, I, F, P])
_native.register_signature("b200_moe_permute", [P, I, I, I, P, P, P, P, P, P])
_native.register_signature("b200_moe_gather_rows", [P, P, P, I, I, I, P, P])
_native.register_signature("b200_moe_combine", [P, P, P, I, I, I, P, I, P])
_native.register_signature("b200_grouped_gemm_fp8_block",
                           [P, P, P, P, P, P, I, L, I, I, I, I, I, P, P])


def available() -> bool:
    return _native.available() and hasattr(_native.lib(), "b200_moe_permute")


def gating_topk(logits: torch.Tensor, k: int, scoring: str, renorm: bool, n_group: int,
                topk_group: int, bias: Optional[torch.Tensor], scale: float):
    T, E = logits.shape
    logits = logits.float().contiguous()
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    rc = _native.lib().b200_moe_gating_topk(
        logits.data_ptr(), _native.ptr(bias), w.data_ptr(), ids.data_ptr(), T, E, k,
        0 if scoring == "softmax" else 1, int(renorm), n_group, topk_group, scale,
        _native.stream_ptr())
    _native.check(rc, "moe_gating_topk")
    launch_counter[0] += 1
    return w, ids


class Permutation:
    """Expert-major ordering of the (token, slot) pairs routed to this rank's experts."""

    def __init__(self, topk_ids: torch.Tensor, expert_map: Optional[torch.Tensor], E_local: int):
        T, k = topk_ids.shape
        dev = topk_ids.device
        ids = topk_ids.to(torch.int32)
        if expert_map is not None:
            ids = expert_map[ids.long()].to(torch.int32)
        self.local_ids = ids.contiguous()
        self.T, self.k, self.E = T, k, E_local
        ws = torch.empty(3 * E_local + 1, dtype=torch.int32, device=dev)
        self.counts, self.cursor = ws[:E_local], ws[E_local:2 * E_local]
        self.offsets = ws[2 * E_local:]
        self.pos = torch.empty(T * k, dtype=torch.int32, device=dev)
        self.src_token = torch.empty(max(T * k, 1), dtype=torch.int32, device=dev)
        rc = _native.lib().b200_moe_permute(
            self.local_ids.data_ptr(), T, k, E_local, self.counts.data_ptr(),
            self.cursor.data_ptr(), self.offsets.data_ptr(), self.pos.data_ptr(),
            self.src_token.data_ptr(), _native.stream_ptr())
        _native.check(rc, "moe_permute")
        launch_counter[0] += 3
        self.max_rows = T * k                      # rows beyond offsets[E] stay unused

    def gather(self, x: torch.Tensor) -> torch.Tensor:
        H = x.shape[1]
        out = torch.empty((max(self.max_rows, 1), H), dtype=x.dtype, device=x.device)
        rc = _native.lib().b200_moe_gather_rows(
            x.data_ptr(), self.src_token.data_ptr(), self.offsets.data_ptr(), self.E, H,
            self.max_rows, out.data_ptr(), _native.stream_ptr())
        _native.check(rc, "moe_gather_rows")
        launch_counter[0] += 1
        return out

    def combine(self, y: torch.Tensor, topk_w: torch.Tensor, out: Optional[torch.Tensor] = None,
                accumulate: bool = False) -> torch.Tensor:
        H = y.shape[1]
        if out is None:
            out = torch.empty((self.T, H), dtype=y.dtype, device=y.device)
        w = topk_w.float().contiguous()
        rc = _native.lib().b200_moe_combine(y.data_ptr(), self.pos.data_ptr(), w.data_ptr(), self.T,
                                            self.k, H, out.data_ptr(), int(accumulate),
                                            _native.stream_ptr())
        _native.check(rc, "moe_combine")
        launch_counter[0] += 1
        return out


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, swiglu: bool) -> torch.Tensor:
    """a [rows, K] grouped by expert; w [E, N(or 2N), K]; -> [rows, N]."""
    rows, K = a.shape
    E = w.shape[0]
    N = w.shape[1] // 2 if swiglu else w.shape[1]
    out = torch.empty((rows, N), dtype=a.dtype, device=a.device)
    rc = _native.lib().b200_grouped_gemm_bf16(
        a.data_ptr(), w.data_ptr(), out.data_ptr(), offsets.data_ptr(), E, rows, N, K,
        a.stride(0), w.stride(1), out.stride(0), int(swiglu),
        _native.status_word(a.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "grouped_gemm_bf16")
    launch_counter[0] += 1
    return out


def grouped_gemm_fp8(a8, a_scale, w8, w_scale, offsets) -> torch.Tensor:
    rows, K = a8.shape
    E, N = w8.shape[0], w8.shape[1]
    out = torch.empty((rows, N), dtype=torch.bfloat16, device=a8.device)
    rc = _native.lib().b200_grouped_gemm_fp8_block(
        a8.data_ptr(), a_scale.data_ptr(), w8.data_ptr(), w_scale.data_ptr(), out.data_ptr(),
        offsets.data_ptr(), E, rows, N, K, a8.stride(0), w8.stride(1), out.stride(0),
        _native.status_word(a8.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "grouped_gemm_fp8")
    launch_counter[0] += 1
    return out


def fused_experts(x, w13, w2, topk_w, topk_ids, expert_map=None) -> torch.Tensor:
    """bf16 experts: permute -> grouped GEMM1 with SwiGLU epilogue -> grouped GEMM2 -> combine."""
    E, two_i, H = w13.shape
    I_ = two_i // 2
    if x.shape[0] == 0:
        return x.clone()
    if I_ % 128 or H % 8 or E > 512:
        from .fused_moe import fused_experts_ref
        return fused_experts_ref(x, w13, w2, topk_w, topk_ids, expert_map)
    perm = Permutation(topk_ids, expert_map, E)
    xs = perm.gather(x)
    h = grouped_gemm(xs, w13, perm.offsets, swiglu=True)          # [rows, I]
    y = grouped_gemm(h, w2, perm.offsets, swiglu=False)           # [rows, H]
    return perm.combine(y, topk_w)


def fused_experts_fp8(x, w13, w13_scale, w2, w2_scale, topk_w, topk_ids, expert_map=None):
    """Block-scaled fp8 experts: 1x128 activation quant -> grouped fp8 GEMM1 -> SwiGLU ->
    requant -> grouped fp8 GEMM2 -> combine."""
    E, two_i, H = w13.shape
    perm = Permutation(topk_ids, expert_map, E)
    xs = perm.gather(x)
    a8, a_s = quant_fp8_group128(xs)
    h = grouped_gemm_fp8(a8, a_s, w13, w13_scale, perm.offsets)   # [rows, 2I]
    act = silu_and_mul(h)
    b8, b_s = quant_fp8_group128(act)
    y = grouped_gemm_fp8(b8, b_s, w2, w2_scale, perm.offsets)
    return perm.combine(y, topk_w)
