"""Device-side bookkeeping ops (``csrc/small_ops.cu``) with their PyTorch definitions.

Each function runs the CUDA kernel when its tensors are on a GPU (in stream order, so it can sit
inside a captured graph) and the plain PyTorch definition on the host; the tests compare the two.

* ``slot_mapping`` / ``expand_block_table``: the block-table kernels of
  vllm_ascend/worker/block_table.py:28-358 (slot of every token from the request's block row; a
  memory-manager block split into several attention-kernel blocks for hybrid models).
* ``bincount``: per-request token histograms for the penalties (vllm_ascend/ops/triton/penalty.py).
* ``scatter_nd_update``: rows written at N-d indices (csrc/moe/scatter_nd_update_v2).
* ``sign_bits_pack`` / ``sign_bits_unpack``: 1-bit sign encodings (csrc/torch_binding.cpp:496
  ``npu_sign_bits_pack``).
* ``swap_blocks``: whole KV blocks between two caches (device, peer, pinned host) through the block
  copy kernel.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from .. import _native

P, I, L, F = c_void_p, c_int, c_long, c_float
_native.register_signature("b200_slot_mapping", [P, L, I, P, P, I, I, L, P, P, P])
_native.register_signature("b200_expand_block_table", [P, L, P, L, I, I, I, P])
_native.register_signature("b200_bincount", [P, P, L, P, I, I, P])
_native.register_signature("b200_scatter_nd_update", [P, P, P, L, I, P, L, P, P])
_native.register_signature("b200_sign_bits_pack", [P, L, I, P, P])
_native.register_signature("b200_sign_bits_unpack", [P, L, F, I, P, P])


def _launch(rc: int, what: str) -> None:
    _native.check(rc, what)
    _native.count_launch()


def slot_mapping(block_table: torch.Tensor, req_idx: torch.Tensor, positions: torch.Tensor, block_size: int,
                 num_blocks: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """block_table int32 [R, B]; req_idx int32 [T] (negative = padding); positions int64 [T].
    Returns int64 [T] slots (-1 for padding and for out-of-range rows)."""
    T = req_idx.shape[0]
    if out is None:
        out = torch.empty(T, dtype=torch.int64, device=req_idx.device)
    if block_table.is_cuda:
        if block_table.dtype != torch.int32 or req_idx.dtype != torch.int32 or positions.dtype != torch.int64 \
                or block_table.stride(1) != 1:
            raise ValueError("slot_mapping takes an int32 block table (unit inner stride), int32 request rows "
                             "and int64 positions")
        _launch(_native.lib().b200_slot_mapping(
            block_table.data_ptr(), block_table.stride(0), block_table.shape[1], req_idx.data_ptr(),
            positions.data_ptr(), T, block_size, num_blocks, out.data_ptr(),
            _native.status_word(block_table.device).data_ptr(), _native.stream_ptr()), "slot_mapping")
        return out
    r = req_idx.long()
    p = positions.long()
    bi = torch.div(p, block_size, rounding_mode="floor")
    ok = (r >= 0) & (p >= 0) & (bi < block_table.shape[1])
    b = block_table[r.clamp(min=0), bi.clamp(0, block_table.shape[1] - 1)].long()
    ok &= (b >= 0) & (b < num_blocks)
    out.copy_(torch.where(ok, b * block_size + (p - bi * block_size), torch.full_like(p, -1)))
    return out


def expand_block_table(block_table: torch.Tensor, ratio: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """int32 [R, B] of manager blocks -> int32 [R, B * ratio] of kernel blocks."""
    R, B = block_table.shape
    if out is None:
        out = torch.empty((R, B * ratio), dtype=torch.int32, device=block_table.device)
    if block_table.is_cuda:
        if block_table.dtype != torch.int32 or block_table.stride(1) != 1 or out.stride(1) != 1:
            raise ValueError("expand_block_table takes int32 tables with unit inner stride")
        _launch(_native.lib().b200_expand_block_table(block_table.data_ptr(), block_table.stride(0), out.data_ptr(),
                                                      out.stride(0), R, B, ratio, _native.stream_ptr()),
                "expand_block_table")
        return out
    j = torch.arange(ratio, dtype=torch.int32)
    e = block_table[:, :, None] * ratio + j[None, None, :]
    e = torch.where(block_table[:, :, None] < 0, torch.full_like(e, -1), e)
    out[:, :B * ratio] = e.reshape(R, B * ratio)
    return out


def bincount(ids: torch.Tensor, rows: Optional[torch.Tensor], num_rows: int, vocab: int,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """ids int64 [n], rows int32 [n] (None: one row).  Adds into ``out`` int32 [num_rows, vocab]."""
    if out is None:
        out = torch.zeros((num_rows, vocab), dtype=torch.int32, device=ids.device)
    n = ids.numel()
    if ids.is_cuda:
        if ids.dtype != torch.int64 or (rows is not None and rows.dtype != torch.int32) or not out.is_contiguous():
            raise ValueError("bincount takes int64 ids, int32 rows and a contiguous int32 output")
        _launch(_native.lib().b200_bincount(ids.data_ptr(), _native.ptr(rows), n, out.data_ptr(), num_rows, vocab,
                                            _native.stream_ptr()), "bincount")
        return out
    r = rows.long() if rows is not None else torch.zeros(n, dtype=torch.long)
    ok = (ids >= 0) & (ids < vocab) & (r >= 0) & (r < num_rows)
    flat = out.view(-1)
    flat.index_add_(0, (r[ok] * vocab + ids[ok]), torch.ones(int(ok.sum()), dtype=torch.int32))
    return out


def scatter_nd_update(var: torch.Tensor, indices: torch.Tensor, updates: torch.Tensor) -> torch.Tensor:
    """``var[tuple(indices[i])] = updates[i]`` for indices int64 [n, k] over var's k leading dims (in place)."""
    n, k = indices.shape
    if not 1 <= k <= min(4, var.dim()):
        raise ValueError("indices must address 1 to 4 leading dimensions of var")
    if updates.shape != (n, *var.shape[k:]) or updates.dtype != var.dtype:
        raise ValueError(f"updates must be {(n, *var.shape[k:])} of {var.dtype}")
    if var.is_cuda:
        if not (var.is_contiguous() and updates.is_contiguous() and indices.is_contiguous()) \
                or indices.dtype != torch.int64:
            raise ValueError("scatter_nd_update takes contiguous tensors and int64 indices")
        row_bytes = var[(0,) * k].numel() * var.element_size() if var.numel() else 0
        dims = (c_long * 4)(*(list(var.shape[:k]) + [1] * (4 - k)))
        _launch(_native.lib().b200_scatter_nd_update(var.data_ptr(), indices.data_ptr(), updates.data_ptr(), n, k,
                                                     dims, row_bytes, _native.status_word(var.device).data_ptr(),
                                                     _native.stream_ptr()), "scatter_nd_update")
        return var
    ok = torch.ones(n, dtype=torch.bool)
    for a in range(k):
        ok &= (indices[:, a] >= 0) & (indices[:, a] < var.shape[a])
    var[tuple(indices[ok, a] for a in range(k))] = updates[ok]
    return var


def sign_bits_pack(x: torch.Tensor) -> torch.Tensor:
    """uint8 [ceil(n / 8)]: bit b of byte j is the sign bit of element 8 j + b of the flattened input."""
    flat = x.contiguous().view(-1)
    n = flat.numel()
    if x.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise ValueError("sign_bits_pack takes bf16, fp16 or fp32")
    out = torch.empty((n + 7) // 8, dtype=torch.uint8, device=x.device)
    if x.is_cuda:
        _launch(_native.lib().b200_sign_bits_pack(flat.data_ptr(), n, x.element_size(), out.data_ptr(),
                                                  _native.stream_ptr()), "sign_bits_pack")
        return out
    bits = torch.signbit(flat).to(torch.uint8)
    bits = torch.nn.functional.pad(bits, (0, out.numel() * 8 - n)).view(-1, 8)
    w = (1 << torch.arange(8, dtype=torch.int32))
    out.copy_((bits.int() * w).sum(-1).to(torch.uint8))
    return out


def sign_bits_unpack(packed: torch.Tensor, n: int, scale: float = 1.0, dtype=torch.float32) -> torch.Tensor:
    """Inverse of ``sign_bits_pack``: +scale / -scale per element."""
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("sign_bits_unpack writes bf16 or fp32")
    y = torch.empty(n, dtype=dtype, device=packed.device)
    if packed.is_cuda:
        _launch(_native.lib().b200_sign_bits_unpack(packed.data_ptr(), n, float(scale), y.element_size(),
                                                    y.data_ptr(), _native.stream_ptr()), "sign_bits_unpack")
        return y
    e = torch.arange(n)
    bit = (packed[e >> 3].int() >> (e & 7).int()) & 1
    y.copy_(torch.where(bit.bool(), -scale, scale).to(dtype))
    return y
