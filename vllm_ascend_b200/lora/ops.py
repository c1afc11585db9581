"""LoRA gather-matvec ops: CUDA kernels on GPU tensors, fp32 torch math otherwise.

Python surface of the reference's native LoRA ops (vllm_ascend/lora/lora_ops.py:19-122):
bgmv_shrink / bgmv_expand(+slice) for one-adapter-per-token batches, sgmv_shrink /
sgmv_expand(+slice) for segments of tokens sharing an adapter.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from .. import _native

P, I, L, F = c_void_p, c_int, c_long, c_float
_native.register_signature("b200_bgmv_shrink", [P, L, P, L, P, P, I, I, I, I, F, I, P, P])
_native.register_signature("b200_bgmv_expand", [P, I, I, P, L, P, P, L, I, I, I, I, I, I, P, P])
_native.register_signature("b200_sgmv_shrink", [P, L, P, L, P, P, P, P, P, I, P, I, I, I, F, I, P, P])
_native.register_signature("b200_sgmv_expand", [P, I, I, P, L, P, P, P, P, P, I, P, L, I, I, I, I, I, P, P])

SG_TOK = 8


class Segments:
    """Segment description for sgmv: consecutive tokens [start, start+len) share ``slot``."""

    def __init__(self, starts, lens, slots, device):
        import numpy as np
        starts, lens, slots = (np.asarray(a, dtype=np.int32) for a in (starts, lens, slots))
        tile_seg, tile_tok0 = [], []
        for s, (st, ln) in enumerate(zip(starts, lens)):
            for t0 in range(int(st), int(st + ln), SG_TOK):
                tile_seg.append(s)
                tile_tok0.append(t0)
        self.num_tiles = len(tile_seg)
        self.num_tokens = int((starts + lens).max()) if len(starts) else 0
        packed = np.concatenate([starts, lens, slots, np.asarray(tile_seg, np.int32),
                                 np.asarray(tile_tok0, np.int32)]).astype(np.int32)
        t = torch.from_numpy(packed)
        if device.type == "cuda":
            t = t.pin_memory().to(device, non_blocking=True)
        n, m = len(starts), self.num_tiles
        self.starts, self.lens, self.slots = t[:n], t[n:2 * n], t[2 * n:3 * n]
        self.tile_seg, self.tile_tok0 = t[3 * n:3 * n + m], t[3 * n + m:]
        self.token_slots = torch.repeat_interleave(self.slots.long(), self.lens.long()).int() \
            if n else torch.zeros(0, dtype=torch.int32, device=device)


def _native_ok(*ts) -> bool:
    return all(t.is_cuda for t in ts) and ts[0].dtype == torch.bfloat16


def bgmv_shrink(x: torch.Tensor, A: torch.Tensor, slots: torch.Tensor, scale: float = 1.0,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, K], A [S, R, K], slots [T] int32 -> v [T, R] fp32 (= scale * A[slot] @ x)."""
    T, K = x.shape
    S, R, _ = A.shape
    if out is None:
        out = torch.empty((T, R), dtype=torch.float32, device=x.device)
    if not _native_ok(x, A):
        valid = slots >= 0
        a = A[slots.clamp(min=0).long()].float()                     # [T, R, K]
        v = torch.einsum("trk,tk->tr", a, x.float()) * scale
        out.copy_(torch.where(valid[:, None], v, torch.zeros_like(v)))
        return out
    assert x.stride(1) == 1 and A.is_contiguous()
    rc = _native.lib().b200_bgmv_shrink(x.data_ptr(), x.stride(0), A.data_ptr(), A.stride(0), slots.data_ptr(),
                                        out.data_ptr(), out.stride(0), T, R, K, scale, S,
                                        _native.status_word(x.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "bgmv_shrink")
    _native.count_launch()
    return out


def bgmv_expand(v: torch.Tensor, B: torch.Tensor, slots: torch.Tensor, y: torch.Tensor, y_offset: int = 0,
                v_offset: int = 0, add: bool = True) -> torch.Tensor:
    """v [T, >=v_offset+R] fp32, B [S, N, R] -> y[:, y_offset:y_offset+N] (+)= B[slot] @ v."""
    T = y.shape[0]
    S, N, R = B.shape
    if not _native_ok(y, B):
        valid = slots >= 0
        b = B[slots.clamp(min=0).long()].float()                     # [T, N, R]
        d = torch.einsum("tnr,tr->tn", b, v[:, v_offset:v_offset + R].float())
        d = torch.where(valid[:, None], d, torch.zeros_like(d))
        sl = y[:, y_offset:y_offset + N]
        sl.copy_((sl.float() + d if add else torch.where(valid[:, None], d, sl.float())).to(y.dtype))
        return y
    assert y.stride(1) == 1 and B.is_contiguous()
    rc = _native.lib().b200_bgmv_expand(v.data_ptr(), v.stride(0), v_offset, B.data_ptr(), B.stride(0),
                                        slots.data_ptr(), y.data_ptr(), y.stride(0), y_offset, T, N, R, S,
                                        int(add), _native.status_word(y.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "bgmv_expand")
    _native.count_launch()
    return y


def sgmv_shrink(x: torch.Tensor, A: torch.Tensor, seg: Segments, scale: float = 1.0,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    T, K = x.shape
    S, R, _ = A.shape
    if out is None:
        out = torch.zeros((T, R), dtype=torch.float32, device=x.device)
    if not _native_ok(x, A):
        return bgmv_shrink(x, A, _pad_slots(seg, T), scale, out)
    rc = _native.lib().b200_sgmv_shrink(x.data_ptr(), x.stride(0), A.data_ptr(), A.stride(0), seg.starts.data_ptr(),
                                        seg.lens.data_ptr(), seg.slots.data_ptr(), seg.tile_seg.data_ptr(),
                                        seg.tile_tok0.data_ptr(), seg.num_tiles, out.data_ptr(), out.stride(0),
                                        R, K, scale, S, _native.status_word(x.device).data_ptr(),
                                        _native.stream_ptr())
    _native.check(rc, "sgmv_shrink")
    _native.count_launch()
    return out


def sgmv_expand(v: torch.Tensor, B: torch.Tensor, seg: Segments, y: torch.Tensor, y_offset: int = 0,
                v_offset: int = 0, add: bool = True) -> torch.Tensor:
    S, N, R = B.shape
    if not _native_ok(y, B):
        return bgmv_expand(v, B, _pad_slots(seg, y.shape[0]), y, y_offset, v_offset, add)
    rc = _native.lib().b200_sgmv_expand(v.data_ptr(), v.stride(0), v_offset, B.data_ptr(), B.stride(0),
                                        seg.starts.data_ptr(), seg.lens.data_ptr(), seg.slots.data_ptr(),
                                        seg.tile_seg.data_ptr(), seg.tile_tok0.data_ptr(), seg.num_tiles,
                                        y.data_ptr(), y.stride(0), y_offset, N, R, S, int(add),
                                        _native.status_word(y.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "sgmv_expand")
    _native.count_launch()
    return y


def _pad_slots(seg: Segments, T: int) -> torch.Tensor:
    s = torch.full((T,), -1, dtype=torch.int32, device=seg.slots.device)
    s[:seg.token_slots.numel()] = seg.token_slots
    return s
