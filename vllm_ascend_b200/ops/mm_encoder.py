"""Vision-encoder ops: bidirectional variable-length attention and table-driven rotary embedding.

The reference runs ViT attention through its fused-infer-attention op on unpadded sequences
(vllm_ascend/ops/mm_encoder_attention.py:66-170: pads head_dim to a kernel-friendly size, runs
per-image variable-length attention from cu_seqlens, slices the padding off).  Here the same
contract runs on the tcgen05 prefill kernel: K / V of the image batch are scattered into a
temporary paged layout (128-token blocks, one run of blocks per sequence), head_dim is
zero-padded to 64 or 128, and the kernel runs with causal masking off.  The per-batch plan
(slots, block table, tile work list) is built once and shared by all layers that use the same
cu_seqlens.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .. import _native
from . import reference as ref

_BLOCK = 128


@dataclass
class EncoderAttnPlan:
    cu_seqlens_cpu: np.ndarray            # int32 [B + 1]
    max_len: int
    # device-side plan of the native path (None on CPU)
    slots: Optional[torch.Tensor] = None          # int64 [N] row of every token in the temp cache
    meta: object = None                           # AttentionMetadata-like view for the kernel
    num_blocks: int = 0


def make_plan(cu_seqlens, device) -> EncoderAttnPlan:
    """cu_seqlens: int array [B + 1] of token offsets (host)."""
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    lens = np.diff(cu)
    plan = EncoderAttnPlan(cu.astype(np.int32), int(lens.max()) if len(lens) else 0)
    device = torch.device(device)
    if device.type != "cuda":
        return plan
    from ..attention.metadata import AttentionMetadata, build_tile_worklist
    nblk = (lens + _BLOCK - 1) // _BLOCK
    blk_start = np.concatenate([[0], np.cumsum(nblk)[:-1]])
    N = int(cu[-1])
    seq_of = np.repeat(np.arange(len(lens)), lens)
    slots = blk_start[seq_of] * _BLOCK + (np.arange(N) - cu[:-1][seq_of])
    max_blocks = int(nblk.max()) if len(nblk) else 1
    bt = np.zeros((len(lens), max_blocks), dtype=np.int32)
    for i, (s, n) in enumerate(zip(blk_start, nblk)):
        bt[i, :n] = np.arange(s, s + n)
    tile_seq, tile_qoff = build_tile_worklist(lens.astype(np.int64), _BLOCK, lens.astype(np.int64))

    def dev(a, dt):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dt).to(device)
    plan.slots = dev(slots, torch.int64)
    plan.num_blocks = int(nblk.sum())
    plan.meta = AttentionMetadata(
        num_reqs=len(lens), num_actual_tokens=N, max_query_len=plan.max_len, max_seq_len=plan.max_len,
        query_start_loc=dev(cu, torch.int32), seq_lens=dev(lens, torch.int32),
        block_table=dev(bt, torch.int32), slot_mapping=plan.slots, positions=plan.slots,
        query_start_loc_cpu=cu.astype(np.int32), seq_lens_cpu=lens.astype(np.int32),
        tile_seq=dev(tile_seq, torch.int32), tile_qoff=dev(tile_qoff, torch.int32),
        num_tiles=len(tile_seq))
    return plan


class StaticEncoderPlan(EncoderAttnPlan):
    """Plan with fixed-capacity device buffers, refreshed in place: what a captured CUDA graph of
    the vision tower reads.  Unused sequence slots have length 0 and unused tiles point at such a
    slot, which the kernel leaves at once; the temporary K / V cache has the capacity's block count."""

    def __init__(self, max_tokens: int, max_seqs: int, device):
        from ..attention.metadata import AttentionMetadata
        device = torch.device(device)
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.max_tiles = max_seqs + (max_tokens + _BLOCK - 1) // _BLOCK
        self.max_blocks_per_seq = (max_tokens + _BLOCK - 1) // _BLOCK
        self.cu_seqlens_cpu = np.zeros(max_seqs + 1, dtype=np.int32)
        self.max_len = max_tokens
        self.num_blocks = self.max_tiles
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=device)     # noqa: E731
        self.slots = z((max_tokens,), torch.int64)
        self._qsl, self._sl = z((max_seqs + 1,), torch.int32), z((max_seqs,), torch.int32)
        self._bt = z((max_seqs, self.max_blocks_per_seq), torch.int32)
        self._ts, self._tq = z((self.max_tiles,), torch.int32), z((self.max_tiles,), torch.int32)
        self.meta = AttentionMetadata(
            num_reqs=max_seqs, num_actual_tokens=max_tokens, max_query_len=max_tokens, max_seq_len=max_tokens,
            query_start_loc=self._qsl, seq_lens=self._sl, block_table=self._bt, slot_mapping=self.slots,
            positions=self.slots, query_start_loc_cpu=self.cu_seqlens_cpu, seq_lens_cpu=np.zeros(max_seqs, np.int32),
            tile_seq=self._ts, tile_qoff=self._tq, num_tiles=self.max_tiles)

    def update(self, cu_seqlens) -> None:
        """cu_seqlens must end at max_tokens (the caller appends the padding rows as a sequence)."""
        from ..attention.metadata import build_tile_worklist
        cu = np.asarray(cu_seqlens, dtype=np.int64)
        lens = np.diff(cu)
        B = len(lens)
        if B > self.max_seqs - 1 or int(cu[-1]) != self.max_tokens:
            raise ValueError("sequence list does not fit the static plan")
        nblk = (lens + _BLOCK - 1) // _BLOCK
        blk_start = np.concatenate([[0], np.cumsum(nblk)[:-1]])
        seq_of = np.repeat(np.arange(B), lens)
        slots = blk_start[seq_of] * _BLOCK + (np.arange(self.max_tokens) - cu[:-1][seq_of])
        qsl = np.full(self.max_seqs + 1, self.max_tokens, dtype=np.int32)
        qsl[:B + 1] = cu
        sl = np.zeros(self.max_seqs, dtype=np.int32)
        sl[:B] = lens
        bt = np.zeros((self.max_seqs, self.max_blocks_per_seq), dtype=np.int32)
        for i, (s, n) in enumerate(zip(blk_start, nblk)):
            bt[i, :n] = np.arange(s, s + n)
        ts, tq = build_tile_worklist(lens.astype(np.int64), _BLOCK, lens.astype(np.int64))
        tile_seq = np.full(self.max_tiles, self.max_seqs - 1, dtype=np.int32)     # an empty slot
        tile_qoff = np.zeros(self.max_tiles, dtype=np.int32)
        tile_seq[:len(ts)], tile_qoff[:len(ts)] = ts, tq
        for dst, a in ((self.slots, slots), (self._qsl, qsl), (self._sl, sl), (self._bt, bt), (self._ts, tile_seq),
                       (self._tq, tile_qoff)):
            dst.copy_(torch.from_numpy(np.ascontiguousarray(a)).to(dst.dtype), non_blocking=True)
        self.cu_seqlens_cpu = qsl


def encoder_attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens,
                          scale: float) -> torch.Tensor:
    """fp32 definition: every token attends to all tokens of its own sequence."""
    out = torch.empty_like(q)
    cu = [int(x) for x in cu_seqlens]
    for a, b in zip(cu[:-1], cu[1:]):
        if b <= a:
            continue
        qs, ks, vs = (t[a:b].float().transpose(0, 1) for t in (q, k, v))      # [H, L, D]
        p = torch.softmax(qs @ ks.transpose(1, 2) * scale, dim=-1)
        out[a:b] = (p @ vs).transpose(0, 1).to(q.dtype)
    return out


def encoder_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, plan: EncoderAttnPlan,
                      scale: float) -> torch.Tensor:
    """q, k, v: [N, H, D] (same head count); returns [N, H, D]."""
    if not (q.is_cuda and q.dtype == torch.bfloat16):
        return encoder_attention_ref(q, k, v, plan.cu_seqlens_cpu, scale)
    from . import paged_attention_tc
    N, H, D = q.shape
    Dp = 64 if D <= 64 else 128
    if D > 128:
        raise RuntimeError("encoder_attention: head_dim above 128 is not supported by the kernel")
    if Dp != D:
        qp = q.new_zeros((N, H, Dp))
        qp[..., :D] = q
    else:
        qp = q.contiguous()
    kc = q.new_zeros((plan.num_blocks * _BLOCK, H, Dp))
    vc = q.new_zeros((plan.num_blocks * _BLOCK, H, Dp))
    if Dp != D:
        kc[plan.slots, :, :D] = k
        vc[plan.slots, :, :D] = v
    else:
        kc.index_copy_(0, plan.slots, k)
        vc.index_copy_(0, plan.slots, v)
    out = torch.empty_like(qp)
    paged_attention_tc(qp, kc.view(plan.num_blocks, _BLOCK, H, Dp), vc.view(plan.num_blocks, _BLOCK, H, Dp),
                       plan.meta, scale, out, causal=False)
    return out[..., :D] if Dp != D else out


def rope_table_ref(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    half = cos.shape[-1]
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:2 * half]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    out = xf.clone()
    out[..., :half] = x1 * c - x2 * s
    out[..., half:2 * half] = x2 * c + x1 * s
    return out.to(x.dtype)


def rope_table_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """In place on x [N, H, D] (last dim contiguous, head stride D): pair (e, e + half) of every
    head rotates by the angle whose cos / sin sit at [token, e] of the fp32 tables [N, half]."""
    N, H, D = x.shape
    half = cos.shape[-1]
    if not (x.is_cuda and x.dtype == torch.bfloat16):
        x.copy_(rope_table_ref(x, cos, sin))
        return x
    assert x.stride(2) == 1 and x.stride(1) == D and cos.is_contiguous() and sin.is_contiguous()
    rc = _native.lib().b200_rope_table(x.data_ptr(), x.stride(0), cos.data_ptr(), sin.data_ptr(), N, H, D,
                                      half, _native.stream_ptr())
    _native.check(rc, "rope_table")
    _native.launch_counter[0] += 1
    return x
