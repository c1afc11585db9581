"""Multi-LoRA batching wrapper.

Holds, per engine step, which adapter slot every token uses, and applies the low-rank
deltas to a layer's output with the gather-matvec kernels: one-slot-per-token (bgmv) when
the step is decode-shaped, segment-based (sgmv) when tokens of a request are consecutive
(prefill).  Role of ``PunicaWrapperNPU`` (vllm_ascend/lora/punica_npu.py:14-470):
add_shrink / add_expand / add_lora_linear / add_lora_embedding / add_lora_logits.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from . import ops as lops


class PunicaWrapperB200:
    def __init__(self, max_num_batched_tokens: int, max_batches: int, device, max_loras: int = 8):
        self.device = torch.device(device)
        self.max_tokens = max_num_batched_tokens
        self.max_loras = max_loras
        # persistent so a captured graph reads the current step's slots
        self.token_slots = torch.full((max_num_batched_tokens,), -1, dtype=torch.int32, device=self.device)
        self._pinned = torch.full((max_num_batched_tokens,), -1, dtype=torch.int32)
        if self.device.type == "cuda":
            self._pinned = self._pinned.pin_memory()
        self.segments: Optional[lops.Segments] = None
        self.num_tokens = 0
        self.is_prefill = False
        self.any_active = False

    # ------------------------------------------------------------------ metadata
    def update_metadata(self, slots_per_request: Sequence[int], query_lens: Sequence[int],
                        padded_tokens: Optional[int] = None) -> None:
        """``slots_per_request[i]`` is the adapter slot (or -1) of request i which contributes
        ``query_lens[i]`` consecutive tokens."""
        q = np.asarray(query_lens, dtype=np.int32)
        s = np.asarray(slots_per_request, dtype=np.int32)
        T = int(q.sum())
        n = padded_tokens or T
        tok = np.repeat(s, q)
        buf = self._pinned.numpy()
        buf[:T] = tok
        buf[T:n] = -1
        self.token_slots[:n].copy_(self._pinned[:n], non_blocking=True)
        self.num_tokens = n
        self.any_active = bool((s >= 0).any())
        self.is_prefill = bool(q.max() > 1) if len(q) else False
        self.segments = None
        if self.is_prefill and self.any_active:
            starts = np.concatenate([[0], np.cumsum(q)[:-1]]).astype(np.int32)
            self.segments = lops.Segments(starts, q, s, self.device)

    # ------------------------------------------------------------------ primitive ops
    def add_shrink(self, x: torch.Tensor, a_stacked: torch.Tensor, scale: float) -> torch.Tensor:
        """x [T, K], a_stacked [slots, slices*r, K] -> v [T, slices*r] fp32."""
        if self.segments is not None and x.shape[0] == self.segments.num_tokens:
            return lops.sgmv_shrink(x, a_stacked, self.segments, scale)
        return lops.bgmv_shrink(x, a_stacked, self.token_slots[:x.shape[0]], scale)

    def add_expand(self, y: torch.Tensor, v: torch.Tensor, b_stacked: Sequence[torch.Tensor],
                   output_slices: Sequence[int], rank: int, offset_start: int = 0) -> torch.Tensor:
        """y[:, off_i : off_i + n_i] += B_i[slot] @ v[:, i*r:(i+1)*r] for every slice i."""
        off = offset_start
        use_seg = self.segments is not None and y.shape[0] == self.segments.num_tokens
        for i, (b, n) in enumerate(zip(b_stacked, output_slices)):
            if b is not None:
                if use_seg:
                    lops.sgmv_expand(v, b, self.segments, y, off, i * rank, add=True)
                else:
                    lops.bgmv_expand(v, b, self.token_slots[:y.shape[0]], y, off, i * rank, add=True)
            off += n
        return y

    # ------------------------------------------------------------------ layer-level ops
    def add_lora_linear(self, y: torch.Tensor, x: torch.Tensor, a_stacked: torch.Tensor,
                        b_stacked: Sequence[torch.Tensor], scale: float, output_slices: Sequence[int],
                        rank: int) -> torch.Tensor:
        if not self.any_active:
            return y
        y2 = y.view(-1, y.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        v = self.add_shrink(x2, a_stacked, scale)
        self.add_expand(y2, v, b_stacked, output_slices, rank)
        return y

    def add_lora_embedding(self, y: torch.Tensor, ids: torch.Tensor, a_embed: torch.Tensor,
                           b_stacked: torch.Tensor, rank: int) -> torch.Tensor:
        """Embedding LoRA: A is a per-slot table [slots, vocab, r]; the shrink is a lookup."""
        if not self.any_active:
            return y
        slots = self.token_slots[:ids.shape[0]]
        v = a_embed[slots.clamp(min=0).long(), ids.long()].float()
        v = torch.where((slots >= 0)[:, None], v, torch.zeros_like(v))
        lops.bgmv_expand(v.contiguous(), b_stacked, slots, y, 0, 0, add=True)
        return y

    def add_lora_logits(self, logits: torch.Tensor, hidden: torch.Tensor, a_stacked: torch.Tensor,
                        b_stacked: torch.Tensor, scale: float, slots: torch.Tensor) -> torch.Tensor:
        """LM-head LoRA on the sampled rows only (``slots`` per sampled row)."""
        if not self.any_active:
            return logits
        v = lops.bgmv_shrink(hidden, a_stacked, slots, scale)
        lg = logits if logits.dtype == hidden.dtype else logits.to(hidden.dtype)
        lops.bgmv_expand(v, b_stacked, slots, lg, 0, 0, add=True)
        if lg is not logits:
            logits.copy_(lg)
        return logits
