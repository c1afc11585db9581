"""3-axis rotary positions of a multimodal prompt.

Text tokens advance all three axes together.  The tokens of an image / video item form a
(t, h, w) grid after spatial merging: they share a start offset, the temporal axis advances per
frame group (scaled by seconds-per-grid * tokens-per-second for video), the height / width axes
follow the grid, and the text after the item resumes at max(position) + 1.  Decoded tokens continue
from ``len(prompt) + delta``.  Same contract as the get_rope_index logic the reference calls
through its runner (vllm_ascend/worker/model_runner_v1.py mrope paths; ops/rotary_embedding.py:582).
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np


def mrope_positions(token_ids: Sequence[int], items: Sequence, merge: int = 2,
                    tokens_per_second: float = 2.0) -> tuple[np.ndarray, int]:
    """items: MMInput-like objects with ``offset``, ``length``, ``grid_thw`` and
    ``second_per_grid`` (None for images), sorted by offset.
    Returns (int64 [3, len(token_ids)], delta)."""
    L = len(token_ids)
    out = np.zeros((3, L), dtype=np.int64)
    cur, nxt = 0, 0                       # token cursor, next free position
    for it in sorted(items, key=lambda m: m.offset):
        n_text = it.offset - cur
        if n_text < 0:
            raise ValueError("multimodal items overlap")
        out[:, cur:it.offset] = nxt + np.arange(n_text)
        nxt += n_text
        t, h, w = it.grid_thw
        gh, gw = h // merge, w // merge
        if t * gh * gw != it.length:
            raise ValueError(f"placeholder run of {it.length} tokens does not match grid {it.grid_thw}")
        spg = getattr(it, "second_per_grid", None)
        if spg is None:                                   # images: every frame group at the same time
            spg = 0.0 if getattr(it, "modality", "image") == "image" else 1.0
        t_idx = np.floor(np.arange(t, dtype=np.float64) * spg * tokens_per_second)
        tt = np.repeat(t_idx.astype(np.int64), gh * gw)
        hh = np.tile(np.repeat(np.arange(gh), gw), t)
        ww = np.tile(np.arange(gw), t * gh)
        seg = slice(it.offset, it.offset + it.length)
        out[0, seg], out[1, seg], out[2, seg] = tt + nxt, hh + nxt, ww + nxt
        nxt = int(out[:, seg].max()) + 1
        cur = it.offset + it.length
    out[:, cur:] = nxt + np.arange(L - cur)
    nxt += L - cur
    return out, int(nxt - L)
