"""Request-side multimodal bookkeeping: items, placeholder expansion, content hashes."""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch


@dataclass
class MMInput:
    modality: str                      # "image" | "video" | "audio" (grid_thw = (valid mel frames,), pixel_values = [mel, frames])
    offset: int                        # first placeholder token in the (expanded) prompt
    length: int                        # number of placeholder tokens = t * h * w / merge^2
    grid_thw: tuple
    pixel_values: Optional[torch.Tensor]   # [t*h*w, patch_dim]; None once the encoder output is cached
    hash: str = ""
    second_per_grid: Optional[float] = None
    embeds: Optional[torch.Tensor] = None  # rows supplied by the caller (prompt embeddings): no encoder run

    @property
    def end(self) -> int:
        return self.offset + self.length


def mm_hash(pixel_values, grid_thw) -> str:
    a = pixel_values.detach().cpu().numpy() if isinstance(pixel_values, torch.Tensor) else np.asarray(pixel_values)
    h = hashlib.sha256()
    h.update(np.asarray(grid_thw, dtype=np.int64).tobytes())
    h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()[:32]


def expand_placeholders(token_ids: Sequence[int], placeholder_id: int, lengths: Sequence[int]) -> tuple[list, list]:
    """Every occurrence of ``placeholder_id`` (one per item, in order) becomes ``lengths[i]`` copies.
    A prompt that already carries runs of the right length is left as it is.
    Returns (expanded ids, offsets of the runs)."""
    ids = list(token_ids)
    runs, i = [], 0
    while i < len(ids):
        if ids[i] == placeholder_id:
            j = i
            while j < len(ids) and ids[j] == placeholder_id:
                j += 1
            runs.append((i, j - i))
            i = j
        else:
            i += 1
    if len(runs) == len(lengths) and all(n == want for (_, n), want in zip(runs, lengths)):
        return ids, [o for o, _ in runs]
    singles = [k for k, t in enumerate(ids) if t == placeholder_id]
    if len(singles) != len(lengths):
        raise ValueError(f"{len(lengths)} multimodal items but {len(singles)} placeholder tokens in the prompt")
    out, offsets, nxt = [], [], 0
    for k, t in enumerate(ids):
        if t == placeholder_id:
            offsets.append(len(out))
            out.extend([placeholder_id] * lengths[nxt])
            nxt += 1
        else:
            out.append(t)
    return out, offsets


def build_mm_request(token_ids: Sequence[int], mm_data: dict, mcfg) -> tuple[list, list]:
    """``mm_data``: {"image": [...], "video": [...]}; every entry is an array of pixels
    ([H, W, 3] / [T, H, W, 3]) or an already patchified ``(pixel_values, grid_thw)`` pair.
    Returns (expanded prompt ids, MMInput list sorted by offset)."""
    ids = list(token_ids)
    items: list[MMInput] = []
    if mcfg.audio_config is not None and mm_data.get("audio") is not None:
        ids, items = _build_audio(ids, mm_data["audio"], mcfg)
    if mcfg.vision_config is None:
        return ids, items
    from ..models.vision import VisionConfig
    from .processor import patchify
    vc = VisionConfig.from_hf(mcfg.vision_config)
    m2 = vc.merge_unit
    for modality, tok in (("image", mcfg.image_token_id), ("video", mcfg.video_token_id)):
        entries = mm_data.get(modality) or []
        if not isinstance(entries, (list, tuple)):
            entries = [entries]
        if not entries:
            continue
        prepared = []
        for e in entries:
            if isinstance(e, dict):
                # produced elsewhere (disaggregated encoder): the hash names the cached output
                grid = tuple(int(x) for x in np.asarray(e["grid_thw"]).reshape(-1))
                pv = e.get("pixel_values")
                pv = None if pv is None else torch.as_tensor(pv)
                prepared.append((pv, grid, e.get("hash") or mm_hash(pv, grid)))
                continue
            if isinstance(e, (tuple, list)) and len(e) == 2:
                pv, grid = e
                pv = torch.as_tensor(np.asarray(pv) if not isinstance(pv, torch.Tensor) else pv)
                grid = tuple(int(x) for x in np.asarray(grid).reshape(-1))
            else:
                arr, grid = patchify(np.asarray(e), vc.patch_size, vc.temporal_patch_size, vc.spatial_merge_size)
                pv = torch.from_numpy(arr)
            prepared.append((pv, grid, mm_hash(pv, grid)))
        lengths = [g[0] * g[1] * g[2] // m2 for _, g, _ in prepared]
        ids, offsets = expand_placeholders(ids, tok, lengths)
        # earlier modalities' offsets move when this one expands
        for it in items:
            it.offset = -1
        for (pv, grid, hsh), off, n in zip(prepared, offsets, lengths):
            items.append(MMInput(modality, off, n, grid, pv, hsh,
                                 second_per_grid=(1.0 if modality == "video" else None)))
    # recompute offsets of items invalidated above
    if any(it.offset < 0 for it in items):
        for modality, tok in (("audio", mcfg.audio_token_id), ("image", mcfg.image_token_id),
                              ("video", mcfg.video_token_id)):
            group = [it for it in items if it.modality == modality]
            if group:
                _, offs = expand_placeholders(ids, tok, [it.length for it in group])
                for it, o in zip(group, offs):
                    it.offset = o
    items.sort(key=lambda m: m.offset)
    return ids, items


def _build_audio(ids: list, entries, mcfg) -> tuple[list, list]:
    """Audio entries: log-mel features [mel bins, frames] (all frames valid), a ``(features,
    valid_frames)`` pair for padded clips, or a dict with ``hash`` / ``valid_frames`` (and optionally
    ``features``) for outputs produced elsewhere."""
    from ..models.audio import audio_output_lengths
    if not isinstance(entries, (list, tuple)) or (len(entries) == 2 and isinstance(entries[1], (int, np.integer))):
        entries = [entries]
    prepared = []
    for e in entries:
        if isinstance(e, dict):
            f = e.get("features")
            f = None if f is None else torch.as_tensor(f)
            n = int(e["valid_frames"])
            prepared.append((f, n, e.get("hash") or mm_hash(f, (n,))))
            continue
        if isinstance(e, (tuple, list)) and len(e) == 2:
            f, n = torch.as_tensor(np.asarray(e[0]) if not isinstance(e[0], torch.Tensor) else e[0]), int(e[1])
        else:
            f = torch.as_tensor(np.asarray(e) if not isinstance(e, torch.Tensor) else e)
            n = int(f.shape[-1])
        prepared.append((f, n, mm_hash(f, (n,))))
    lengths = [int(audio_output_lengths(n)[1]) for _, n, _ in prepared]
    ids, offsets = expand_placeholders(ids, mcfg.audio_token_id, lengths)
    return ids, [MMInput("audio", off, ln, (n,), f, hsh) for (f, n, hsh), off, ln in zip(prepared, offsets, lengths)]
