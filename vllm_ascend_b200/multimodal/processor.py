"""Image / video -> patch rows for the vision tower (numpy, host side).

Layout contract of the Qwen2-VL family: the image is resized so both sides are multiples of
patch * merge, normalised, repeated to a multiple of temporal_patch frames, and cut into patches
ordered (frame group, merge-row, merge-col, row-in-merge, col-in-merge); each row holds
(channel, temporal, patch_h, patch_w) flattened, which is the Conv3d weight's own layout.
"""
from __future__ import annotations

import math

import numpy as np

CLIP_MEAN = np.array([0.48145466, 0.4578275, 0.40821073], dtype=np.float32)
CLIP_STD = np.array([0.26862954, 0.26130258, 0.27577711], dtype=np.float32)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280) -> tuple[int, int]:
    """Closest (h, w) divisible by ``factor`` with the pixel count inside [min, max], aspect kept."""
    if max(height, width) / max(1, min(height, width)) > 200:
        raise ValueError("aspect ratio above 200 is not supported")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def _resize_bilinear(img: np.ndarray, h: int, w: int) -> np.ndarray:
    """img [H, W, C] float32 -> [h, w, C] (align_corners=False)."""
    H, W, _ = img.shape
    if (H, W) == (h, w):
        return img
    ys = np.clip((np.arange(h) + 0.5) * H / h - 0.5, 0, H - 1)
    xs = np.clip((np.arange(w) + 0.5) * W / w - 0.5, 0, W - 1)
    y0, x0 = np.floor(ys).astype(int), np.floor(xs).astype(int)
    y1, x1 = np.minimum(y0 + 1, H - 1), np.minimum(x0 + 1, W - 1)
    wy, wx = (ys - y0)[:, None, None], (xs - x0)[None, :, None]
    top = img[y0][:, x0] * (1 - wx) + img[y0][:, x1] * wx
    bot = img[y1][:, x0] * (1 - wx) + img[y1][:, x1] * wx
    return top * (1 - wy) + bot * wy


def patchify(frames: np.ndarray, patch: int = 14, temporal_patch: int = 2, merge: int = 2,
             min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280,
             normalize: bool = True) -> tuple[np.ndarray, tuple[int, int, int]]:
    """frames: [H, W, 3] image or [T, H, W, 3] video, uint8 (0..255) or float (0..1).
    Returns (pixel_values [t * gh * gw, 3 * temporal_patch * patch * patch] float32, (t, gh, gw))."""
    x = np.asarray(frames)
    if x.ndim == 3:
        x = x[None]
    x = x.astype(np.float32) / (255.0 if frames.dtype == np.uint8 else 1.0)
    T, H, W, C = x.shape
    h, w = smart_resize(H, W, patch * merge, min_pixels, max_pixels)
    x = np.stack([_resize_bilinear(f, h, w) for f in x])
    if normalize:
        x = (x - CLIP_MEAN[:C]) / CLIP_STD[:C]
    if T % temporal_patch:
        x = np.concatenate([x, np.repeat(x[-1:], temporal_patch - T % temporal_patch, axis=0)])
    T = x.shape[0]
    t, gh, gw = T // temporal_patch, h // patch, w // patch
    x = x.transpose(0, 3, 1, 2)                                            # [T, C, h, w]
    x = x.reshape(t, temporal_patch, C, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)      # t, gh/m, gw/m, m, m, C, tp, p, p
    return np.ascontiguousarray(x.reshape(t * gh * gw, C * temporal_patch * patch * patch)), (t, gh, gw)
