"""Vision tower of Qwen2.5-VL style multimodal models.

Patch embedding (the stride-equals-kernel Conv3d is one GEMM over flattened patches), a stack of
pre-norm blocks with 2-D rotary attention (windowed in most layers, per-frame full attention in
the rest) and a SwiGLU MLP, then the patch merger that folds spatial_merge_size^2 neighbouring
patches into one token of the language model's width.  Attention runs through
``ops.mm_encoder.encoder_attention`` (tcgen05 prefill kernel, causal masking off), GEMMs through
the bf16 GEMM kernels with their bias / residual epilogues.

Covers the reference's ViT path: vllm_ascend/ops/mm_encoder_attention.py (attention),
vllm_ascend/ops/conv.py (Conv3d as matmul), patch/worker/patch_qwen*_vl.py (window index and
rotary-position computation kept on the host).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, Optional

import numpy as np
import torch

from .. import ops
from ..ops import mm_encoder as enc
from .layers import Linear


@dataclass
class VisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    num_heads: int = 16
    intermediate_size: int = 3420
    out_hidden_size: int = 3584
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    in_channels: int = 3
    window_size: int = 112
    fullatt_block_indexes: list = field(default_factory=lambda: [7, 15, 23, 31])
    rms_norm_eps: float = 1e-6
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size ** 2

    @property
    def merge_unit(self) -> int:
        return self.spatial_merge_size ** 2

    @classmethod
    def from_hf(cls, d: dict) -> "VisionConfig":
        names = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in names})


# ---------------------------------------------------------------- host-side index math
def rot_pos_ids(grid_thw: np.ndarray, merge: int) -> np.ndarray:
    """[N, 2] (row, column) of every patch, patches ordered merge-group by merge-group."""
    out = []
    for t, h, w in grid_thw:
        hp = np.broadcast_to(np.arange(h)[:, None], (h, w))
        wp = np.broadcast_to(np.arange(w)[None, :], (h, w))

        def regroup(a):
            return a.reshape(h // merge, merge, w // merge, merge).transpose(0, 2, 1, 3).reshape(-1)
        ids = np.stack([regroup(hp), regroup(wp)], axis=-1)
        out.append(np.tile(ids, (t, 1)))
    return np.concatenate(out, axis=0)


def window_index(grid_thw: np.ndarray, window_size: int, merge: int, patch: int) -> tuple[np.ndarray, np.ndarray]:
    """Permutation of merged tokens that makes every attention window contiguous, and the
    cumulative PATCH counts of the windows (empty windows dropped)."""
    ws = window_size // merge // patch
    index, cu, base = [], [0], 0
    for t, h, w in grid_thw:
        lh, lw = h // merge, w // merge
        idx = np.arange(t * lh * lw).reshape(t, lh, lw)
        ph, pw = (-lh) % ws, (-lw) % ws
        padded = np.pad(idx, ((0, 0), (0, ph), (0, pw)), constant_values=-100)
        nh, nw = (lh + ph) // ws, (lw + pw) // ws
        padded = padded.reshape(t, nh, ws, nw, ws).transpose(0, 1, 3, 2, 4).reshape(t, nh * nw, ws, ws)
        seqlens = (padded != -100).sum(axis=(2, 3)).reshape(-1)
        flat = padded.reshape(-1)
        index.append(flat[flat != -100] + base)
        cu.extend((np.cumsum(seqlens) * merge * merge + cu[-1]).tolist())
        base += t * lh * lw
    cu = np.asarray(cu, dtype=np.int64)
    keep = np.concatenate([[True], np.diff(cu) != 0])
    return np.concatenate(index), cu[keep]


class VisionBlock:
    def __init__(self, cfg: VisionConfig, mk, idx: int):
        H, I = cfg.hidden_size, cfg.intermediate_size
        self.norm1 = mk.ones((H,))
        self.norm2 = mk.ones((H,))
        self.qkv = Linear(mk.normal((3 * H, H)), mk.zeros((3 * H,)), f"blocks.{idx}.attn.qkv")
        self.proj = Linear(mk.normal((H, H)), mk.zeros((H,)), f"blocks.{idx}.attn.proj")
        self.gate_up = Linear(mk.normal((2 * I, H)), mk.zeros((2 * I,)), f"blocks.{idx}.mlp.gate_up_proj")
        self.down = Linear(mk.normal((H, I)), mk.zeros((H,)), f"blocks.{idx}.mlp.down_proj")
        self.cfg = cfg

    def __call__(self, h: torch.Tensor, plan, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        N, nh, D = h.shape[0], cfg.num_heads, cfg.head_dim
        x, _ = ops.rms_norm(h, self.norm1, cfg.rms_norm_eps)
        qkv = self.qkv(x)
        qk = qkv[:, :2 * nh * D].view(N, 2 * nh, D)
        if qkv.is_cuda:
            enc.rope_table_(qkv.view(N, 3 * nh, D)[:, :2 * nh], cos, sin)
        else:
            qk.copy_(enc.rope_table_ref(qk, cos, sin))
        q, k, v = (qkv[:, i * nh * D:(i + 1) * nh * D].view(N, nh, D) for i in range(3))
        o = enc.encoder_attention(q, k, v, plan, D ** -0.5)
        h = self.proj(o.reshape(N, nh * D), residual=h)
        x, _ = ops.rms_norm(h, self.norm2, cfg.rms_norm_eps)
        return self.down(ops.silu_and_mul(self.gate_up(x)), residual=h)


class _Maker:
    def __init__(self, device, dtype, std, seed=1234):
        self.device, self.dtype, self.std = device, dtype, std
        self.gen = torch.Generator().manual_seed(seed)

    def normal(self, shape):
        return (torch.randn(shape, generator=self.gen) * self.std).to(self.dtype).to(self.device)

    def zeros(self, shape):
        return torch.zeros(shape, dtype=self.dtype, device=self.device)

    def ones(self, shape):
        return torch.ones(shape, dtype=self.dtype, device=self.device)


class VisionTransformer:
    """``forward(pixel_values [N, patch_dim], grid_thw [n_images, 3])`` -> [N / merge_unit, out_hidden]."""

    def __init__(self, cfg: VisionConfig, device, dtype=torch.bfloat16):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        mk = _Maker(self.device, dtype, cfg.init_std)
        self.patch_embed = Linear(mk.normal((cfg.hidden_size, cfg.patch_dim)), None, "patch_embed.proj")
        self.blocks = [VisionBlock(cfg, mk, i) for i in range(cfg.depth)]
        Hm = cfg.hidden_size * cfg.merge_unit
        self.merger_norm = mk.ones((cfg.hidden_size,))
        self.merger_fc1 = Linear(mk.normal((Hm, Hm)), mk.zeros((Hm,)), "merger.mlp.0")
        self.merger_fc2 = Linear(mk.normal((cfg.out_hidden_size, Hm)), mk.zeros((cfg.out_hidden_size,)),
                                 "merger.mlp.2")
        q = cfg.head_dim // 4
        self.inv_freq = 1.0 / (10000.0 ** (np.arange(0, q, dtype=np.float64) * 2 / (cfg.head_dim // 2)))

    # -- forward -------------------------------------------------------------
    def host_inputs(self, grid_thw) -> dict:
        """Index math of a batch of images (host): window permutation of the patches, rotary angle
        tables, the per-frame and per-window sequence boundaries."""
        cfg = self.cfg
        grid = np.asarray(grid_thw, dtype=np.int64).reshape(-1, 3)
        unit = cfg.merge_unit
        win_idx, cu_win = window_index(grid, cfg.window_size, cfg.spatial_merge_size, cfg.patch_size)
        pos = rot_pos_ids(grid, cfg.spatial_merge_size)                       # [N, 2]
        # window order: permute merge groups, keep the patches of a group together
        perm = (win_idx[:, None] * unit + np.arange(unit)[None, :]).reshape(-1)
        pos = pos[perm]
        ang = np.concatenate([pos[:, 0:1] * self.inv_freq[None], pos[:, 1:2] * self.inv_freq[None]], axis=1)
        cu_full = np.concatenate([[0], np.cumsum(np.repeat(grid[:, 1] * grid[:, 2], grid[:, 0]))])
        return dict(n=int(perm.shape[0]), perm=perm, inverse=np.argsort(win_idx), cos=np.cos(ang).astype(np.float32),
                    sin=np.sin(ang).astype(np.float32), cu_full=cu_full, cu_win=cu_win)

    def run(self, pixel_values: torch.Tensor, perm: torch.Tensor, inverse: torch.Tensor, cos: torch.Tensor,
            sin: torch.Tensor, plan_full, plan_win) -> torch.Tensor:
        """Device side of the tower (capturable: no host reads)."""
        cfg = self.cfg
        N, unit = pixel_values.shape[0], cfg.merge_unit
        h = self.patch_embed(pixel_values)
        h = h[perm]
        full = set(cfg.fullatt_block_indexes)
        for i, blk in enumerate(self.blocks):
            h = blk(h, plan_full if i in full else plan_win, cos, sin)
        x, _ = ops.rms_norm(h, self.merger_norm, cfg.rms_norm_eps)
        x = self.merger_fc1(x.view(N // unit, -1))
        x = ops.activation(x, "gelu")
        x = self.merger_fc2(x)
        return x[inverse]

    def forward(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        hi = self.host_inputs(grid_thw)
        assert pixel_values.shape[0] == hi["n"], "pixel_values rows must equal the patch count of grid_thw"
        dev = self.device
        return self.run(pixel_values.to(dev, self.dtype), torch.from_numpy(hi["perm"]).to(dev),
                        torch.from_numpy(hi["inverse"]).to(dev), torch.from_numpy(hi["cos"]).to(dev),
                        torch.from_numpy(hi["sin"]).to(dev), enc.make_plan(hi["cu_full"], dev),
                        enc.make_plan(hi["cu_win"], dev))

    __call__ = forward

    # -- parameters ------------------------------------------------------------
    def named_parameters(self):
        yield "patch_embed.proj.weight", self.patch_embed.weight
        for i, b in enumerate(self.blocks):
            p = f"blocks.{i}"
            yield f"{p}.norm1.weight", b.norm1
            yield f"{p}.norm2.weight", b.norm2
            for nm, lin in (("attn.qkv", b.qkv), ("attn.proj", b.proj), ("mlp.gate_up_proj", b.gate_up),
                            ("mlp.down_proj", b.down)):
                yield f"{p}.{nm}.weight", lin.weight
                yield f"{p}.{nm}.bias", lin.bias
        yield "merger.ln_q.weight", self.merger_norm
        for nm, lin in (("merger.mlp.0", self.merger_fc1), ("merger.mlp.2", self.merger_fc2)):
            yield f"{nm}.weight", lin.weight
            yield f"{nm}.bias", lin.bias

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        """HF names relative to the tower (``visual.`` prefix already stripped)."""
        params = dict(self.named_parameters())
        I = self.cfg.intermediate_size
        loaded = set()
        for name, w in weights:
            if name == "patch_embed.proj.weight":
                w = w.reshape(w.shape[0], -1)
            tgt, rows = name, None
            for hf, off in (("gate_proj", 0), ("up_proj", I)):
                if f".mlp.{hf}." in name:
                    tgt, rows = name.replace(hf, "gate_up_proj"), (off, off + I)
            if tgt not in params:
                continue
            dst = params[tgt] if rows is None else params[tgt][rows[0]:rows[1]]
            dst.copy_(w.to(dst.dtype))
            loaded.add(name)
        return loaded
