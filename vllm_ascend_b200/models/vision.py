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
    # Qwen3-VL tower: learned position table (bilinearly interpolated to the image grid), LayerNorm
    # blocks with a plain GELU MLP, no windows, extra "deepstack" mergers after the listed blocks
    num_position_embeddings: int = 0
    deepstack_visual_indexes: list = field(default_factory=list)

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


# ---------------------------------------------------------------- Qwen3-VL tower
def pos_embed_interpolation(grid_thw: np.ndarray, side: int, merge: int):
    """Bilinear sampling of a side x side position table on every image's h x w patch grid, in the
    merge-group patch order: (indices [4, N], weights [4, N])."""
    idx, wts = [[] for _ in range(4)], [[] for _ in range(4)]
    for t, h, w in grid_thw:
        hs = torch.linspace(0, side - 1, int(h))
        ws = torch.linspace(0, side - 1, int(w))
        hf, wf = hs.int(), ws.int()
        hc, wc = (hf + 1).clip(max=side - 1), (wf + 1).clip(max=side - 1)
        dh, dw = hs - hf, ws - wf
        combos = [(hf, wf, (1 - dh)[:, None] * (1 - dw)[None]), (hf, wc, (1 - dh)[:, None] * dw[None]),
                  (hc, wf, dh[:, None] * (1 - dw)[None]), (hc, wc, dh[:, None] * dw[None])]

        def regroup(a):          # [h, w] -> merge-group order, repeated over the t frame groups
            a = a.reshape(int(h) // merge, merge, int(w) // merge, merge).permute(0, 2, 1, 3).reshape(-1)
            return a.repeat(int(t))
        for k, (hi, wi, wt) in enumerate(combos):
            idx[k].append(regroup((hi[:, None] * side + wi[None]).long()))
            wts[k].append(regroup(wt))
    return torch.stack([torch.cat(x) for x in idx]), torch.stack([torch.cat(x) for x in wts])


class _LN:
    def __init__(self, mk, size, eps: float = 1e-6):
        self.weight, self.bias, self.eps = mk.ones((size,)), mk.zeros((size,)), eps

    def __call__(self, x):
        return ops.layer_norm(x, self.weight, self.bias, self.eps)


class Qwen3VisionBlock:
    def __init__(self, cfg: VisionConfig, mk, idx: int):
        H, I = cfg.hidden_size, cfg.intermediate_size
        self.cfg = cfg
        self.norm1, self.norm2 = _LN(mk, H), _LN(mk, H)
        self.qkv = Linear(mk.normal((3 * H, H)), mk.zeros((3 * H,)), f"blocks.{idx}.attn.qkv")
        self.proj = Linear(mk.normal((H, H)), mk.zeros((H,)), f"blocks.{idx}.attn.proj")
        self.fc1 = Linear(mk.normal((I, H)), mk.zeros((I,)), f"blocks.{idx}.mlp.linear_fc1")
        self.fc2 = Linear(mk.normal((H, I)), mk.zeros((H,)), f"blocks.{idx}.mlp.linear_fc2")

    def __call__(self, h, plan, cos, sin):
        cfg = self.cfg
        N, nh, D = h.shape[0], cfg.num_heads, cfg.head_dim
        qkv = self.qkv(self.norm1(h))
        qk = qkv[:, :2 * nh * D].view(N, 2 * nh, D)
        if qkv.is_cuda:
            enc.rope_table_(qkv.view(N, 3 * nh, D)[:, :2 * nh], cos, sin)
        else:
            qk.copy_(enc.rope_table_ref(qk, cos, sin))
        q, k, v = (qkv[:, i * nh * D:(i + 1) * nh * D].view(N, nh, D) for i in range(3))
        o = enc.encoder_attention(q, k, v, plan, D ** -0.5)
        h = self.proj(o.reshape(N, nh * D), residual=h)
        return self.fc2(ops.activation(self.fc1(self.norm2(h)).contiguous(), "gelu_tanh"), residual=h)


class _Qwen3Merger:
    def __init__(self, cfg: VisionConfig, mk, name: str, postshuffle: bool):
        Hm = cfg.hidden_size * cfg.merge_unit
        self.postshuffle, self.Hm = postshuffle, Hm
        self.norm = _LN(mk, Hm if postshuffle else cfg.hidden_size)
        self.fc1 = Linear(mk.normal((Hm, Hm)), mk.zeros((Hm,)), f"{name}.linear_fc1")
        self.fc2 = Linear(mk.normal((cfg.out_hidden_size, Hm)), mk.zeros((cfg.out_hidden_size,)), f"{name}.linear_fc2")

    def __call__(self, x):
        x = self.norm(x.view(-1, self.Hm)) if self.postshuffle else self.norm(x).view(-1, self.Hm)
        return self.fc2(ops.activation(self.fc1(x).contiguous(), "gelu"))


class Qwen3VisionTransformer:
    """``forward(pixel_values, grid_thw)`` -> [N / merge_unit, (1 + len(deepstack)) * out_hidden]: the merged
    image tokens followed, along the feature axis, by the deepstack features the decoder adds to the
    residual stream after its first layers."""

    def __init__(self, cfg: VisionConfig, device, dtype=torch.bfloat16):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        mk = _Maker(self.device, dtype, cfg.init_std)
        self.patch_embed = Linear(mk.normal((cfg.hidden_size, cfg.patch_dim)), mk.zeros((cfg.hidden_size,)),
                                  "patch_embed.proj")
        self.pos_embed = mk.normal((cfg.num_position_embeddings, cfg.hidden_size))
        self.side = int(round(cfg.num_position_embeddings ** 0.5))
        self.blocks = [Qwen3VisionBlock(cfg, mk, i) for i in range(cfg.depth)]
        self.merger = _Qwen3Merger(cfg, mk, "merger", False)
        self.deepstack = [_Qwen3Merger(cfg, mk, f"deepstack_merger_list.{i}", True)
                          for i in range(len(cfg.deepstack_visual_indexes))]
        q = cfg.head_dim // 4
        self.inv_freq = 1.0 / (10000.0 ** (np.arange(0, q, dtype=np.float64) * 2 / (cfg.head_dim // 2)))

    def forward(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        cfg = self.cfg
        grid = np.asarray(grid_thw, dtype=np.int64).reshape(-1, 3)
        dev = self.device
        idx, wts = pos_embed_interpolation(grid, self.side, cfg.spatial_merge_size)
        pos = (self.pos_embed[idx.to(dev)] * wts.to(dev, self.dtype).unsqueeze(-1)).sum(0)
        h = self.patch_embed(pixel_values.to(dev, self.dtype)) + pos
        ids = rot_pos_ids(grid, cfg.spatial_merge_size)
        ang = np.concatenate([ids[:, 0:1] * self.inv_freq[None], ids[:, 1:2] * self.inv_freq[None]], axis=1)
        cos = torch.from_numpy(np.cos(ang)).float().to(dev).contiguous()
        sin = torch.from_numpy(np.sin(ang)).float().to(dev).contiguous()
        cu = np.concatenate([[0], np.cumsum(np.repeat(grid[:, 1] * grid[:, 2], grid[:, 0]))])
        plan = enc.make_plan(cu, dev)
        feats = []
        for i, blk in enumerate(self.blocks):
            h = blk(h, plan, cos, sin)
            if i in cfg.deepstack_visual_indexes:
                feats.append(self.deepstack[cfg.deepstack_visual_indexes.index(i)](h))
        return torch.cat([self.merger(h)] + feats, dim=-1)

    __call__ = forward

    def named_parameters(self):
        yield "patch_embed.proj.weight", self.patch_embed.weight
        yield "patch_embed.proj.bias", self.patch_embed.bias
        yield "pos_embed.weight", self.pos_embed
        for i, b in enumerate(self.blocks):
            p = f"blocks.{i}"
            for nm, ln in (("norm1", b.norm1), ("norm2", b.norm2)):
                yield f"{p}.{nm}.weight", ln.weight
                yield f"{p}.{nm}.bias", ln.bias
            for nm, lin in (("attn.qkv", b.qkv), ("attn.proj", b.proj), ("mlp.linear_fc1", b.fc1), ("mlp.linear_fc2", b.fc2)):
                yield f"{p}.{nm}.weight", lin.weight
                yield f"{p}.{nm}.bias", lin.bias
        for nm, mg in [("merger", self.merger)] + [(f"deepstack_merger_list.{i}", m) for i, m in enumerate(self.deepstack)]:
            yield f"{nm}.norm.weight", mg.norm.weight
            yield f"{nm}.norm.bias", mg.norm.bias
            for sub, lin in (("linear_fc1", mg.fc1), ("linear_fc2", mg.fc2)):
                yield f"{nm}.{sub}.weight", lin.weight
                yield f"{nm}.{sub}.bias", lin.bias

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            if name == "patch_embed.proj.weight":
                w = w.reshape(w.shape[0], -1)
            if name in params:
                params[name].copy_(w.to(params[name].dtype))
                loaded.add(name)
        return loaded
