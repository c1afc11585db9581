"""CUDA-graph capture of the vision tower for bucketed patch counts.

A ViT forward over a small image is a few hundred short kernels; replaying one graph per bucket
removes the launch overhead the same way decode graphs do.  Inputs live in static buffers: pixel
rows padded to the bucket, the window permutation, rotary tables and two static attention plans
(per-frame and per-window sequences); padding rows form one extra sequence whose outputs are
dropped.  Counterpart of the reference's encoder graph manager (vllm_ascend/worker/encoder_acl_graph.py).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..ops.mm_encoder import StaticEncoderPlan
from .cuda_graph import global_graph_pool


class _Bucket:
    def __init__(self, tower, n: int):
        cfg, dev = tower.cfg, tower.device
        self.n = n
        half = cfg.head_dim // 2
        self.px = torch.zeros((n, cfg.patch_dim), dtype=tower.dtype, device=dev)
        self.perm = torch.arange(n, dtype=torch.int64, device=dev)
        self.inverse = torch.arange(n // cfg.merge_unit, dtype=torch.int64, device=dev)
        self.cos = torch.ones((n, half), dtype=torch.float32, device=dev)
        self.sin = torch.zeros((n, half), dtype=torch.float32, device=dev)
        # full windows hold 64 patches; batches of many tiny windows run eagerly instead
        self.max_seqs = max_seqs = n // 16 + 8
        self.plan_full = StaticEncoderPlan(n, max_seqs, dev)
        self.plan_win = StaticEncoderPlan(n, max_seqs, dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.out: Optional[torch.Tensor] = None

    def load(self, tower, px: torch.Tensor, hi: dict) -> None:
        n_real, n, unit = hi["n"], self.n, tower.cfg.merge_unit
        pad = np.arange(n_real, n)
        self.px[:n_real].copy_(px, non_blocking=True)
        up = lambda dst, a: dst.copy_(torch.from_numpy(np.ascontiguousarray(a)).to(dst.dtype), non_blocking=True)  # noqa: E731
        up(self.perm, np.concatenate([hi["perm"], pad]))
        up(self.inverse, np.concatenate([hi["inverse"], np.arange(n_real // unit, n // unit)]))
        up(self.cos[:n_real], hi["cos"])
        up(self.sin[:n_real], hi["sin"])
        tail = [n] if n > n_real else []
        self.plan_full.update(np.concatenate([hi["cu_full"], tail]))
        self.plan_win.update(np.concatenate([hi["cu_win"], tail]))


class EncoderGraphManager:
    def __init__(self, tower, bucket_sizes=(256, 1024, 4096)):
        unit = tower.cfg.merge_unit
        self.tower = tower
        self.sizes = sorted({max(unit, (int(b) + unit - 1) // unit * unit) for b in bucket_sizes})
        self.buckets: dict[int, _Bucket] = {}
        self.stats = {"captures": 0, "replays": 0, "eager": 0}

    def _bucket_for(self, n: int) -> Optional[int]:
        for b in self.sizes:
            if n <= b:
                return b
        return None

    def _run(self, bk: _Bucket) -> torch.Tensor:
        return self.tower.run(bk.px, bk.perm, bk.inverse, bk.cos, bk.sin, bk.plan_full, bk.plan_win)

    @torch.inference_mode()
    def run(self, px: torch.Tensor, grid_thw) -> torch.Tensor:
        tower = self.tower
        hi = tower.host_inputs(grid_thw)
        n = hi["n"]
        size = self._bucket_for(n)
        bk = self.buckets.get(size) if size is not None else None
        if size is not None and bk is None:
            bk = self.buckets[size] = _Bucket(tower, size)
        # a sequence list longer than the static plan holds (many tiny windows) runs eagerly
        if bk is None or max(len(hi["cu_win"]), len(hi["cu_full"])) + 1 > bk.max_seqs - 1:
            self.stats["eager"] += 1
            return tower(px, grid_thw)
        bk.load(tower, px.to(tower.device, tower.dtype), hi)
        if bk.graph is None:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._run(bk)                       # warm-up outside capture
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            bk.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(bk.graph, pool=global_graph_pool()):
                bk.out = self._run(bk)
            self.stats["captures"] += 1
        bk.graph.replay()
        self.stats["replays"] += 1
        return bk.out[:n // tower.cfg.merge_unit].clone()
