"""Sharded-state checkpoints: every rank saves exactly the tensors it holds (already sliced for its
TP / EP / PP position, quantized tensors as they are) and later loads them back by name without
touching the other ranks' shards or re-slicing.  Start-up from such a directory reads 1 / world of
the bytes per rank.  Same contract as the ``sharded_state`` load format and the
``save_sharded_state`` example of the reference (examples/save_sharded_state_310.py)."""
from __future__ import annotations

import glob
import os

import torch

PATTERN = "model-rank-{rank}-part-{part}.safetensors"


def save_sharded_state(model, path: str, rank: int, max_bytes: int = 5 << 30) -> list[str]:
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    files, part, cur, size = [], 0, {}, 0

    def flush():
        nonlocal part, cur, size
        if cur:
            f = os.path.join(path, PATTERN.format(rank=rank, part=part))
            save_file(cur, f)
            files.append(f)
            part, cur, size = part + 1, {}, 0
    for name, t in model.named_parameters():
        t = t.detach().contiguous().cpu()
        n = t.numel() * t.element_size()
        if cur and size + n > max_bytes:
            flush()
        cur[name] = t
        size += n
    flush()
    return files


class ShardedStateLoader:
    def __init__(self, path: str, rank: int):
        self.path, self.rank = path, rank

    def load(self, model) -> bool:
        from safetensors import safe_open
        files = sorted(glob.glob(os.path.join(self.path, PATTERN.format(rank=self.rank, part="*"))))
        if not files:
            raise FileNotFoundError(f"no sharded state of rank {self.rank} under {self.path}")
        params = dict(model.named_parameters())
        seen = set()
        for f in files:
            with safe_open(f, framework="pt", device="cpu") as sf:
                for k in sf.keys():
                    if k not in params:
                        raise KeyError(f"{f}: tensor {k} does not exist in this model / parallel layout")
                    t = sf.get_tensor(k)
                    if tuple(t.shape) != tuple(params[k].shape):
                        raise ValueError(f"{k}: saved shard {tuple(t.shape)} != local shard {tuple(params[k].shape)} "
                                         "(the state was saved with another parallel layout)")
                    params[k].copy_(t.to(params[k].dtype))
                    seen.add(k)
        missing = set(params) - seen
        if missing:
            raise KeyError(f"sharded state lacks {sorted(missing)[:5]} ...")
        if hasattr(model, "layers"):
            for L in model.layers:            # derived tensors follow the loaded values
                a = L.self_attn
                if hasattr(a, "process_weights_after_loading"):
                    a.process_weights_after_loading()
                if hasattr(L.mlp, "_gate_bf16"):
                    L.mlp._gate_bf16 = None
        return True
