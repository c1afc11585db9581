"""KV-cache housekeeping on the worker: zeroing of freshly allocated blocks, debug print.

``KVBlockZeroer`` clears whole blocks of every layer's cache in one launch (the reference's
``AscendKVBlockZeroer``, vllm_ascend/worker/utils.py:15-184): a block handed to a new
request must not expose the previous owner's values to masked positions, where 0 x NaN
would poison the attention output."""
from __future__ import annotations

from ctypes import c_int, c_long, c_void_p

import torch

from .. import _native

P, I, L = c_void_p, c_int, c_long
_native.register_signature("b200_zero_blocks", [P, I, P, I, L, L, P])
_native.register_signature("b200_device_print", [P, I, L, I, P])


class KVBlockZeroer:
    def __init__(self, kv_caches: list):
        self.tensors = [t for pair in kv_caches for t in pair]
        t0 = self.tensors[0]
        self.is_cuda = t0.is_cuda
        # dense storage of one block (HND caches are permuted views of dense storage)
        self.block_bytes = t0[0].numel() * t0.element_size()
        same = all(t[0].numel() * t.element_size() == self.block_bytes for t in self.tensors)
        self.groups = [self.tensors] if same else [[t] for t in self.tensors]
        if self.is_cuda:
            self.ptrs = [torch.tensor([t.data_ptr() for t in g], dtype=torch.int64, device=t0.device)
                         for g in self.groups]

    def zero(self, block_ids) -> None:
        if not len(block_ids):
            return
        if not self.is_cuda:
            idx = torch.as_tensor(list(block_ids), dtype=torch.long)
            for t in self.tensors:
                t[idx] = 0
            return
        dev = self.tensors[0].device
        blocks = torch.tensor(list(block_ids), dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        for g, ptrs in zip(self.groups, self.ptrs):
            bb = g[0][0].numel() * g[0].element_size()
            rc = _native.lib().b200_zero_blocks(ptrs.data_ptr(), len(g), blocks.data_ptr(), blocks.numel(), bb, bb,
                                                _native.stream_ptr())
            _native.check(rc, "zero_blocks")
            _native.count_launch()


def device_print(t: torch.Tensor, tag: int = 0, n: int = 8) -> None:
    """Print the first values of a tensor in stream order (works inside captured graphs)."""
    if not t.is_cuda:
        print(f"[device_print {tag}]", t.flatten()[:n].tolist())
        return
    flat = t.reshape(-1)
    dtype = {torch.float32: 0, torch.bfloat16: 1}.get(t.dtype)
    if dtype is None:
        flat, dtype = flat[:n].float(), 0
    _native.check(_native.lib().b200_device_print(flat.data_ptr(), dtype, min(n, flat.numel()), tag,
                                                  _native.stream_ptr()), "device_print")
