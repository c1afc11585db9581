"""Packing of many named tensors into a few large transfer buckets.

Thousands of small broadcasts are launch-latency bound; weights are therefore copied into
flat byte buckets of a fixed size (tensors larger than a bucket travel alone) together with
a manifest of (name, dtype, shape, offset), the packed-tensor scheme of
vllm_ascend/distributed/weight_transfer (packed tensor chunking)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Iterator

import torch

_ALIGN = 256


@dataclass
class Entry:
    name: str
    dtype: str
    shape: tuple
    offset: int
    nbytes: int


def _dtype(name: str) -> torch.dtype:
    return getattr(torch, name.replace("torch.", ""))


def plan_buckets(meta: Iterable[tuple[str, torch.dtype, tuple]], bucket_bytes: int) -> list[list[Entry]]:
    """Greedy in-order packing; both sides derive the same plan from the same manifest."""
    buckets, cur, off = [], [], 0
    for name, dtype, shape in meta:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if cur and off + nbytes > bucket_bytes:
            buckets.append(cur)
            cur, off = [], 0
        cur.append(Entry(name, str(dtype), tuple(shape), off, nbytes))
        off += (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
    if cur:
        buckets.append(cur)
    return buckets


def bucket_size(entries: list[Entry]) -> int:
    last = entries[-1]
    return (last.offset + last.nbytes + _ALIGN - 1) // _ALIGN * _ALIGN


def pack(entries: list[Entry], tensors: dict, device) -> torch.Tensor:
    buf = torch.empty(bucket_size(entries), dtype=torch.uint8, device=device)
    for e in entries:
        t = tensors[e.name].contiguous()
        buf[e.offset:e.offset + e.nbytes].copy_(t.view(-1).view(torch.uint8) if t.numel() else t.view(torch.uint8))
    return buf


def unpack(entries: list[Entry], buf: torch.Tensor) -> Iterator[tuple[str, torch.Tensor]]:
    for e in entries:
        yield e.name, buf[e.offset:e.offset + e.nbytes].view(_dtype(e.dtype)).view(e.shape)
