"""Weight offloading with prefetch: some decoder layers keep their linear weights in pinned host
memory and stream them into a small ring of device buffers a few layers ahead of use, on a copy
stream, so models larger than HBM (or a larger KV cache) fit at the cost of PCIe traffic.

Layers ``i`` with ``i % group_size < num_in_group`` are offloaded; ``prefetch_step`` layers are in
flight ahead of the one computing.  Role of the reference's prefetch offloader
(vllm_ascend/model_executor/offloader/prefetch.py:83-201).  Steps run eagerly while offloading is
on (the weights' device addresses rotate, which a captured graph could not follow).
"""
from __future__ import annotations

from typing import Optional

import torch


def _layer_linears(layer) -> list:
    out = []
    a = layer.self_attn
    for name in ("qkv_proj", "o_proj", "q_proj", "q_a_proj", "q_b_proj", "kv_a_proj", "kv_b_proj"):
        lin = getattr(a, name, None)
        if lin is not None and getattr(lin, "quant", None) is None:
            out.append(lin)
    m = layer.mlp
    for name in ("gate_up_proj", "down_proj"):
        lin = getattr(m, name, None)
        if lin is not None and getattr(lin, "quant", None) is None:
            out.append(lin)
    return out


class PrefetchOffloader:
    def __init__(self, model, group_size: int, num_in_group: int, prefetch_step: int = 1):
        if group_size < 1 or not (0 < num_in_group <= group_size) or prefetch_step < 1:
            raise ValueError("need group_size >= 1, 0 < num_in_group <= group_size, prefetch_step >= 1")
        self.model = model
        self.device = model.device
        self.is_cuda = self.device.type == "cuda"
        self.layers = [L for i, L in enumerate(model.layers) if i % group_size < num_in_group]
        self.order = {id(L): k for k, L in enumerate(self.layers)}
        self.linears = [_layer_linears(L) for L in self.layers]
        self.host: list[list[torch.Tensor]] = []
        self.bytes_offloaded = 0
        for lins in self.linears:
            hs = []
            for lin in lins:
                h = torch.empty(lin.weight.shape, dtype=lin.weight.dtype, pin_memory=self.is_cuda)
                h.copy_(lin.weight)
                hs.append(h)
                self.bytes_offloaded += h.numel() * h.element_size()
            self.host.append(hs)
        # ring of device slots, each as large as the biggest offloaded layer
        self.num_slots = min(len(self.layers), prefetch_step + 1)
        per_layer = [sum(h.numel() * h.element_size() for h in hs) for hs in self.host]
        self.slot_bytes = (max(per_layer) + 255) // 256 * 256 if per_layer else 0
        self.slots = [torch.empty(self.slot_bytes, dtype=torch.uint8, device=self.device)
                      for _ in range(self.num_slots)]
        self.ready = [None] * len(self.layers)        # event: weights of layer k are in its slot
        self.freed = [None] * self.num_slots          # event: slot no longer read by compute
        self.copy_stream = torch.cuda.Stream(device=self.device) if self.is_cuda else None
        self.prefetch_step = prefetch_step
        self.stats = {"prefetches": 0, "bytes": 0}
        for lins in self.linears:                     # release the resident copies
            for lin in lins:
                lin.weight = torch.empty(0, dtype=lin.weight.dtype, device=self.device)
        self._install()

    # ------------------------------------------------------------------
    def _views(self, k: int) -> list[torch.Tensor]:
        slot = self.slots[k % self.num_slots]
        out, off = [], 0
        for h in self.host[k]:
            n = h.numel() * h.element_size()
            out.append(slot[off:off + n].view(h.dtype).view(h.shape))
            off += n
        return out

    def _prefetch(self, k: int) -> None:
        if k >= len(self.layers):
            return
        s = k % self.num_slots
        views = self._views(k)
        if self.is_cuda:
            if self.freed[s] is not None:
                self.copy_stream.wait_event(self.freed[s])
            with torch.cuda.stream(self.copy_stream):
                for v, h in zip(views, self.host[k]):
                    v.copy_(h, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
            self.ready[k] = ev
        else:
            for v, h in zip(views, self.host[k]):
                v.copy_(h)
        self.stats["prefetches"] += 1
        self.stats["bytes"] += sum(h.numel() * h.element_size() for h in self.host[k])

    def begin_step(self) -> None:
        for k in range(min(self.prefetch_step, len(self.layers))):
            self._prefetch(k)

    def _before(self, k: int) -> None:
        if self.is_cuda and self.ready[k] is not None:
            torch.cuda.current_stream().wait_event(self.ready[k])
        for lin, v in zip(self.linears[k], self._views(k)):
            lin.weight = v

    def _after(self, k: int) -> None:
        if self.is_cuda:
            ev = torch.cuda.Event()
            ev.record()
            self.freed[k % self.num_slots] = ev
        self._prefetch(k + self.prefetch_step)

    def _install(self) -> None:
        off = self
        for k, layer in enumerate(self.layers):
            cls = type(layer)

            def wrapped(h, residual, meta, kv_cache, _k=k, _layer=layer, _cls=cls):
                off._before(_k)
                out = _cls.__call__(_layer, h, residual, meta, kv_cache)
                off._after(_k)
                return out
            layer.offloaded_call = wrapped
        fwd = self.model.forward
        model = self.model

        def forward(input_ids, meta, kv_caches, intermediate=None):
            off.begin_step()
            return fwd(input_ids, meta, kv_caches, intermediate)
        model.forward = forward
