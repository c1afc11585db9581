"""CUDA-graph capture/replay cache keyed by batch descriptor.

Dispatch contract of vllm_ascend/compilation/acl_graph.py:133-267: a wrapper owns one
captured graph per ``BatchDescriptor``; at run time the descriptor of the current step
either matches an entry (replay) or the call falls through to the eager callable.  All
graphs of a process share one memory pool.  Unlike the reference there is no host-side
refresh of attention arguments before a replay (acl_graph.py:279-296): the attention
kernels read sequence lengths and block tables from persistent device buffers, so the
graph's arguments never change.
"""
from __future__ import annotations

import gc
from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch

_POOLS: dict = {}


def global_graph_pool():
    """One memory pool per device shared by every captured graph (the reference shares one pool
    the same way, acl_graph.py:60-75).  The caching allocator retires a pool once its last graph
    is destroyed and refuses the handle afterwards, so a one-kernel graph captured into the pool
    here stays alive for the life of the process."""
    dev = torch.cuda.current_device()
    ent = _POOLS.get(dev)
    if ent is None:
        handle = torch.cuda.graph_pool_handle()
        keep = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(keep, pool=handle):
            anchor = torch.zeros(8, device=f"cuda:{dev}")
        ent = _POOLS[dev] = (handle, keep, anchor)
    return ent[0]


@dataclass(frozen=True)
class BatchDescriptor:
    num_tokens: int
    uniform_decode: bool = True
    query_len: int = 1            # tokens per sequence (1 + speculative tokens)
    has_lora: bool = False


@dataclass
class GraphEntry:
    descriptor: BatchDescriptor
    graph: Optional["torch.cuda.CUDAGraph"] = None
    output: Any = None
    num_launches: int = 0         # this package's kernel launches recorded in the graph
    replays: int = 0
    input_addresses: Optional[list] = None


class CUDAGraphWrapper:
    """``mode`` is "FULL" (whole forward in one graph) or "PIECEWISE" (the callable is one
    piece between two opaque attention calls); a wrapper only acts when the runtime mode of
    the step equals its own mode."""

    def __init__(self, runnable: Callable, mode: str = "FULL", pool=None, debug_addresses: bool = False,
                 launch_counter: Optional[list] = None):
        self.runnable = runnable
        self.mode = mode
        self.pool = pool
        self.entries: dict[BatchDescriptor, GraphEntry] = {}
        self.debug_addresses = debug_addresses
        self.launch_counter = launch_counter

    def __contains__(self, desc: BatchDescriptor) -> bool:
        e = self.entries.get(desc)
        return e is not None and e.graph is not None

    def descriptors(self) -> list[BatchDescriptor]:
        return sorted(self.entries, key=lambda d: d.num_tokens)

    def capture(self, desc: BatchDescriptor, *args, warmup: Optional[Callable] = None, **kwargs) -> GraphEntry:
        """Warm up on a side stream, then record ``runnable(*args)`` into a graph.  Garbage
        collection is paused during capture: a collection that frees a tensor allocated from
        the graph pool mid-capture would corrupt the recording (acl_graph.py:186-199)."""
        if self.pool is None:
            self.pool = global_graph_pool()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            (warmup or self.runnable)(*args, **kwargs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        entry = GraphEntry(desc, torch.cuda.CUDAGraph())
        if self.debug_addresses:
            entry.input_addresses = [a.data_ptr() for a in args if isinstance(a, torch.Tensor)]
        c0 = self.launch_counter[0] if self.launch_counter is not None else 0
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(entry.graph, pool=self.pool):
                entry.output = self.runnable(*args, **kwargs)
        finally:
            if was_enabled:
                gc.enable()
        if self.launch_counter is not None:
            # kernels recorded into a graph run at replay time, not at capture time
            entry.num_launches = self.launch_counter[0] - c0
            self.launch_counter[0] = c0
        self.entries[desc] = entry
        return entry

    def replay(self, desc: BatchDescriptor, *args) -> Any:
        entry = self.entries[desc]
        if self.debug_addresses and entry.input_addresses is not None:
            now = [a.data_ptr() for a in args if isinstance(a, torch.Tensor)]
            if now != entry.input_addresses:
                raise RuntimeError(f"graph for {desc} replayed with different input addresses: "
                                   f"{now} vs {entry.input_addresses}")
        entry.graph.replay()
        entry.replays += 1
        return entry.output

    def __call__(self, desc: Optional[BatchDescriptor], runtime_mode: str, *args, **kwargs) -> Any:
        if desc is None or runtime_mode != self.mode or desc not in self:
            return self.runnable(*args, **kwargs)
        return self.replay(desc, *args)

    def clear(self) -> None:
        """Drop every captured graph (sleep mode releases their memory)."""
        self.entries.clear()
