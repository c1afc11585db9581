"""Tagged sleep-mode memory pool on top of the native VMM allocator.

``VmmAllocator.get_instance().use_memory_pool(tag)`` routes every tensor allocated
inside the context through the native allocator (csrc/vmm_allocator.cu) with that
tag.  ``sleep(offload_tags)`` copies the allocations whose tag is in
``offload_tags`` to pinned host memory and releases the physical memory of ALL
pool allocations; ``wake_up(tags)`` maps new physical memory at the same virtual
addresses and restores the saved contents.  Same contract as ``CaMemAllocator``
(vllm_ascend/device_allocator/camem.py:113-305).
"""
from __future__ import annotations

import ctypes
from contextlib import contextmanager
from ctypes import c_char_p, c_int, c_uint64, c_void_p, POINTER
from dataclasses import dataclass
from typing import Iterable, Optional

import torch

from .. import _native

_TAG_STRIDE = 32


@dataclass
class AllocationInfo:
    ptr: int
    size: int
    mapped: bool
    tag: str


class NativeVmm:
    """Thin ctypes view of the C entry points (replaced by a fake in CPU tests)."""

    def __init__(self):
        lib = _native.lib()
        self.lib = lib
        lib.b200_vmm_available.restype = c_int
        lib.b200_vmm_set_tag.argtypes = [c_char_p]
        lib.b200_vmm_num_allocs.restype = c_int
        lib.b200_vmm_list.argtypes = [c_int, POINTER(c_uint64), POINTER(c_uint64), POINTER(c_int),
                                      ctypes.c_char_p, c_int]
        lib.b200_vmm_list.restype = c_int
        lib.b200_vmm_unmap_and_release.argtypes = [c_void_p]
        lib.b200_vmm_create_and_map.argtypes = [c_void_p]
        lib.b200_vmm_memcpy.argtypes = [c_void_p, c_void_p, c_uint64, c_int]
        lib.b200_vmm_last_error.restype = c_int

    def available(self) -> bool:
        return bool(self.lib.b200_vmm_available())

    def set_tag(self, tag: str) -> None:
        self.lib.b200_vmm_set_tag(tag.encode())

    def list(self) -> list[AllocationInfo]:
        n = self.lib.b200_vmm_num_allocs()
        if n == 0:
            return []
        ptrs = (c_uint64 * n)()
        sizes = (c_uint64 * n)()
        mapped = (c_int * n)()
        tags = ctypes.create_string_buffer(n * _TAG_STRIDE)
        k = self.lib.b200_vmm_list(n, ptrs, sizes, mapped, tags, _TAG_STRIDE)
        raw = tags.raw
        return [AllocationInfo(int(ptrs[i]), int(sizes[i]), bool(mapped[i]),
                               raw[i * _TAG_STRIDE:(i + 1) * _TAG_STRIDE].split(b"\0")[0].decode())
                for i in range(k)]

    def unmap_and_release(self, ptr: int) -> None:
        _native.check(self.lib.b200_vmm_unmap_and_release(ptr), "vmm unmap")

    def create_and_map(self, ptr: int) -> None:
        _native.check(self.lib.b200_vmm_create_and_map(ptr), "vmm map")

    def copy_to_host(self, host: torch.Tensor, ptr: int, nbytes: int) -> None:
        _native.check(self.lib.b200_vmm_memcpy(host.data_ptr(), ptr, nbytes, 1), "vmm d2h")

    def copy_to_device(self, ptr: int, host: torch.Tensor, nbytes: int) -> None:
        _native.check(self.lib.b200_vmm_memcpy(ptr, host.data_ptr(), nbytes, 0), "vmm h2d")

    def make_pool(self):
        alloc = torch.cuda.memory.CUDAPluggableAllocator(_native._LIB_PATH, "b200_vmm_malloc",
                                                         "b200_vmm_free")
        return alloc, torch.cuda.MemPool(alloc.allocator())


class VmmAllocator:
    _instance: Optional["VmmAllocator"] = None
    DEFAULT_TAG = "default"

    @classmethod
    def get_instance(cls) -> "VmmAllocator":
        if cls._instance is None:
            cls._instance = cls(NativeVmm())
        return cls._instance

    def __init__(self, backend):
        self.backend = backend
        self._pool = None
        self._alloc = None
        self._backups: dict[int, torch.Tensor] = {}
        self.current_tag = self.DEFAULT_TAG
        self.sleeping_tags: set[str] = set()

    # ------------------------------------------------------------------
    @contextmanager
    def use_memory_pool(self, tag: Optional[str] = None):
        tag = tag or self.DEFAULT_TAG
        if self._pool is None:
            self._alloc, self._pool = self.backend.make_pool()
        prev = self.current_tag
        self.current_tag = tag
        self.backend.set_tag(tag)
        try:
            with torch.cuda.use_mem_pool(self._pool):
                yield
        finally:
            self.current_tag = prev
            self.backend.set_tag(prev)

    def allocations(self, tags: Optional[Iterable[str]] = None) -> list[AllocationInfo]:
        out = self.backend.list()
        if tags is not None:
            tags = set(tags)
            out = [a for a in out if a.tag in tags]
        return out

    def get_current_usage(self) -> int:
        return sum(a.size for a in self.backend.list() if a.mapped)

    # ------------------------------------------------------------------
    def sleep(self, offload_tags: Optional[Iterable[str]] = None) -> int:
        """Release the physical memory of every pool allocation; allocations whose tag is in
        ``offload_tags`` are saved to pinned host memory first.  Returns bytes released."""
        if offload_tags is None:
            offload_tags = (self.DEFAULT_TAG,)
        elif isinstance(offload_tags, str):
            offload_tags = (offload_tags,)
        offload = set(offload_tags)
        freed = 0
        for a in self.backend.list():
            if not a.mapped:
                continue
            if a.tag in offload:
                host = torch.empty(a.size, dtype=torch.uint8, pin_memory=torch.cuda.is_available())
                self.backend.copy_to_host(host, a.ptr, a.size)
                self._backups[a.ptr] = host
            self.backend.unmap_and_release(a.ptr)
            self.sleeping_tags.add(a.tag)
            freed += a.size
        return freed

    def wake_up(self, tags: Optional[Iterable[str]] = None) -> int:
        """Map new physical memory at the old addresses; restore saved contents."""
        want = None if tags is None else set(tags)
        restored = 0
        for a in self.backend.list():
            if a.mapped or (want is not None and a.tag not in want):
                continue
            self.backend.create_and_map(a.ptr)
            host = self._backups.pop(a.ptr, None)
            if host is not None:
                self.backend.copy_to_device(a.ptr, host, a.size)
            restored += a.size
        if want is None:
            self.sleeping_tags.clear()
        else:
            self.sleeping_tags -= want
        return restored
