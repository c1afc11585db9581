"""Symmetric (peer-mapped) device memory for one process group.

Every rank allocates one buffer of the same size with the native allocator,
exports it as a CUDA IPC handle, and maps all peers' buffers, so kernels can
load/store any rank's copy through NVLink.  The buffer starts with the control
block (epoch flags, see csrc/comm.cuh); the rest is carved into named regions at
identical offsets on every rank.

This layer replaces the HCCL "window" the reference's device-initiated ops use as
peer memory (csrc/mc2/*/op_kernel/utils/hccl_shmem.hpp; buffer sizing in
vllm_ascend/ops/fused_moe/moe_comm_method.py:283-336).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_long, c_void_p, POINTER
from typing import Optional

import torch

from .. import _native
from .state import GroupCoordinator

P, I, L, F = c_void_p, c_int, c_long, ctypes.c_float
_native.register_signature("b200_symm_alloc", [L, POINTER(c_void_p)])
_native.register_signature("b200_symm_free", [P])
_native.register_signature("b200_ipc_get_handle", [P, P])
_native.register_signature("b200_ipc_open", [P, POINTER(c_void_p)])
_native.register_signature("b200_ipc_close", [P])
_native.register_signature("b200_comm_ctl_bytes", [])
_native.register_signature("b200_comm_barrier", [P, I, I, P])
_native.register_signature("b200_comm_ctl_reset", [P, P])
_native.register_signature("b200_comm_read_status", [P, POINTER(c_int), P])
_native.register_signature("b200_allreduce_oneshot", [P, P, P, L, I, I, P])
_native.register_signature("b200_reduce_add_norm_push", [P, I, P, P, P, F, P, P, I, I, I, I, I, P])
_native.register_signature("b200_reduce_add_norm_push_mc", [P, I, P, P, P, F, P, P, I, I, I, I, I, P, P])
_native.register_signature("b200_nvls_reduce_add_norm_push", [P, I, P, P, P, F, P, P, I, I, I, I, I, P])
_native.register_signature("b200_gemm_pub_bf16", [P, P, P, P, I, I, I, I, I, I, P, I, I, I, P, P])
_native.register_signature("b200_gemm_pub_bf16_2cta", [P, P, P, P, I, I, I, I, I, I, P, I, I, P, P])
_native.register_signature("b200_ag_wait", [P, I, I, P])
_native.register_signature("b200_gemm_ag_bf16", [P, P, P, P, I, I, I, I, I, I, P, I, I, I, I, P, P])
_native.register_signature("b200_gemm_rs_bf16", [P, P, P, I, I, I, I, I, P, P, I, I, I, I, P, P])
_native.register_signature("b200_gemm_ag_bf16_2cta", [P, P, P, P, I, I, I, I, I, I, P, I, I, I, I, P, P])
_native.register_signature("b200_gemm_rs_bf16_2cta", [P, P, P, I, I, I, I, I, P, P, I, I, I, P, P])
_native.register_signature("b200_gemm_swiglu_bf16", [P, P, P, I, I, I, I, I, I, P, P])
_native.register_signature("b200_grouped_gemm_bf16", [P, P, P, P, I, L, I, I, I, I, I, I, P, P])


class _RawCudaBuffer:
    """Exposes a raw device pointer through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class SymmetricMemory:
    ALIGN = 1024

    def __init__(self, group: GroupCoordinator, device: torch.device, nbytes: int, multicast: bool = False):
        """``multicast``: ask for memory that is also bound to an NVSwitch multicast object, so that
        kernels can use ``multimem.ld_reduce`` / ``multimem.st`` on ``mc_ptr + offset`` (in-switch
        reduction and replication).  The allocation and the handle exchange are then done by
        ``torch.distributed._symmetric_memory`` (CUDA virtual memory + multicast binding); when that
        is not available the buffer falls back to CUDA IPC and ``mc_ptr`` is 0."""
        self.group = group
        self.device = device
        self.rank = group.rank_in_group
        self.world = group.world_size
        lib = _native.lib()
        self.ctl_bytes = ((lib.b200_comm_ctl_bytes() + self.ALIGN - 1) // self.ALIGN) * self.ALIGN
        self.nbytes = self.ctl_bytes + ((nbytes + self.ALIGN - 1) // self.ALIGN) * self.ALIGN
        self.mc_ptr = 0
        self._torch_buf = self._hdl = None
        self.peer_ptrs: list[int] = []
        if multicast:
            self._try_multicast()
        if not self.peer_ptrs:
            p = c_void_p()
            _native.check(lib.b200_symm_alloc(self.nbytes, ctypes.byref(p)), "symm_alloc")
            self.local_ptr = p.value
            handle = (ctypes.c_ubyte * 64)()
            _native.check(lib.b200_ipc_get_handle(self.local_ptr, handle), "ipc_get_handle")
            handles = group.all_gather_object(bytes(handle))
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.peer_ptrs.append(self.local_ptr)
                    continue
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                q = c_void_p()
                _native.check(lib.b200_ipc_open(buf, ctypes.byref(q)), f"ipc_open(rank {r})")
                self.peer_ptrs.append(q.value)
        self._offset = self.ctl_bytes
        self._keep = _RawCudaBuffer(self.local_ptr, self.nbytes)
        self.local = torch.as_tensor(self._keep, device=device)     # uint8 view of the whole buffer
        self.ctl_ptrs = (c_void_p * self.world)(*self.peer_ptrs)
        group.barrier()

    def _try_multicast(self) -> None:
        """Allocate through torch's symmetric-memory allocator; every rank must take the same
        branch, so the outcome is agreed on before any pointer is used."""
        ok, err = 1, ""
        try:
            import torch.distributed._symmetric_memory as tsm
            buf = tsm.empty(self.nbytes, dtype=torch.uint8, device=self.device)
            hdl = tsm.rendezvous(buf, self.group.device_group.group_name)
            mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
            if mc == 0:
                ok, err = 0, "no multicast pointer (NVSwitch multicast unsupported here)"
        except Exception as e:              # older torch, no fabric support, ...
            ok, err = 0, f"{type(e).__name__}: {e}"
        if min(self.group.all_gather_object(ok)) == 0:
            if err:
                from ..logger import logger
                logger.info("multicast symmetric memory unavailable (%s): using CUDA IPC peer memory", err[:200])
            return
        buf.zero_()
        torch.cuda.synchronize(self.device)
        self._torch_buf, self._hdl = buf, hdl
        self.local_ptr = int(buf.data_ptr())
        self.peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
        self.peer_ptrs[self.rank] = self.local_ptr
        self.mc_ptr = mc

    def region(self, nbytes: int) -> int:
        """Reserve a region; returns its byte offset (identical on every rank)."""
        off = self._offset
        self._offset += ((nbytes + self.ALIGN - 1) // self.ALIGN) * self.ALIGN
        if self._offset > self.nbytes:
            raise RuntimeError("symmetric buffer exhausted")
        return off

    def tensor(self, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        n = int(torch.tensor([], dtype=dtype).element_size())
        numel = 1
        for s in shape:
            numel *= s
        return self.local[offset:offset + numel * n].view(dtype).view(*shape)

    def ptr_array(self, offset: int):
        """ctypes array of every rank's pointer to the region at ``offset``."""
        return (c_void_p * self.world)(*[p + offset for p in self.peer_ptrs])

    def barrier(self) -> None:
        _native.check(_native.lib().b200_comm_barrier(self.ctl_ptrs, self.rank, self.world,
                                                      _native.stream_ptr()), "comm_barrier")

    def read_status(self) -> int:
        out = c_int(0)
        _native.check(_native.lib().b200_comm_read_status(self.local_ptr, ctypes.byref(out),
                                                          _native.stream_ptr()), "read_status")
        return out.value

    def close(self) -> None:
        lib = _native.lib()
        if self._torch_buf is not None:      # torch owns the mapping and the multicast binding
            self._torch_buf = self._hdl = None
            self.local_ptr = 0
            return
        for r, p in enumerate(self.peer_ptrs):
            if r != self.rank and p:
                lib.b200_ipc_close(p)
        if self.local_ptr:
            lib.b200_symm_free(self.local_ptr)
            self.local_ptr = 0
