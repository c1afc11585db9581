"""Device communicator: the collectives a model layer may call on its group.

NCCL (through ``torch.distributed``) carries everything that is not on a fused path; small
all-reduces go through the one-shot peer-memory kernel when the group has a symmetric
buffer.  Equivalent of vllm_ascend/distributed/device_communicators/npu_communicator.py:23-58
(which adds nothing over its base) and of the ctypes HCCL binding
(device_communicators/pyhccl.py:37-171), which NCCL-through-torch makes unnecessary.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..parallel.state import GroupCoordinator


class B200Communicator:
    ONESHOT_MAX_BYTES = 512 * 1024

    def __init__(self, group: GroupCoordinator, symm=None):
        self.group = group
        self.symm = symm                    # parallel.symm_mem.SymmetricMemory or None
        self.world_size = group.world_size
        self.rank = group.rank_in_group
        self._oneshot_off = None

    # the reference's manager reports no fault tolerance for all-to-all either
    supports_all2all_fault_tolerance = False

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return x
        if self.symm is not None and x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() \
                and x.numel() * 2 <= self.ONESHOT_MAX_BYTES and (x.numel() * 2) % 16 == 0:
            return self._oneshot(x)
        return self.group.all_reduce(x)

    def _oneshot(self, x: torch.Tensor) -> torch.Tensor:
        from .. import _native
        if self._oneshot_off is None:
            self._oneshot_off = self.symm.region(self.ONESHOT_MAX_BYTES)
        stage = self.symm.tensor(self._oneshot_off, (x.numel(),), torch.bfloat16)
        stage.copy_(x.view(-1))
        out = torch.empty_like(x)
        ptrs = self.symm.ptr_array(self._oneshot_off)
        _native.check(_native.lib().b200_allreduce_oneshot(
            ptrs, self.symm.ctl_ptrs, out.data_ptr(), x.numel(), self.rank, self.world_size,
            _native.stream_ptr()), "allreduce_oneshot")
        return out

    def all_gather(self, x: torch.Tensor, dim: int = 0) -> torch.Tensor:
        return self.group.all_gather(x, dim)

    def reduce_scatter(self, x: torch.Tensor, dim: int = 0) -> torch.Tensor:
        return self.group.reduce_scatter(x, dim)

    def all_to_all_single(self, x: torch.Tensor, out_splits: Optional[list] = None,
                          in_splits: Optional[list] = None) -> torch.Tensor:
        if self.world_size == 1:
            return x
        n_out = sum(out_splits) if out_splits is not None else x.shape[0]
        out = x.new_empty((n_out,) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=self.group.device_group)
        return out

    def broadcast(self, x: torch.Tensor, src: int = 0) -> torch.Tensor:
        return self.group.broadcast(x, src)

    def send(self, x: torch.Tensor, dst: int) -> None:
        dist.send(x, self.group.ranks[dst], group=self.group.device_group)

    def recv(self, shape, dtype, src: int, device) -> torch.Tensor:
        t = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(t, self.group.ranks[src], group=self.group.device_group)
        return t

    def destroy(self) -> None:
        if self.symm is not None:
            self.symm.close()
            self.symm = None
