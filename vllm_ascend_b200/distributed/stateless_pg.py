"""Process groups that exist beside the job's own ``torch.distributed`` world.

A trainer and its inference workers, or a starting instance and the running instance it
pulls weights from, are separate jobs: they rendezvous through a TCP store of their own and
talk over a dedicated NCCL (GPU) or gloo (CPU) communicator.  Role of the "stateless"
process groups behind vllm_ascend/distributed/weight_transfer/hccl_engine.py:105-340 and
the netloader's send/recv (model_loader/netloader/*).
"""
from __future__ import annotations

import datetime
from typing import Optional

import torch
import torch.distributed as dist


class StatelessGroup:
    def __init__(self, host: str, port: int, rank: int, world_size: int, backend: Optional[str] = None,
                 timeout_s: float = 120.0, device: Optional[torch.device] = None, prefix: str = "b200"):
        self.rank, self.world_size = rank, world_size
        t = datetime.timedelta(seconds=timeout_s)
        self.store = dist.TCPStore(host, port, world_size, rank == 0, timeout=t, wait_for_workers=True)
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        self.backend = backend
        store = dist.PrefixStore(prefix, self.store)
        if backend == "nccl":
            self.device = device or torch.device("cuda", torch.cuda.current_device())
            opts = dist.ProcessGroupNCCL.Options()
            self.pg = dist.ProcessGroupNCCL(store, rank, world_size, opts)
        else:
            self.device = torch.device("cpu")
            self.pg = dist.ProcessGroupGloo(store, rank, world_size, t)

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        opts = dist.BroadcastOptions()
        opts.rootRank = src
        self.pg.broadcast([t], opts).wait()
        return t

    def send(self, t: torch.Tensor, dst: int, tag: int = 0) -> None:
        self.pg.send([t], dst, tag).wait()

    def recv(self, t: torch.Tensor, src: int, tag: int = 0) -> torch.Tensor:
        self.pg.recv([t], src, tag).wait()
        return t

    def barrier(self) -> None:
        self.pg.barrier().wait()

    def set(self, key: str, value: bytes) -> None:
        self.store.set(key, value)

    def get(self, key: str) -> bytes:
        return self.store.get(key)

    def close(self) -> None:
        self.pg = None
        self.store = None
