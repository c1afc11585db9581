"""Weight transfer from a trainer to inference workers (RL loops).

``NCCLWeightTransferEngine``: trainer (rank 0 of a stateless group) broadcasts packed
buckets, every worker rank unpacks them into ``worker.update_weights`` — behaviour of
vllm_ascend/distributed/weight_transfer/hccl_engine.py:105-340.
``IPCWeightTransferEngine``: trainer and worker share a GPU or a node; the trainer exports
CUDA IPC handles of its tensors, the worker maps them and copies device-to-device —
npu_ipc_engine.py:112-426.
"""
from __future__ import annotations

import pickle
from typing import Callable, Iterable, Optional

import torch

from ..stateless_pg import StatelessGroup
from . import packed


class NCCLWeightTransferEngine:
    def __init__(self, host: str, port: int, rank: int, world_size: int, backend: Optional[str] = None,
                 bucket_bytes: int = 512 << 20, timeout_s: float = 300.0):
        self.group = StatelessGroup(host, port, rank, world_size, backend, timeout_s, prefix="wt")
        self.rank, self.bucket_bytes = rank, bucket_bytes
        self.version = 0
        self.stats = {"updates": 0, "bytes": 0, "buckets": 0}

    # trainer side -----------------------------------------------------------------
    def send_weights(self, named_tensors: Iterable[tuple[str, torch.Tensor]]) -> None:
        assert self.rank == 0, "only the trainer rank sends"
        tensors = dict(named_tensors)
        manifest = [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()]
        self.version += 1
        self.group.set(f"manifest/{self.version}", pickle.dumps([(n, str(d), s) for n, d, s in manifest]))
        for entries in packed.plan_buckets(manifest, self.bucket_bytes):
            buf = packed.pack(entries, tensors, self.group.device)
            self.group.broadcast(buf, 0)
            self.stats["bytes"] += buf.numel()
            self.stats["buckets"] += 1
        self.stats["updates"] += 1

    # worker side ------------------------------------------------------------------
    def receive_weights(self, apply: Callable[[Iterable[tuple[str, torch.Tensor]]], int]) -> int:
        """Blocks until the trainer's next ``send_weights``; ``apply`` gets (name, tensor)
        pairs bucket by bucket (e.g. ``worker.update_weights``).  Returns tensors applied."""
        self.version += 1
        raw = pickle.loads(self.group.get(f"manifest/{self.version}"))
        manifest = [(n, packed._dtype(d), tuple(s)) for n, d, s in raw]
        n = 0
        for entries in packed.plan_buckets(manifest, self.bucket_bytes):
            buf = torch.empty(packed.bucket_size(entries), dtype=torch.uint8, device=self.group.device)
            self.group.broadcast(buf, 0)
            n += apply(packed.unpack(entries, buf)) or 0
            self.stats["bytes"] += buf.numel()
            self.stats["buckets"] += 1
        self.stats["updates"] += 1
        return n

    def close(self) -> None:
        self.group.close()


class IPCWeightTransferEngine:
    """Same-node transfer through CUDA IPC: ``export`` on the trainer produces a picklable
    manifest (one handle per tensor), ``apply`` on the worker maps every handle and copies."""

    @staticmethod
    def export(named_tensors: Iterable[tuple[str, torch.Tensor]], allow_host: bool = False) -> bytes:
        from torch.multiprocessing.reductions import reduce_tensor
        out = []
        for name, t in named_tensors:
            if not t.is_cuda and not allow_host:
                raise ValueError(f"{name}: IPC transfer needs CUDA tensors")
            fn, args = reduce_tensor(t.detach())
            out.append((name, fn, args))
        return pickle.dumps(out)

    @staticmethod
    def apply(manifest: bytes, apply: Callable[[Iterable[tuple[str, torch.Tensor]]], int],
              device_index: Optional[int] = None) -> int:
        items = pickle.loads(manifest)

        def gen():
            for name, fn, args in items:
                a = list(args)
                if device_index is not None and len(a) > 6:
                    a[6] = device_index          # the importing process may number its GPUs differently
                yield name, fn(*a)
        n = apply(gen()) or 0
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        return n

    # ---- packed form: a few large buffers instead of one handle per tensor -------------------------
    @staticmethod
    def apply_packed(message: bytes, apply: Callable[[Iterable[tuple[str, torch.Tensor]]], int],
                     device_index: Optional[int] = None) -> tuple[int, int, bool]:
        """Worker side of ``PackedIPCSender``: maps the bucket named by ``message``, hands its tensors
        to ``apply`` (which must copy them: the buffer is reused after the acknowledgement) and returns
        (tensors applied, buffer index to acknowledge, last bucket of the update?)."""
        fn, args, entries, index, last = pickle.loads(message)
        a = list(args)
        if device_index is not None and len(a) > 6:
            a[6] = device_index
        buf = fn(*a)
        n = apply(packed.unpack(entries, buf)) or 0
        if buf.is_cuda:
            torch.cuda.synchronize()
        return n, index, last


class PackedIPCSender:
    """Trainer side of the packed same-node transfer.  Weights are copied into ``num_buffers``
    rotating byte buffers of ``bucket_bytes`` (tensors larger than a bucket get a buffer of their own
    size, made once); one message per bucket carries the buffer's IPC handle and the manifest of the
    tensors inside.  A buffer is refilled only after the worker acknowledged the bucket that used it,
    so packing of bucket i+1 overlaps the worker's copy of bucket i
    (vllm_ascend/distributed/weight_transfer/packed_tensor.py:201-325: producer / consumer over IPC
    handles with double buffering; npu_ipc_engine.py:375-426)."""

    def __init__(self, bucket_bytes: int = 256 << 20, device="cuda", num_buffers: int = 2):
        self.bucket_bytes, self.device, self.num_buffers = int(bucket_bytes), torch.device(device), int(num_buffers)
        self._buffers: dict[tuple[int, int], torch.Tensor] = {}
        self.stats = {"updates": 0, "buckets": 0, "bytes": 0}

    def _buffer(self, index: int, nbytes: int) -> torch.Tensor:
        size = max(nbytes, self.bucket_bytes)
        b = self._buffers.get((index, size))
        if b is None:
            b = torch.empty(size, dtype=torch.uint8, device=self.device)
            if not b.is_cuda:
                b.share_memory_()
            self._buffers[(index, size)] = b
        return b

    def send(self, named_tensors: Iterable[tuple[str, torch.Tensor]], post: Callable[[bytes], None],
             wait_ack: Callable[[], int]) -> int:
        """``post(message)`` delivers one message to the worker; ``wait_ack()`` blocks for the next
        acknowledgement and returns the buffer index it frees.  Returns the number of buckets."""
        from torch.multiprocessing.reductions import reduce_tensor
        tensors = dict(named_tensors)
        manifest = [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()]
        plan = packed.plan_buckets(manifest, self.bucket_bytes)
        busy: set[int] = set()
        for i, entries in enumerate(plan):
            index = i % self.num_buffers
            while index in busy:
                busy.discard(wait_ack())
            size = packed.bucket_size(entries)
            buf = self._buffer(index, size)
            for e in entries:
                t = tensors[e.name].contiguous()
                buf[e.offset:e.offset + e.nbytes].copy_(t.reshape(-1).view(torch.uint8), non_blocking=True)
            if buf.is_cuda:
                torch.cuda.synchronize()
            fn, args = reduce_tensor(buf)
            post(pickle.dumps((fn, args, entries, index, i == len(plan) - 1)))
            busy.add(index)
            self.stats["buckets"] += 1
            self.stats["bytes"] += size
        while busy:
            busy.discard(wait_ack())
        self.stats["updates"] += 1
        return len(plan)
