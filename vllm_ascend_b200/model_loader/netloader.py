"""Weight loading from a running instance instead of from storage.

A serving instance exposes a small control endpoint; a starting instance with the same
architecture and parallel layout asks it for a transfer, both join a two-rank stateless
group (NCCL between GPUs, gloo on CPU) and the weights stream across in packed buckets
straight into the new model's parameters.  Any failure falls back to the default loader.
Role of vllm_ascend/model_loader/netloader/* (P2P weight pull over the device interconnect).
"""
from __future__ import annotations

import socket
import threading
from typing import Optional

import torch

from ..distributed.kv_transfer.side_channel import SideChannelError, SideChannelServer, request
from ..distributed.stateless_pg import StatelessGroup
from ..distributed.weight_transfer import packed
from ..logger import logger


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _manifest(model) -> list:
    return [(n, str(t.dtype), tuple(t.shape)) for n, t in model.named_parameters()]


class WeightSource:
    """Control endpoint of a running instance (one per rank, at ``port + tp_rank``)."""

    def __init__(self, model, host: str = "127.0.0.1", port: int = 0, tp_rank: int = 0, tp_size: int = 1,
                 model_id: str = "", bucket_bytes: int = 256 << 20, backend: Optional[str] = None):
        self.model, self.host, self.tp_rank, self.tp_size = model, host, tp_rank, tp_size
        self.model_id, self.bucket_bytes, self.backend = model_id, bucket_bytes, backend
        self.active = 0
        self.served = 0
        self.server = SideChannelServer(host, port + tp_rank if port else 0, self._handle)
        self.port = self.server.port
        self.server.start()

    def _handle(self, msg: dict) -> dict:
        op = msg.get("op")
        if op == "info":
            return {"ok": True, "model_id": self.model_id, "tp_rank": self.tp_rank, "tp_size": self.tp_size,
                    "active": self.active, "manifest": [[n, d, list(s)] for n, d, s in _manifest(self.model)]}
        if op == "pull":
            if int(msg.get("tp_size", 1)) != self.tp_size or int(msg.get("tp_rank", 0)) != self.tp_rank:
                return {"ok": False, "error": "parallel layout differs"}
            t = threading.Thread(target=self._send, args=(msg["host"], int(msg["port"])), daemon=True)
            self.active += 1
            t.start()
            return {"ok": True}
        return {"ok": False, "error": f"unknown op {op!r}"}

    def _send(self, host: str, port: int) -> None:
        try:
            dev = next(iter(self.model.named_parameters()))[1].device
            if dev.type == "cuda":
                torch.cuda.set_device(dev)
            g = StatelessGroup(host, port, 1, 2, self.backend or ("nccl" if dev.type == "cuda" else "gloo"),
                               timeout_s=60, prefix="netloader")
            tensors = dict(self.model.named_parameters())
            meta = [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()]
            for entries in packed.plan_buckets(meta, self.bucket_bytes):
                g.send(packed.pack(entries, tensors, g.device), 0)
            g.barrier()
            g.close()
            self.served += 1
        except Exception as e:
            logger.warning("weight transfer to %s:%s failed: %s", host, port, e)
        finally:
            self.active -= 1

    def close(self) -> None:
        self.server.stop()


class NetLoader:
    def __init__(self, source_host: str, source_port: int, tp_rank: int = 0, tp_size: int = 1,
                 listen_host: str = "127.0.0.1", bucket_bytes: int = 256 << 20, backend: Optional[str] = None,
                 timeout_ms: int = 5000):
        self.src = (source_host, source_port + tp_rank)
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.listen_host, self.bucket_bytes, self.backend, self.timeout_ms = listen_host, bucket_bytes, backend, timeout_ms

    def load(self, model) -> bool:
        """True when every parameter was received; False means "use the default loader"."""
        try:
            info = request(*self.src, {"op": "info"}, self.timeout_ms)
            mine = _manifest(model)
            theirs = [(n, d, tuple(s)) for n, d, s in info["manifest"]]
            if mine != theirs:
                raise SideChannelError("the source holds a different set of parameters")
            port = _free_port()
            params = dict(model.named_parameters())
            dev = next(iter(params.values())).device
            result: dict = {}

            def recv():
                try:
                    g = StatelessGroup(self.listen_host, port, 0, 2,
                                       self.backend or ("nccl" if dev.type == "cuda" else "gloo"),
                                       timeout_s=60, prefix="netloader")
                    meta = [(n, t.dtype, tuple(t.shape)) for n, t in params.items()]
                    for entries in packed.plan_buckets(meta, self.bucket_bytes):
                        buf = torch.empty(packed.bucket_size(entries), dtype=torch.uint8, device=g.device)
                        g.recv(buf, 1)
                        for name, t in packed.unpack(entries, buf):
                            params[name].copy_(t)
                    g.barrier()
                    g.close()
                    result["ok"] = True
                except Exception as e:          # reported by the caller
                    result["error"] = e
            # the store master (rank 0) must be listening before the source connects
            th = threading.Thread(target=recv, daemon=True)
            th.start()
            request(*self.src, {"op": "pull", "host": self.listen_host, "port": port, "tp_rank": self.tp_rank,
                                "tp_size": self.tp_size}, self.timeout_ms)
            th.join(timeout=600)
            if "error" in result or not result.get("ok"):
                raise SideChannelError(f"transfer failed: {result.get('error', 'timed out')}")
            if hasattr(model, "process_weights_after_loading"):
                model.process_weights_after_loading()
            return True
        except Exception as e:
            logger.warning("netloader: %s; falling back to the default loader", e)
            return False
