"""Shared KV pool: a prefix-keyed block store outside the engines.

Any engine (prefill or decode instance, any replica) publishes the full KV blocks of finished
requests under their prefix hashes and looks blocks up before prefilling, so a prefix computed
once is reused across the fleet.  ``KVStoreServer`` is the store (LRU by bytes) with a lookup
endpoint; ``KVPoolConnector`` is the engine side.  Roles of the reference's store connector
(vllm_ascend/distributed/kv_transfer/kv_pool/ascend_store/: pool_scheduler.py lookup client,
pool_worker.py put/get, backend/* stores); the backend here is an in-memory server reached over
ZMQ, payloads are staged through pinned host memory.
"""
from __future__ import annotations

import threading
from collections import OrderedDict
from concurrent.futures import ThreadPoolExecutor
from typing import Optional

import numpy as np
import torch

from ...engine.block_pool import BlockPool
from ...logger import logger
from .base import ConnectorMetadata, KVConnectorBase
from .side_channel import SideChannelError, SideChannelServer, request


class KVStoreServer:
    def __init__(self, host: str = "127.0.0.1", port: int = 0, capacity_bytes: int = 1 << 30):
        self.capacity = capacity_bytes
        self.used = 0
        self.blocks: "OrderedDict[bytes, bytes]" = OrderedDict()
        self.lock = threading.Lock()
        self.stats = {"puts": 0, "gets": 0, "hits": 0, "evictions": 0}
        self.server = SideChannelServer(host, port, self._handle)
        self.port = self.server.port
        self.server.start()

    def _handle(self, msg: dict) -> dict:
        op = msg.get("op")
        with self.lock:
            if op == "exists":
                return {"ok": True, "mask": [h in self.blocks for h in msg["hashes"]]}
            if op == "put":
                for h, payload in zip(msg["hashes"], msg["payloads"]):
                    if h in self.blocks:
                        self.blocks.move_to_end(h)
                        continue
                    while self.used + len(payload) > self.capacity and self.blocks:
                        _, old = self.blocks.popitem(last=False)
                        self.used -= len(old)
                        self.stats["evictions"] += 1
                    if len(payload) <= self.capacity:
                        self.blocks[h] = payload
                        self.used += len(payload)
                        self.stats["puts"] += 1
                return {"ok": True}
            if op == "get":
                out = []
                for h in msg["hashes"]:
                    p = self.blocks.get(h)
                    if p is None:
                        return {"ok": False, "error": "block evicted"}
                    self.blocks.move_to_end(h)
                    out.append(p)
                self.stats["gets"] += 1
                self.stats["hits"] += len(out)
                return {"ok": True, "payloads": out}
            if op == "stats":
                return {"ok": True, "used": self.used, "blocks": len(self.blocks), **self.stats}
        return {"ok": False, "error": f"unknown op {op!r}"}

    def close(self) -> None:
        self.server.stop()


class KVPoolConnector(KVConnectorBase):
    def __init__(self, engine_cfg, runner):
        ktc = dict(engine_cfg.kv_transfer_config or {})
        extra = dict(ktc.get("kv_connector_extra_config") or {})
        self.store = (extra.get("store_host", "127.0.0.1"), int(extra["store_port"]))
        self.timeout_ms = int(extra.get("timeout_ms", 3000))
        self.block_size = engine_cfg.cache.block_size
        self.tensors = [t for pair in runner.kv_caches for t in pair]
        self._fingerprint = BlockPool.store_fingerprint(engine_cfg, self.tensors)
        self.is_cuda = self.tensors[0].is_cuda
        self.role = ktc.get("kv_role", "kv_both")
        self._pending_load: list[tuple[list, list]] = []        # (hashes, gpu blocks)
        self._pool = ThreadPoolExecutor(max_workers=2, thread_name_prefix="kv-pool")
        self._puts: list = []
        self.stats = {"published_blocks": 0, "loaded_blocks": 0, "hit_tokens": 0, "lookup_failures": 0}

    # ------------------------------------------------------------------ helpers
    def _hashes(self, req, num_tokens: int) -> list[bytes]:
        toks = np.concatenate([req.prompt_token_ids, np.asarray(req.output_token_ids or [], dtype=np.int32)])
        extra = BlockPool.request_key_extra(req, self._fingerprint)
        if extra is None:               # nothing of this request may be looked up or published
            return []
        out, parent = [], None
        for i in range(num_tokens // self.block_size):
            parent = BlockPool.hash_block(parent, toks[i * self.block_size:(i + 1) * self.block_size], extra)
            out.append(parent)
        return out

    def _ask(self, msg: dict) -> Optional[dict]:
        try:
            return request(*self.store, msg, self.timeout_ms)
        except SideChannelError as e:
            self.stats["lookup_failures"] += 1
            logger.warning("KV pool: %s", e)
            return None

    def _serialize(self, block: int) -> bytes:
        return b"".join(t[block].contiguous().view(torch.uint8).cpu().numpy().tobytes() for t in self.tensors)

    def _deserialize(self, payload: bytes, block: int) -> None:
        off = 0
        for t in self.tensors:
            n = t[block].numel() * t.element_size()
            src = torch.frombuffer(bytearray(payload[off:off + n]), dtype=torch.uint8).view(t.dtype).view(t[block].shape)
            t[block].copy_(src.to(t.device, non_blocking=False))
            off += n

    # ------------------------------------------------------------------ scheduler side
    def get_num_new_matched_tokens(self, req, num_computed_tokens: int) -> tuple[int, bool]:
        if self.role == "kv_producer":
            return 0, False
        hashes = self._hashes(req, req.num_prompt_tokens - 1)[num_computed_tokens // self.block_size:]
        if not hashes:
            return 0, False
        r = self._ask({"op": "exists", "hashes": hashes})
        if r is None:
            return 0, False
        n = 0
        for hit in r["mask"]:
            if not hit:
                break
            n += 1
        return n * self.block_size, False

    def update_state_after_alloc(self, req, block_ids: list, num_external_tokens: int) -> None:
        if num_external_tokens <= 0:
            return
        first = req.num_cached_tokens // self.block_size
        n = num_external_tokens // self.block_size
        hashes = self._hashes(req, (first + n) * self.block_size)[first:first + n]
        self._pending_load.append((hashes, list(block_ids[first:first + n])))
        self.stats["hit_tokens"] += num_external_tokens

    def build_connector_meta(self, scheduler_output) -> ConnectorMetadata:
        return ConnectorMetadata(reqs_to_recv={i: j for i, j in enumerate(self._pending_load)})

    def request_finished(self, req, block_ids: list) -> tuple[bool, Optional[dict]]:
        if self.role == "kv_consumer":
            return False, None
        n_full = min(req.num_computed_tokens, req.num_tokens) // self.block_size
        if n_full == 0 or not block_ids:
            return False, None
        hashes = self._hashes(req, n_full * self.block_size)
        r = self._ask({"op": "exists", "hashes": hashes})
        if r is None:
            return False, None
        todo = [(h, b) for h, b, hit in zip(hashes, block_ids, r["mask"]) if not hit]
        if not todo:
            return False, None
        if self.is_cuda:
            torch.cuda.current_stream().synchronize()       # the blocks' last writes are complete
        # serialise now (the blocks go back to the pool right after), publish in the background
        payloads = [self._serialize(b) for _, b in todo]
        self._puts.append(self._pool.submit(self._ask, {"op": "put", "hashes": [h for h, _ in todo],
                                                        "payloads": payloads}))
        self.stats["published_blocks"] += len(todo)
        return False, None

    # ------------------------------------------------------------------ worker side
    def start_load_kv(self, scheduler_output) -> None:
        jobs, self._pending_load = self._pending_load, []
        for hashes, blocks in jobs:
            r = self._ask({"op": "get", "hashes": hashes})
            if r is None:
                raise RuntimeError("KV pool lost blocks between lookup and load")
            for payload, b in zip(r["payloads"], blocks):
                self._deserialize(payload, b)
            self.stats["loaded_blocks"] += len(blocks)

    def flush(self) -> None:
        for f in self._puts:
            f.result()
        self._puts = []

    def step_finished(self, scheduler_output, scheduler) -> None:
        self._puts = [f for f in self._puts if not f.done()]

    def close(self) -> None:
        self.flush()
        self._pool.shutdown(wait=True)
