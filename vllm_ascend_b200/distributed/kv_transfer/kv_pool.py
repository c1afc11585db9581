"""Shared KV pool: a prefix-keyed block store outside the engines.

Any engine (prefill or decode instance, any replica) publishes the full KV blocks of finished
requests under their prefix hashes and looks blocks up before prefilling, so a prefix computed
once is reused across the fleet.  ``KVStoreServer`` is the store (LRU by bytes) with a lookup
endpoint; ``KVPoolConnector`` is the engine side.  Roles of the reference's store connector
(vllm_ascend/distributed/kv_transfer/kv_pool/ascend_store/: pool_scheduler.py lookup client,
pool_worker.py put/get, backend/* stores).  Where the blocks live is a backend chosen by name
(``kv_store_backends``: the in-tree server, a process-local store, a directory on a shared
filesystem, or one a deployment registers).  With ``layerwise: true`` a block travels as one
payload per layer under ``<prefix hash>/L<layer>`` keys, so that stores see smaller objects, pipeline
stages publish only the layers they hold, and a load can proceed layer by layer.
"""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from typing import Optional

import numpy as np
import torch

from ...engine.block_pool import BlockPool
from ...logger import logger
from .base import ConnectorMetadata, KVConnectorBase
from .kv_store_backends import LRUBytes, create_kv_store_backend
from .side_channel import SideChannelServer


class KVStoreServer:
    """The in-tree store: a byte-capacity LRU map behind the side-channel protocol."""

    def __init__(self, host: str = "127.0.0.1", port: int = 0, capacity_bytes: int = 1 << 30):
        self.lru = LRUBytes(capacity_bytes)
        self.server = SideChannelServer(host, port, self._handle)
        self.port = self.server.port
        self.server.start()

    @property
    def stats(self) -> dict:
        return self.lru.counters

    @property
    def blocks(self):
        return self.lru.blocks

    @property
    def used(self) -> int:
        return self.lru.used

    def _handle(self, msg: dict) -> dict:
        op = msg.get("op")
        if op == "exists":
            return {"ok": True, "mask": self.lru.exists(msg["hashes"])}
        if op == "put":
            self.lru.put(msg["hashes"], msg["payloads"])
            return {"ok": True}
        if op == "get":
            out = self.lru.get(msg["hashes"])
            if out is None:
                return {"ok": False, "error": "block evicted"}
            return {"ok": True, "payloads": out}
        if op == "stats":
            return {"ok": True, **self.lru.stats()}
        return {"ok": False, "error": f"unknown op {op!r}"}

    def close(self) -> None:
        self.server.stop()


class KVPoolConnector(KVConnectorBase):
    def __init__(self, engine_cfg, runner):
        ktc = dict(engine_cfg.kv_transfer_config or {})
        extra = dict(ktc.get("kv_connector_extra_config") or {})
        self.backend = create_kv_store_backend(extra)
        self.layerwise = bool(extra.get("layerwise", False))
        self.block_size = engine_cfg.cache.block_size
        self.tensors = [t for pair in runner.kv_caches for t in pair]
        # tensors of one layer travel together in layer-wise mode
        self.layers = [[t for t in pair] for pair in runner.kv_caches]
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

    def _keys(self, hashes: list[bytes]) -> list[bytes]:
        """Store keys of the given blocks: the hash itself, or one key per (block, layer)."""
        if not self.layerwise:
            return list(hashes)
        return [h + b"/L%d" % li for h in hashes for li in range(len(self.layers))]

    def _exists(self, hashes: list[bytes]) -> Optional[list[bool]]:
        """Per block: is it (every layer of it) in the store?"""
        mask = self.backend.exists(self._keys(hashes))
        if mask is None:
            self.stats["lookup_failures"] += 1
            return None
        if not self.layerwise:
            return mask
        n = len(self.layers)
        return [all(mask[i * n:(i + 1) * n]) for i in range(len(hashes))]

    @staticmethod
    def _pack(tensors, block: int) -> bytes:
        return b"".join(t[block].contiguous().view(torch.uint8).cpu().numpy().tobytes() for t in tensors)

    @staticmethod
    def _unpack(tensors, payload: bytes, block: int) -> None:
        off = 0
        for t in tensors:
            n = t[block].numel() * t.element_size()
            src = torch.frombuffer(bytearray(payload[off:off + n]), dtype=torch.uint8).view(t.dtype).view(t[block].shape)
            t[block].copy_(src.to(t.device, non_blocking=False))
            off += n

    def _serialize(self, block: int) -> list[bytes]:
        """Payloads of one block in key order."""
        if not self.layerwise:
            return [self._pack(self.tensors, block)]
        return [self._pack(layer, block) for layer in self.layers]

    def _deserialize(self, payloads: list[bytes], block: int) -> None:
        if not self.layerwise:
            self._unpack(self.tensors, payloads[0], block)
            return
        for layer, payload in zip(self.layers, payloads):
            self._unpack(layer, payload, block)

    # ------------------------------------------------------------------ scheduler side
    def get_num_new_matched_tokens(self, req, num_computed_tokens: int) -> tuple[int, bool]:
        if self.role == "kv_producer":
            return 0, False
        hashes = self._hashes(req, req.num_prompt_tokens - 1)[num_computed_tokens // self.block_size:]
        if not hashes:
            return 0, False
        mask = self._exists(hashes)
        if mask is None:
            return 0, False
        n = 0
        for hit in mask:
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
        mask = self._exists(hashes)
        if mask is None:
            return False, None
        todo = [(h, b) for h, b, hit in zip(hashes, block_ids, mask) if not hit]
        if not todo:
            return False, None
        if self.is_cuda:
            torch.cuda.current_stream().synchronize()       # the blocks' last writes are complete
        # serialise now (the blocks go back to the pool right after), publish in the background
        payloads = [p for _, b in todo for p in self._serialize(b)]
        self._puts.append(self._pool.submit(self.backend.put, self._keys([h for h, _ in todo]), payloads))
        self.stats["published_blocks"] += len(todo)
        return False, None

    # ------------------------------------------------------------------ worker side
    def start_load_kv(self, scheduler_output) -> None:
        jobs, self._pending_load = self._pending_load, []
        for hashes, blocks in jobs:
            payloads = self.backend.get(self._keys(hashes))
            if payloads is None:
                raise RuntimeError("KV pool lost blocks between lookup and load")
            per = len(self.layers) if self.layerwise else 1
            for i, b in enumerate(blocks):
                self._deserialize(payloads[i * per:(i + 1) * per], b)
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
        self.backend.close()
