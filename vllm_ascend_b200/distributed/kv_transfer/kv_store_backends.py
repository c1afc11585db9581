"""Storage backends of the shared KV pool.

The pool connector talks to a backend through four calls (``exists``, ``put``, ``get``, ``stats``)
on opaque keys (prefix hash, optionally suffixed with a layer index for layer-wise transfers) and
opaque byte payloads.  Backends are looked up by name in a registry so that a deployment can add
its own store without touching the connector:

    register_kv_store_backend("mystore", lambda extra: MyStore(**extra))
    kv_connector_extra_config = {"backend": "mystore", ...}

Built in:

* ``remote``: the in-tree store server (``KVStoreServer``) over the side channel, one store shared by
  every engine that knows its address (the default; ``store_host`` / ``store_port``);
* ``memory``: a process-local LRU store, shared by the engines of one process through ``name``
  (tests, single-process P/D);
* ``file``: one file per key under a directory on a shared filesystem (node-local NVMe, NFS, a
  parallel filesystem), written atomically (temp file + rename), capacity enforced by evicting the
  least recently used files.

The reference selects among its store clients the same way (vllm_ascend/distributed/kv_transfer/
kv_pool/ascend_store/backend/: a backend base class with mooncake, memcache and yuanrong
implementations chosen by ``backend`` in the connector's extra config).
"""
from __future__ import annotations

import hashlib
import os
import threading
import time
from collections import OrderedDict
from typing import Callable, Optional

from ...logger import logger
from .side_channel import SideChannelError, request


class KVStoreBackend:
    """Contract of a pool backend.  Keys and payloads are bytes."""

    def exists(self, keys: list[bytes]) -> Optional[list[bool]]:
        """Presence mask, or None when the store cannot be reached."""
        raise NotImplementedError

    def put(self, keys: list[bytes], payloads: list[bytes]) -> bool:
        raise NotImplementedError

    def get(self, keys: list[bytes]) -> Optional[list[bytes]]:
        """All payloads, or None if any key is missing (evicted between lookup and load)."""
        raise NotImplementedError

    def stats(self) -> dict:
        return {}

    def close(self) -> None:
        pass


class LRUBytes:
    """Byte-capacity LRU map used by the in-memory stores."""

    def __init__(self, capacity_bytes: int):
        self.capacity = capacity_bytes
        self.used = 0
        self.blocks: "OrderedDict[bytes, bytes]" = OrderedDict()
        self.lock = threading.Lock()
        self.counters = {"puts": 0, "gets": 0, "hits": 0, "evictions": 0}

    def exists(self, keys):
        with self.lock:
            return [k in self.blocks for k in keys]

    def put(self, keys, payloads) -> None:
        with self.lock:
            for k, payload in zip(keys, payloads):
                if k in self.blocks:
                    self.blocks.move_to_end(k)
                    continue
                while self.used + len(payload) > self.capacity and self.blocks:
                    _, old = self.blocks.popitem(last=False)
                    self.used -= len(old)
                    self.counters["evictions"] += 1
                if len(payload) <= self.capacity:
                    self.blocks[k] = payload
                    self.used += len(payload)
                    self.counters["puts"] += 1

    def get(self, keys):
        with self.lock:
            out = []
            for k in keys:
                p = self.blocks.get(k)
                if p is None:
                    return None
                self.blocks.move_to_end(k)
                out.append(p)
            self.counters["gets"] += 1
            self.counters["hits"] += len(out)
            return out

    def stats(self) -> dict:
        with self.lock:
            return {"used": self.used, "blocks": len(self.blocks), **self.counters}


class RemoteStoreBackend(KVStoreBackend):
    """Client of ``KVStoreServer``."""

    def __init__(self, host: str, port: int, timeout_ms: int = 3000):
        self.addr, self.timeout_ms = (host, int(port)), int(timeout_ms)
        self.failures = 0

    def _ask(self, msg: dict) -> Optional[dict]:
        try:
            return request(*self.addr, msg, self.timeout_ms)
        except SideChannelError as e:
            self.failures += 1
            logger.warning("KV pool: %s", e)
            return None

    def exists(self, keys):
        r = self._ask({"op": "exists", "hashes": keys})
        return None if r is None else r["mask"]

    def put(self, keys, payloads):
        return self._ask({"op": "put", "hashes": keys, "payloads": payloads}) is not None

    def get(self, keys):
        r = self._ask({"op": "get", "hashes": keys})
        return r["payloads"] if r is not None and r.get("ok") else None

    def stats(self):
        r = self._ask({"op": "stats"}) or {}
        return dict(r, client_failures=self.failures)


_MEMORY_STORES: dict[str, LRUBytes] = {}
_MEMORY_LOCK = threading.Lock()


class MemoryBackend(KVStoreBackend):
    """Process-local store; engines that name the same store share it."""

    def __init__(self, name: str = "default", capacity_bytes: int = 1 << 30):
        with _MEMORY_LOCK:
            self.store = _MEMORY_STORES.setdefault(name, LRUBytes(capacity_bytes))

    def exists(self, keys):
        return self.store.exists(keys)

    def put(self, keys, payloads):
        self.store.put(keys, payloads)
        return True

    def get(self, keys):
        return self.store.get(keys)

    def stats(self):
        return self.store.stats()


class FileBackend(KVStoreBackend):
    """One file per key under ``root`` (two-level fan-out by key digest).  Safe for several
    processes and hosts on a POSIX filesystem: a payload becomes visible by an atomic rename, a
    reader that loses a race with eviction reports the key as missing."""

    def __init__(self, root: str, capacity_bytes: int = 64 << 30, evict_batch: int = 64):
        self.root = root
        self.capacity = int(capacity_bytes)
        self.evict_batch = evict_batch
        os.makedirs(root, exist_ok=True)
        self.counters = {"puts": 0, "gets": 0, "hits": 0, "evictions": 0}
        self._lock = threading.Lock()
        self._approx_used: Optional[int] = None

    def _path(self, key: bytes) -> str:
        d = hashlib.blake2b(key, digest_size=20).hexdigest()
        return os.path.join(self.root, d[:2], d[2:4], d)

    def exists(self, keys):
        return [os.path.exists(self._path(k)) for k in keys]

    def _scan(self) -> list[tuple[float, int, str]]:
        out = []
        for dirpath, _, files in os.walk(self.root):
            for f in files:
                if f.endswith(".tmp"):
                    continue
                p = os.path.join(dirpath, f)
                try:
                    st = os.stat(p)
                    out.append((st.st_atime if st.st_atime > st.st_mtime else st.st_mtime, st.st_size, p))
                except OSError:
                    pass
        return out

    def _make_room(self, need: int) -> None:
        with self._lock:
            if self._approx_used is None:
                self._approx_used = sum(s for _, s, _ in self._scan())
            if self._approx_used + need <= self.capacity:
                self._approx_used += need
                return
            files = sorted(self._scan())
            used = sum(s for _, s, _ in files)
            for _, size, path in files:
                if used + need <= self.capacity:
                    break
                try:
                    os.remove(path)
                    used -= size
                    self.counters["evictions"] += 1
                except OSError:
                    pass
            self._approx_used = used + need

    def put(self, keys, payloads):
        for k, payload in zip(keys, payloads):
            path = self._path(k)
            if os.path.exists(path) or len(payload) > self.capacity:
                continue
            self._make_room(len(payload))
            os.makedirs(os.path.dirname(path), exist_ok=True)
            tmp = f"{path}.{os.getpid()}.{threading.get_ident()}.tmp"
            with open(tmp, "wb") as f:
                f.write(payload)
            os.replace(tmp, path)
            self.counters["puts"] += 1
        return True

    def get(self, keys):
        out = []
        now = time.time()
        for k in keys:
            path = self._path(k)
            try:
                with open(path, "rb") as f:
                    out.append(f.read())
                os.utime(path, (now, os.stat(path).st_mtime))      # recency for the eviction order
            except OSError:
                return None
        self.counters["gets"] += 1
        self.counters["hits"] += len(out)
        return out

    def stats(self):
        files = self._scan()
        return {"used": sum(s for _, s, _ in files), "blocks": len(files), **self.counters}


_BACKENDS: dict[str, Callable[[dict], KVStoreBackend]] = {}


def register_kv_store_backend(name: str, factory: Callable[[dict], KVStoreBackend]) -> None:
    """``factory(extra_config) -> backend``; a later registration of the same name replaces the earlier."""
    _BACKENDS[name] = factory


def create_kv_store_backend(extra: dict) -> KVStoreBackend:
    name = extra.get("backend", "remote")
    if name not in _BACKENDS:
        raise ValueError(f"unknown KV store backend {name!r}; registered: {sorted(_BACKENDS)}")
    return _BACKENDS[name](extra)


register_kv_store_backend("remote", lambda e: RemoteStoreBackend(e.get("store_host", "127.0.0.1"), int(e["store_port"]),
                                                                 int(e.get("timeout_ms", 3000))))
register_kv_store_backend("memory", lambda e: MemoryBackend(e.get("name", "default"),
                                                            int(e.get("capacity_bytes", 1 << 30))))
register_kv_store_backend("file", lambda e: FileBackend(e["path"], int(e.get("capacity_bytes", 64 << 30))))
