"""Encoder-cache transfer for disaggregated vision encoders (E | PD split).

An encoder instance runs only the vision tower and publishes each item's output under the
item's content hash; prefill / decode instances look the hash up instead of running the tower, and
fall back to computing locally when the lookup misses and the request carries pixels.  The store is
the same in-memory server the KV pool uses (``KVStoreServer``), keys are namespaced.  Role of the
upstream EC connector the reference plugs into its runner
(vllm_ascend/worker/model_runner_v1.py:1866-1869, examples/disaggregated_encoder).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..logger import logger
from .kv_transfer.side_channel import SideChannelError, request

_PREFIX = b"ec:"


class ECStoreConnector:
    def __init__(self, config: dict):
        extra = dict(config.get("ec_connector_extra_config") or {})
        self.store = (extra.get("store_host", "127.0.0.1"), int(extra["store_port"]))
        self.timeout_ms = int(extra.get("timeout_ms", 3000))
        self.role = config.get("ec_role", "ec_both")
        self.stats = {"saved": 0, "loaded": 0, "misses": 0, "failures": 0}

    @property
    def is_producer(self) -> bool:
        return self.role in ("ec_producer", "ec_both")

    @property
    def is_consumer(self) -> bool:
        return self.role in ("ec_consumer", "ec_both")

    def _ask(self, msg: dict) -> Optional[dict]:
        try:
            return request(*self.store, msg, self.timeout_ms)
        except SideChannelError as e:
            self.stats["failures"] += 1
            logger.warning("EC store: %s", e)
            return None

    def has(self, mm_hash: str) -> bool:
        rep = self._ask({"op": "exists", "hashes": [_PREFIX + mm_hash.encode()]})
        return bool(rep and rep.get("ok") and rep["mask"][0])

    def save(self, mm_hash: str, emb: torch.Tensor) -> None:
        if not self.is_producer:
            return
        a = emb.detach().float().cpu().numpy().astype(np.float32)
        head = np.asarray(a.shape, dtype=np.int64).tobytes()
        rep = self._ask({"op": "put", "hashes": [_PREFIX + mm_hash.encode()],
                         "payloads": [len(a.shape).to_bytes(1, "little") + head + a.tobytes()]})
        if rep and rep.get("ok"):
            self.stats["saved"] += 1

    def load(self, mm_hash: str, device, dtype) -> Optional[torch.Tensor]:
        if not self.is_consumer:
            return None
        rep = self._ask({"op": "get", "hashes": [_PREFIX + mm_hash.encode()]})
        if not rep or not rep.get("ok"):
            self.stats["misses"] += 1
            return None
        p = rep["payloads"][0]
        nd = p[0]
        shape = tuple(np.frombuffer(p[1:1 + 8 * nd], dtype=np.int64).tolist())
        a = np.frombuffer(p[1 + 8 * nd:], dtype=np.float32).reshape(shape)
        self.stats["loaded"] += 1
        return torch.from_numpy(a.copy()).to(device=device, dtype=dtype)


def create_ec_connector(config: Optional[dict]):
    if not config:
        return None
    name = config.get("ec_connector", "ECStoreConnector")
    if name not in ("ECStoreConnector", "ECSharedStorageConnector", "ECExampleConnector"):
        raise ValueError(f"unknown ec_connector {name!r}")
    return ECStoreConnector(config)
