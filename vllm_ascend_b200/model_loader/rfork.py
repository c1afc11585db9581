""""Fork" a new instance from running ones.

A planner keeps the list of live seed instances per model and layout; a starting instance
asks it for the least busy seed, pulls the weights from it (same transfer as the netloader),
reports back, and can register itself as a further seed, so capacity for scale-out grows
with the fleet.  Protocol roles of vllm_ascend/model_loader/rfork/* (seed, planner,
transfer engine); falls back to the default loader when no seed is available.
"""
from __future__ import annotations

import time
from typing import Optional

from ..distributed.kv_transfer.side_channel import SideChannelError, SideChannelServer, request
from ..logger import logger
from .netloader import NetLoader


class RForkPlanner:
    def __init__(self, host: str = "127.0.0.1", port: int = 0, seed_ttl_s: float = 30.0):
        self.seeds: dict[tuple, dict] = {}        # (model_id, tp_size, host, port) -> state
        self.ttl = seed_ttl_s
        self.server = SideChannelServer(host, port, self._handle)
        self.port = self.server.port
        self.server.start()

    def _live(self, model_id: str, tp_size: int) -> list[tuple]:
        now = time.monotonic()
        return [k for k, v in self.seeds.items()
                if k[0] == model_id and k[1] == tp_size and now - v["seen"] < self.ttl]

    def _handle(self, msg: dict) -> dict:
        op = msg.get("op")
        if op in ("register", "heartbeat"):
            k = (msg["model_id"], int(msg["tp_size"]), msg["host"], int(msg["port"]))
            st = self.seeds.setdefault(k, {"inflight": 0, "served": 0})
            st["seen"] = time.monotonic()
            return {"ok": True}
        if op == "unregister":
            self.seeds.pop((msg["model_id"], int(msg["tp_size"]), msg["host"], int(msg["port"])), None)
            return {"ok": True}
        if op == "acquire":
            live = self._live(msg["model_id"], int(msg["tp_size"]))
            if not live:
                return {"ok": False, "error": "no live seed for this model"}
            k = min(live, key=lambda k: (self.seeds[k]["inflight"], self.seeds[k]["served"]))
            self.seeds[k]["inflight"] += 1
            return {"ok": True, "host": k[2], "port": k[3]}
        if op == "release":
            k = (msg["model_id"], int(msg["tp_size"]), msg["host"], int(msg["port"]))
            if k in self.seeds:
                self.seeds[k]["inflight"] = max(0, self.seeds[k]["inflight"] - 1)
                self.seeds[k]["served"] += int(bool(msg.get("success", True)))
            return {"ok": True}
        return {"ok": False, "error": f"unknown op {op!r}"}

    def close(self) -> None:
        self.server.stop()


class RForkLoader:
    def __init__(self, planner_host: str, planner_port: int, model_id: str, tp_rank: int = 0, tp_size: int = 1,
                 timeout_ms: int = 3000, backend: Optional[str] = None):
        self.planner = (planner_host, planner_port)
        self.model_id, self.tp_rank, self.tp_size = model_id, tp_rank, tp_size
        self.timeout_ms, self.backend = timeout_ms, backend

    def load(self, model) -> bool:
        try:
            seed = request(*self.planner, {"op": "acquire", "model_id": self.model_id, "tp_size": self.tp_size},
                           self.timeout_ms)
        except SideChannelError as e:
            logger.warning("rfork: %s; falling back to the default loader", e)
            return False
        ok = NetLoader(seed["host"], seed["port"], self.tp_rank, self.tp_size, backend=self.backend,
                       timeout_ms=self.timeout_ms).load(model)
        try:
            request(*self.planner, {"op": "release", "model_id": self.model_id, "tp_size": self.tp_size,
                                    "host": seed["host"], "port": seed["port"], "success": ok}, self.timeout_ms)
        except SideChannelError:
            pass
        return ok

    def register_as_seed(self, host: str, port: int) -> None:
        request(*self.planner, {"op": "register", "model_id": self.model_id, "tp_size": self.tp_size,
                                "host": host, "port": port}, self.timeout_ms)
