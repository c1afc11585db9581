"""Several connectors behind one: loads come from the first connector that has the KV, every
connector sees finished requests (the reference's MultiConnector override,
vllm_ascend/distributed/kv_transfer/__init__.py:21-40)."""
from __future__ import annotations

from typing import Optional

from .base import ConnectorMetadata, KVConnectorBase


class MultiConnector(KVConnectorBase):
    def __init__(self, engine_cfg, runner):
        import copy
        from . import create_connector
        subs = (engine_cfg.kv_transfer_config.get("kv_connector_extra_config") or {}).get("connectors") or []
        if not subs:
            raise ValueError("MultiConnector needs kv_connector_extra_config['connectors']")
        self.connectors: list[KVConnectorBase] = []
        for sub in subs:
            c = copy.copy(engine_cfg)
            c.kv_transfer_config = sub
            self.connectors.append(create_connector(c, runner))
        self._owner: dict[str, KVConnectorBase] = {}

    def get_num_new_matched_tokens(self, req, num_computed_tokens: int) -> tuple[int, bool]:
        for c in self.connectors:
            n, is_async = c.get_num_new_matched_tokens(req, num_computed_tokens)
            if n > 0:
                self._owner[req.request_id] = c
                return n, is_async
        return 0, False

    def update_state_after_alloc(self, req, block_ids: list, num_external_tokens: int) -> None:
        c = self._owner.get(req.request_id)
        if c is not None:
            c.update_state_after_alloc(req, block_ids, num_external_tokens)

    def build_connector_meta(self, scheduler_output) -> ConnectorMetadata:
        meta = ConnectorMetadata()
        meta.reqs_to_recv = {i: c.build_connector_meta(scheduler_output) for i, c in enumerate(self.connectors)}
        return meta

    def request_finished(self, req, block_ids: list) -> tuple[bool, Optional[dict]]:
        self._owner.pop(req.request_id, None)
        delay, params = False, None
        for c in self.connectors:
            d, p = c.request_finished(req, block_ids)
            if d and delay:
                raise RuntimeError("two connectors asked to keep the blocks of one request")
            delay = delay or d
            params = params or p
        return delay, params

    def is_ready(self, req) -> bool:
        c = self._owner.get(req.request_id)
        return c.is_ready(req) if c is not None else True

    def take_failed_requests(self) -> list[str]:
        return [r for c in self.connectors for r in c.take_failed_requests()]

    def start_load_kv(self, scheduler_output) -> None:
        for c in self.connectors:
            c.start_load_kv(scheduler_output)

    def step_finished(self, scheduler_output, scheduler) -> None:
        for c in self.connectors:
            c.step_finished(scheduler_output, scheduler)

    def reap(self, scheduler) -> None:
        for c in self.connectors:
            if hasattr(c, "reap"):
                c.reap(scheduler)

    @property
    def num_delayed(self) -> int:
        return sum(getattr(c, "num_delayed", 0) for c in self.connectors)

    def close(self) -> None:
        for c in self.connectors:
            c.close()
