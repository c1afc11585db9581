"""Connector for an external unified cache manager (UCM).

A unified cache manager is a separate package that owns a tiered KV store (device, host, SSD,
remote) with its own lookup, placement and transfer engines and ships an engine-side connector
object.  This connector is the thin adapter: it imports that object by name, constructs it with
the engine's configuration and this rank's runner, and forwards every hook of the connector
contract to it.  The manager's connector may itself be a dispatcher around an inner connector
(``.connector``) that implements hooks the dispatcher does not redeclare; such hooks are looked
up on the inner object so that a base-class no-op cannot hide them.  Hooks neither object has
keep the contract's defaults (nothing matched, nothing to load).

Configuration (``kv_connector_extra_config``):

* ``ucm_connector_module``: module that holds the manager's connector (default
  ``ucm.integration.vllm.ucm_connector``),
* ``ucm_connector_class``: its class name (default ``UCMConnector``); it is called as
  ``cls(engine_cfg, runner)``.

The reference wraps the same external object the same way
(vllm_ascend/distributed/kv_transfer/kv_pool/ucm_connector/connector.py:37-75: ``UCMConnectorV1``
constructs ``ucm.integration.vllm.ucm_connector.UCMConnector`` and delegates, preferring the
dispatcher's own methods and falling through to its inner connector).
"""
from __future__ import annotations

import importlib
from typing import Any, Optional

from .base import ConnectorMetadata, KVConnectorBase

DEFAULT_MODULE = "ucm.integration.vllm.ucm_connector"
DEFAULT_CLASS = "UCMConnector"


class UCMConnector(KVConnectorBase):
    def __init__(self, engine_cfg, runner):
        extra = (engine_cfg.kv_transfer_config or {}).get("kv_connector_extra_config") or {}
        module = extra.get("ucm_connector_module", DEFAULT_MODULE)
        cls = extra.get("ucm_connector_class", DEFAULT_CLASS)
        try:
            impl = getattr(importlib.import_module(module), cls)
        except (ImportError, AttributeError) as e:
            raise ImportError(f"UCMConnector: cannot load {module}.{cls} ({e}); install the unified cache "
                              "manager or point ucm_connector_module / ucm_connector_class at its connector") from e
        self._engine = impl(engine_cfg, runner)
        self.role = getattr(self._engine, "role", self.role)

    # ------------------------------------------------------------------ delegation
    def _owner_of(self, name: str) -> Any:
        """The object that implements ``name``: the manager's connector when its class declares the
        hook itself, else its inner connector when it has one."""
        declared = any(name in vars(c) for c in type(self._engine).__mro__ if c is not object
                       and c is not KVConnectorBase)
        if not declared:
            inner = getattr(self._engine, "connector", None)
            if inner is not None and callable(getattr(inner, name, None)):
                return inner
        return self._engine

    def _call(self, name: str, default, *args, **kwargs):
        hook = getattr(self._owner_of(name), name, None)
        if callable(hook):
            return hook(*args, **kwargs)
        return default() if callable(default) else default

    # ---- scheduler side
    def get_num_new_matched_tokens(self, req, num_computed_tokens: int) -> tuple[int, bool]:
        return self._call("get_num_new_matched_tokens", (0, False), req, num_computed_tokens)

    def update_state_after_alloc(self, req, block_ids: list, num_external_tokens: int) -> None:
        self._call("update_state_after_alloc", None, req, block_ids, num_external_tokens)

    def build_connector_meta(self, scheduler_output) -> Optional[ConnectorMetadata]:
        return self._call("build_connector_meta", None, scheduler_output)

    def request_finished(self, req, block_ids: list) -> tuple[bool, Optional[dict]]:
        return self._call("request_finished", (False, None), req, block_ids)

    def request_preempted(self, req) -> None:
        self._call("request_preempted", None, req)

    def is_ready(self, req) -> bool:
        return self._call("is_ready", True, req)

    def take_failed_requests(self) -> list[str]:
        return self._call("take_failed_requests", list)

    # ---- worker side
    def register_kv_caches(self, kv_caches: list) -> None:
        self._call("register_kv_caches", None, kv_caches)

    def start_load_kv(self, scheduler_output) -> None:
        self._call("start_load_kv", None, scheduler_output)

    def step_finished(self, scheduler_output, scheduler) -> None:
        self._call("step_finished", None, scheduler_output, scheduler)

    def stats(self) -> dict:
        return self._call("stats", dict)

    def close(self) -> None:
        if callable(getattr(self._owner_of("close"), "close", None)):
            self._call("close", None)
        else:
            self._call("shutdown", None)
