"""Alternative model loaders ("netloader", "rfork") next to the default safetensors loader.

``get_model_loader(load_format, extra)`` serves the standalone engine;
``register_model_loaders`` makes the same names known to a host vLLM
(vllm_ascend/__init__.py:64-101 registers its loaders the same way)."""
from __future__ import annotations

from typing import Optional

LOAD_FORMATS = ("auto", "netloader", "rfork", "sharded_state")


def get_model_loader(load_format: str, extra: Optional[dict], tp_rank: int = 0, tp_size: int = 1, model_id: str = ""):
    extra = extra or {}
    if load_format in (None, "auto", "safetensors", "dummy"):
        return None
    if load_format == "netloader":
        from .netloader import NetLoader
        return NetLoader(extra.get("source_host", "127.0.0.1"), int(extra["source_port"]), tp_rank, tp_size,
                         backend=extra.get("backend"))
    if load_format == "rfork":
        from .rfork import RForkLoader
        return RForkLoader(extra.get("planner_host", "127.0.0.1"), int(extra["planner_port"]),
                           extra.get("model_id", model_id), tp_rank, tp_size, backend=extra.get("backend"))
    if load_format == "sharded_state":
        import os
        from .sharded_state import ShardedStateLoader
        return ShardedStateLoader(extra["path"], int(os.environ.get("RANK", "0")))
    raise ValueError(f"unknown load_format {load_format!r}; known: {LOAD_FORMATS}")


def register_model_loaders() -> None:
    try:
        from vllm.model_executor.model_loader import register_model_loader
    except Exception:
        return
    for name in ("netloader", "rfork"):
        try:
            register_model_loader(name)(_HostLoaderShim.for_format(name))
        except Exception:
            pass


class _HostLoaderShim:
    """Adapter with the host framework's loader call shape (``load_weights(model, model_config)``)."""
    fmt = "netloader"

    def __init__(self, load_config=None):
        self.load_config = load_config

    @classmethod
    def for_format(cls, fmt: str):
        return type(f"B200{fmt.capitalize()}Loader", (cls,), {"fmt": fmt})

    def download_model(self, model_config) -> None:
        return None

    def load_weights(self, model, model_config=None) -> None:
        extra = getattr(self.load_config, "model_loader_extra_config", None) or {}
        loader = get_model_loader(self.fmt, extra)
        if loader is None or not loader.load(model):
            raise RuntimeError(f"{self.fmt}: no weights received and no fallback configured")
