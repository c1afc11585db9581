"""Service-level profiling: which Python entry points get a timing span.

The reference writes a YAML of (module path, symbol, span name) triples that an external
service profiler reads to hook the engine (vllm_ascend/profiler/ — registered through
``register_service_profiling``).  The same file is produced here for this package's
symbols, and ``install_spans`` applies it in-process with NVTX ranges + wall-clock totals.
"""
from __future__ import annotations

import functools
import importlib
import os
import time
from typing import Optional

import yaml

DEFAULT_SYMBOLS = [
    {"module": "vllm_ascend_b200.engine.llm", "symbol": "LLMEngine.step", "span": "engine.step"},
    {"module": "vllm_ascend_b200.engine.scheduler", "symbol": "Scheduler.schedule", "span": "scheduler.schedule"},
    {"module": "vllm_ascend_b200.engine.scheduler", "symbol": "Scheduler.update_from_output", "span": "scheduler.update"},
    {"module": "vllm_ascend_b200.engine.model_runner", "symbol": "ModelRunner.execute", "span": "runner.execute"},
    {"module": "vllm_ascend_b200.engine.model_runner", "symbol": "ModelRunner._prepare_inputs", "span": "runner.prepare_inputs"},
    {"module": "vllm_ascend_b200.distributed.kv_transfer.nvlink_connector", "symbol": "NVLinkConnector.start_load_kv",
     "span": "kv.start_load"},
]

totals: dict[str, list] = {}      # span -> [calls, seconds]


def config_path() -> str:
    base = os.getenv("VLLM_B200_SERVICE_PROFILING_DIR") or os.path.join(os.path.expanduser("~"), ".vllm_b200")
    return os.path.join(base, "service_profiling_symbols.yaml")


def generate_service_profiling_config(path: Optional[str] = None, overwrite: bool = False) -> str:
    path = path or config_path()
    if os.path.exists(path) and not overwrite:
        return path
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w") as f:
        yaml.safe_dump({"version": 1, "symbols": DEFAULT_SYMBOLS}, f, sort_keys=False)
    return path


def install_spans(path: Optional[str] = None, nvtx: bool = True) -> list[str]:
    """Wraps every configured symbol; returns the span names installed."""
    path = path or config_path()
    symbols = DEFAULT_SYMBOLS
    if os.path.exists(path):
        with open(path) as f:
            symbols = (yaml.safe_load(f) or {}).get("symbols", DEFAULT_SYMBOLS)
    done = []
    for s in symbols:
        try:
            mod = importlib.import_module(s["module"])
            owner, attr = mod, s["symbol"]
            for part in s["symbol"].split(".")[:-1]:
                owner = getattr(owner, part)
            attr = s["symbol"].split(".")[-1]
            fn = getattr(owner, attr)
        except Exception:
            continue
        if getattr(fn, "_b200_span", None):
            done.append(s["span"])
            continue
        setattr(owner, attr, _wrap(fn, s["span"], nvtx))
        done.append(s["span"])
    return done


def _wrap(fn, span: str, nvtx: bool):
    import torch
    use_nvtx = nvtx and torch.cuda.is_available()

    @functools.wraps(fn)
    def inner(*a, **k):
        if use_nvtx:
            torch.cuda.nvtx.range_push(span)
        t0 = time.perf_counter()
        try:
            return fn(*a, **k)
        finally:
            rec = totals.setdefault(span, [0, 0.0])
            rec[0] += 1
            rec[1] += time.perf_counter() - t0
            if use_nvtx:
                torch.cuda.nvtx.range_pop()
    inner._b200_span = span
    inner.__wrapped__ = fn
    return inner


def uninstall_spans() -> None:
    for s in DEFAULT_SYMBOLS:
        try:
            mod = importlib.import_module(s["module"])
            owner = mod
            for part in s["symbol"].split(".")[:-1]:
                owner = getattr(owner, part)
            attr = s["symbol"].split(".")[-1]
            fn = getattr(owner, attr)
            if getattr(fn, "_b200_span", None):
                setattr(owner, attr, fn.__wrapped__)
        except Exception:
            pass
