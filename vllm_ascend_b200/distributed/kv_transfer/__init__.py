"""KV-transfer connectors (disaggregated prefill, KV offload).

``create_connector`` resolves ``kv_transfer_config["kv_connector"]`` the way the reference
registers its connectors with the engine (vllm_ascend/distributed/kv_transfer/__init__.py:21-56).
"""
from __future__ import annotations

from .base import ConnectorMetadata, KVConnectorBase, plan_head_slices

_CONNECTORS = {
    "NVLinkConnector": ("nvlink_connector", "NVLinkConnector"),
    # names the reference registers, mapped to their B200 counterparts
    "MooncakeConnectorV1": ("nvlink_connector", "NVLinkConnector"),
    "LayerwiseConnector": ("layerwise_connector", "LayerwiseConnector"),
    "MooncakeLayerwiseConnector": ("layerwise_connector", "LayerwiseConnector"),
    "CPUOffloadingConnector": ("cpu_offload_connector", "CPUOffloadConnector"),
    "KVPoolConnector": ("kv_pool", "KVPoolConnector"),
    "AscendStoreConnector": ("kv_pool", "KVPoolConnector"),
    "MooncakeConnectorStoreV1": ("kv_pool", "KVPoolConnector"),
    "SimpleCPUOffloadConnector": ("cpu_offload_connector", "CPUOffloadConnector"),
    "OffloadingConnector": ("cpu_offload_connector", "CPUOffloadConnector"),
    "RecomputeCPUOffloadConnector": ("cpu_offload_connector", "RecomputeCPUOffloadConnector"),
    "RecomputeCPUOffloadConnectorV1": ("cpu_offload_connector", "RecomputeCPUOffloadConnector"),
    "MultiConnector": ("multi_connector", "MultiConnector"),
    "HybridConnector": ("hybrid_connector", "HybridConnector"),
    "SfaRemoteD2HConnector": ("sfa_remote_d2h", "SfaRemoteD2HConnector"),
    "MooncakeHybridConnector": ("hybrid_connector", "HybridConnector"),
    "UCMConnector": ("ucm_connector", "UCMConnector"),
    "UCMConnectorV1": ("ucm_connector", "UCMConnector"),
}


def register_connector(name: str, module: str, cls: str) -> None:
    _CONNECTORS[name] = (module, cls)


def create_connector(engine_cfg, runner) -> KVConnectorBase:
    import importlib
    name = (engine_cfg.kv_transfer_config or {}).get("kv_connector", "NVLinkConnector")
    if name not in _CONNECTORS:
        raise ValueError(f"unknown kv_connector {name!r}; known: {sorted(_CONNECTORS)}")
    module, cls = _CONNECTORS[name]
    mod = importlib.import_module(module if "." in module else f"{__name__}.{module}")
    return getattr(mod, cls)(engine_cfg, runner)


__all__ = ["ConnectorMetadata", "KVConnectorBase", "plan_head_slices", "create_connector",
           "register_connector"]


def register_with_vllm() -> None:
    """Register the connectors with an installed vLLM's ``KVConnectorFactory`` under the
    names this package uses; a no-op when vLLM (or that factory) is absent."""
    try:
        from vllm.distributed.kv_transfer.kv_connector.factory import KVConnectorFactory
    except Exception:
        return
    for name, (module, cls) in _CONNECTORS.items():
        if name in getattr(KVConnectorFactory, "_registry", {}):
            continue
        try:
            KVConnectorFactory.register_connector(
                name, f"vllm_ascend_b200.distributed.kv_transfer.{module}", cls)
        except Exception:
            pass
