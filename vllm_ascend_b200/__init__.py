"""B200-native LLM serving framework: standalone engine plus vLLM plugin entry points.

The four ``register*`` functions are the entry points a host vLLM discovers through the
``vllm.platform_plugins`` / ``vllm.general_plugins`` groups, the contract of
vllm_ascend/__init__.py:21-45 (register -> platform class path, register_connector,
register_model_loader, register_service_profiling).  Everything heavy is imported lazily so
``import vllm_ascend_b200`` stays cheap and works without a GPU.
"""
from __future__ import annotations

__version__ = "0.1.0"

_LAZY = {
    "LLM": ("vllm_ascend_b200.engine.llm", "LLM"),
    "LLMEngine": ("vllm_ascend_b200.engine.llm", "LLMEngine"),
    "SamplingParams": ("vllm_ascend_b200.engine.request", "SamplingParams"),
    "RequestOutput": ("vllm_ascend_b200.engine.request", "RequestOutput"),
    "EngineConfig": ("vllm_ascend_b200.config", "EngineConfig"),
    "ModelConfig": ("vllm_ascend_b200.config", "ModelConfig"),
}


def __getattr__(name: str):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def register() -> str:
    """Platform plugin entry point: the dotted path of the platform class."""
    return "vllm_ascend_b200.platform.B200Platform"


def register_connector() -> None:
    """General plugin: make the KV connectors known to a host vLLM's connector factory."""
    from .distributed.kv_transfer import register_with_vllm
    register_with_vllm()


def register_model_loader() -> None:
    """General plugin: register the peer-to-peer weight loaders."""
    from .model_loader import register_model_loaders
    register_model_loaders()


def register_service_profiling() -> None:
    """General plugin: write the default service-profiling symbol configuration."""
    from .profiler.service_profiling import generate_service_profiling_config
    generate_service_profiling_config()


def register_model() -> None:
    """General plugin: expose the model classes to a host vLLM's model registry."""
    from .models import register_with_vllm
    register_with_vllm()
