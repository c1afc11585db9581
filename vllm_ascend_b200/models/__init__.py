"""Model registry: architecture name -> constructor (the role of
``register_model`` in vllm_ascend/models/__init__.py:4-29)."""
from __future__ import annotations

from typing import Callable

from ..parallel import state as pstate

_REGISTRY: dict[str, Callable] = {}


def register_model(arch: str, ctor: Callable) -> None:
    _REGISTRY[arch] = ctor


def _causal_lm(cfg, device, **kw):
    from .transformer import CausalLM
    return CausalLM(cfg, device, **kw)


for _arch in ("LlamaForCausalLM", "MistralForCausalLM", "Qwen2ForCausalLM", "Qwen3ForCausalLM",
              "Qwen2MoeForCausalLM", "Qwen3MoeForCausalLM", "MixtralForCausalLM", "DeepseekV2ForCausalLM",
              "DeepseekV3ForCausalLM", "DeepseekV32ForCausalLM", "InternLM2ForCausalLM", "Phi3ForCausalLM",
              "GemmaForCausalLM", "Qwen3NextForCausalLM", "GlmForCausalLM", "Glm4ForCausalLM",
              "Ernie4_5ForCausalLM", "Ernie4_5_ForCausalLM", "MiniMaxM2ForCausalLM", "MiniMaxForCausalLM",
              "MiniMaxText01ForCausalLM", "BambaForCausalLM", "Glm4MoeForCausalLM", "Ernie4_5_MoeForCausalLM", "OlmoeForCausalLM", "GraniteForCausalLM", "GraniteMoeHybridForCausalLM", "SeedOssForCausalLM", "SmolLM3ForCausalLM",
              "MinistralForCausalLM", "Dots1ForCausalLM", "HeliumForCausalLM", "Olmo2ForCausalLM", "ArceeForCausalLM"):
    register_model(_arch, _causal_lm)


def _qwen_vl(cfg, device, **kw):
    from .qwen_vl import QwenVLForConditionalGeneration
    return QwenVLForConditionalGeneration(cfg, device, **kw)


for _arch in ("Qwen2_5_VLForConditionalGeneration", "Qwen2VLForConditionalGeneration",
              "Qwen3VLForConditionalGeneration"):
    register_model(_arch, _qwen_vl)


def _audio_lm(cfg, device, **kw):
    from .audio import AudioLMForConditionalGeneration
    return AudioLMForConditionalGeneration(cfg, device, **kw)


register_model("Qwen2AudioForConditionalGeneration", _audio_lm)


def supported_architectures() -> list[str]:
    return sorted(_REGISTRY)


def build_model(engine_cfg, device, moe_runtime=None):
    cfg = engine_cfg.model
    ctor = _REGISTRY.get(cfg.architecture)
    if ctor is None:
        raise ValueError(f"unsupported architecture {cfg.architecture}; known: {supported_architectures()}")
    st = pstate.get_state()
    ep_group = st.ep if (engine_cfg.parallel.enable_expert_parallel and st.ep is not None) else None
    pp = st.pp
    layer_range = None
    if pp is not None and pp.world_size > 1:
        n = cfg.num_hidden_layers
        per = (n + pp.world_size - 1) // pp.world_size
        lo = pp.rank_in_group * per
        layer_range = (lo, min(n, lo + per))
    return ctor(cfg, device, max_model_len=engine_cfg.scheduler.max_model_len,
                tp_group=st.tp, ep_group=ep_group, moe_runtime=moe_runtime,
                layer_range=layer_range)


def register_with_vllm() -> list[str]:
    """General-plugin hook: architectures this package serves that the installed vLLM's registry does
    not know are registered with a description-only class (``host_stub.HostModelStub``), so that
    vLLM's config validation accepts them; the worker builds the real model from this package's
    registry.  Architectures vLLM already knows keep vLLM's own entry (only its metadata is read).
    Returns the names it added."""
    try:
        from vllm import ModelRegistry
    except Exception:
        return []
    known = set(ModelRegistry.get_supported_archs())
    added = []
    for arch in supported_architectures():
        if arch not in known:
            ModelRegistry.register_model(arch, "vllm_ascend_b200.models.host_stub:HostModelStub")
            added.append(arch)
    return added
