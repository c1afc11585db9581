"""Out-of-tree vLLM platform for B200 GPUs.

This is the class a host vLLM instantiates after ``register()`` returned its dotted path.
It plays the role of ``NPUPlatform`` (vllm_ascend/platform.py:76-515): device identity,
capability flags, class-path getters (attention backend, worker, punica wrapper, device
communicator, graph wrapper), quantization names, and the ``check_and_update_config``
pipeline that sanitises a ``VllmConfig`` and installs the typed ``additional_config``.

The standalone engine does not need this module; it calls ``platform_config`` directly.
Without an importable vLLM the class still works as a plain object (used by CPU tests).
"""
from __future__ import annotations

import os
from typing import Any, Optional

import torch

from . import envs
from .logger import logger

try:  # the host framework is optional
    from vllm.platforms.interface import Platform as _Base, PlatformEnum as _Enum
    _OOT = _Enum.OOT
except Exception:  # pragma: no cover - exercised only without vLLM
    class _Base:  # type: ignore
        pass
    _OOT = "OOT"

SUPPORTED_QUANTIZATION = ["fp8", "compressed-tensors", "b200", "w8a8_dynamic", "modelopt"]

_HAS_GPU = torch.cuda.is_available()

#: the worker class a host vLLM's executor constructs (a ``WorkerBase`` subclass)
WORKER_CLS = "vllm_ascend_b200.worker.vllm_worker.B200VllmWorker"


class B200Platform(_Base):
    _enum = _OOT
    # without a visible GPU the platform still loads (CPU runs of the whole stack, used by the
    # tests of the plugin path): tensors then live on the host and the ops take their PyTorch path
    device_name: str = "cuda" if _HAS_GPU else "cpu"
    device_type: str = "cuda" if _HAS_GPU else "cpu"
    dispatch_key: str = "CUDA" if _HAS_GPU else "CPU"
    ray_device_key: str = "GPU"
    dist_backend: str = "nccl" if _HAS_GPU else "gloo"
    device_control_env_var: str = "CUDA_VISIBLE_DEVICES"
    simple_compile_backend: str = "eager"
    supported_quantization: list = SUPPORTED_QUANTIZATION
    additional_env_vars: list = [k for k in envs.env_variables if k.startswith("VLLM_B200")]

    # ---- identity / capability -------------------------------------------------------
    @classmethod
    def get_device_capability(cls, device_id: int = 0):
        if not torch.cuda.is_available():
            return None
        major, minor = torch.cuda.get_device_capability(device_id)
        try:
            from vllm.platforms.interface import DeviceCapability
            return DeviceCapability(major=major, minor=minor)
        except Exception:
            return (major, minor)

    @classmethod
    def get_device_name(cls, device_id: int = 0) -> str:
        return torch.cuda.get_device_name(device_id) if torch.cuda.is_available() else "B200 (absent)"

    @classmethod
    def get_device_total_memory(cls, device_id: int = 0) -> int:
        if not _HAS_GPU:
            import psutil
            return int(psutil.virtual_memory().total)
        return torch.cuda.get_device_properties(device_id).total_memory

    @classmethod
    def get_current_memory_usage(cls, device=None) -> float:
        if not _HAS_GPU:
            return 0.0
        torch.cuda.reset_peak_memory_stats(device)
        return torch.cuda.max_memory_allocated(device)

    @classmethod
    def set_device(cls, device: torch.device) -> None:
        if _HAS_GPU:
            torch.cuda.set_device(device)

    @classmethod
    def inference_mode(cls):
        return torch.inference_mode()

    @classmethod
    def is_pin_memory_available(cls) -> bool:
        return _HAS_GPU

    @classmethod
    def is_sleep_mode_available(cls) -> bool:
        return True

    @classmethod
    def is_cumem_allocator_available(cls) -> bool:
        return True

    @classmethod
    def opaque_attention_op(cls) -> bool:
        return True

    @classmethod
    def support_hybrid_kv_cache(cls) -> bool:
        return True

    @classmethod
    def support_static_graph_mode(cls) -> bool:
        return True

    @classmethod
    def use_custom_op_collectives(cls) -> bool:
        return True

    @classmethod
    def supports_fp8(cls) -> bool:
        return True

    @classmethod
    def fp8_dtype(cls) -> torch.dtype:
        return torch.float8_e4m3fn

    @classmethod
    def num_compute_units(cls, device_id: int = 0) -> int:
        return torch.cuda.get_device_properties(device_id).multi_processor_count \
            if torch.cuda.is_available() else 148

    # ---- class-path getters (platform.py:163-197) ------------------------------------
    @classmethod
    def get_attn_backend_cls(cls, selected_backend=None, *args, **kwargs) -> str:
        cfg = kwargs.get("attn_selector_config")
        use_mla = bool(kwargs.get("use_mla", getattr(cfg, "use_mla", False)))
        use_sparse = bool(kwargs.get("use_sparse", getattr(cfg, "use_sparse", False)))
        use_compress = bool(kwargs.get("use_compress", getattr(cfg, "use_compress", False)))
        from .attention.backend import attn_backend_path
        return attn_backend_path(use_mla, use_sparse, use_compress)

    @classmethod
    def get_punica_wrapper(cls) -> str:
        return "vllm_ascend_b200.lora.punica.PunicaWrapperB200"

    @classmethod
    def get_device_communicator_cls(cls) -> str:
        return "vllm_ascend_b200.distributed.communicator.B200Communicator"

    @classmethod
    def get_static_graph_wrapper_cls(cls) -> str:
        return "vllm_ascend_b200.compilation.cuda_graph.CUDAGraphWrapper"

    @classmethod
    def get_pass_manager_cls(cls) -> str:
        return "vllm_ascend_b200.compilation.fusion.FusionPlan"

    @classmethod
    def get_compile_backend(cls) -> str:
        return "vllm_ascend_b200.compilation.fusion.EagerFusedBackend"

    # ---- config pipeline ---------------------------------------------------------------
    @classmethod
    def pre_register_and_update(cls, parser=None) -> None:
        """Adds this package's quantization names to the CLI choices and imports the quant
        configs so the registry is populated (platform.py:261-286)."""
        from . import quantization  # noqa: F401
        if parser is None:
            return
        for action in getattr(parser, "_actions", []):
            if getattr(action, "dest", None) == "quantization" and action.choices is not None:
                for q in SUPPORTED_QUANTIZATION:
                    if q not in action.choices:
                        action.choices.append(q)

    @classmethod
    def apply_config_platform_defaults(cls, vllm_config: Any) -> None:
        """Default largest capture size = min(max_num_seqs * decode_query_len, 512)
        (platform.py:1275-1309)."""
        comp = getattr(vllm_config, "compilation_config", None)
        sched = getattr(vllm_config, "scheduler_config", None)
        if comp is None or sched is None:
            return
        if getattr(comp, "max_cudagraph_capture_size", None) is None and \
                not getattr(comp, "cudagraph_capture_sizes", None):
            spec = getattr(vllm_config, "speculative_config", None)
            qlen = 1 + (getattr(spec, "num_speculative_tokens", 0) or 0 if spec is not None else 0)
            comp.max_cudagraph_capture_size = min(sched.max_num_seqs * qlen, 512)

    @classmethod
    def check_and_update_config(cls, vllm_config: Any) -> None:
        """The finalisation pipeline of vllm_ascend/platform.py:343-395 on a host
        ``VllmConfig``: typed additional_config, sanitising of knobs that do not apply,
        validation of EPLB / scheduler extensions, graph-mode normalisation, class
        selection and allocator environment."""
        from .platform_config import (GRAPH_MODES, _validate_eplb, _validate_finegrained,
                                      init_b200_config)
        cfg = init_b200_config(getattr(vllm_config, "additional_config", None) or {}, refresh=True)
        pc = getattr(vllm_config, "parallel_config", None)
        sc = getattr(vllm_config, "scheduler_config", None)
        cc = getattr(vllm_config, "compilation_config", None)
        mc = getattr(vllm_config, "model_config", None)
        cache = getattr(vllm_config, "cache_config", None)
        _validate_parallel_config(vllm_config)
        _auto_detect_quantization(vllm_config)
        _fix_incompatible_config(vllm_config)
        if pc is not None:
            _validate_finegrained(cfg, pc.tensor_parallel_size, max(1, getattr(pc, "data_parallel_size", 1)))
            is_moe = bool(mc is not None and getattr(getattr(mc, "hf_config", None), "num_experts", 0)
                          or getattr(getattr(mc, "hf_config", None), "n_routed_experts", 0))
            _validate_eplb(cfg.eplb_config, is_moe, getattr(pc, "enable_expert_parallel", False))
            if getattr(pc, "worker_cls", "auto") == "auto":
                pc.worker_cls = WORKER_CLS
        if cc is not None:
            mode = getattr(cc, "cudagraph_mode", None)
            name = getattr(mode, "name", mode)
            if isinstance(name, str) and name.upper() not in GRAPH_MODES:
                raise ValueError(f"cudagraph_mode must be one of {GRAPH_MODES}")
            if mc is not None and getattr(mc, "enforce_eager", False):
                try:
                    cc.cudagraph_mode = type(mode).NONE if hasattr(type(mode), "NONE") else "NONE"
                except Exception:
                    cc.cudagraph_mode = "NONE"
            if pc is not None and getattr(pc, "use_sequence_parallel_moe", False) and \
                    getattr(cc, "cudagraph_capture_sizes", None):
                tp = pc.tensor_parallel_size
                cc.cudagraph_capture_sizes = sorted({((s + tp - 1) // tp) * tp
                                                     for s in cc.cudagraph_capture_sizes})
        if cache is not None and (getattr(cache, "block_size", None) in (None, 0)
                                  or not getattr(cache, "user_specified_block_size", True)):
            cache.block_size = 128 if _HAS_GPU else 16      # 128-token pages: one TMA box per KV head
        if cc is not None:
            # the worker runs this package's own model code and CUDA graphs: the host's tracing
            # compiler has nothing to compile
            try:
                from vllm.config import CompilationMode
                cc.mode = CompilationMode.NONE
            except Exception:
                pass
        if sc is not None:
            s = cfg.scheduler_config
            if s.recompute_scheduler_enable:
                sc.scheduler_cls = "vllm_ascend_b200.core.recompute.RecomputeScheduler"
            elif s.short_request_first_config.enabled:
                sc.scheduler_cls = "vllm_ascend_b200.core.short_request_first.ShortRequestFirstScheduler"
            elif s.batch_job_sched_config.enabled:
                sc.scheduler_cls = "vllm_ascend_b200.core.batch_job_aware.BatchJobAwareScheduler"
            elif s.profiling_chunk_config.enabled:
                sc.scheduler_cls = "vllm_ascend_b200.core.profiling_chunk.ProfilingChunkScheduler"
            elif s.enable_balance_scheduling:
                sc.scheduler_cls = "vllm_ascend_b200.core.balance.BalanceScheduler"
        _validate_cp_kv(vllm_config)
        _set_allocator_env()
        logger.debug("B200 platform config finalised: %s", cfg)

    @classmethod
    def set_additional_forward_context(cls, *args, **kwargs) -> dict:
        """Per-step extras a runner adds to the forward context (platform.py:398-515)."""
        from .forward_context import build_extra_context
        return build_extra_context(*args, **kwargs)

    @classmethod
    def import_kernels(cls) -> None:
        """Loads the native library and defines the ``torch.ops.b200`` dispatcher ops with their meta
        functions (the reference imports its compiled op library and the meta registrations here,
        platform.py import_kernels)."""
        from . import _native
        _native.load(required=torch.cuda.is_available())
        from .ops.torch_bindings import register as register_torch_ops
        register_torch_ops()


# GPU-side knobs of a host config that this runtime does not honour are reset so they can
# not select a foreign code path (the reference resets the CUDA-only ones the same way,
# platform.py:518-746).
_RESET_ATTRS = {
    "model_config": {"disable_cascade_attn": True},
    "parallel_config": {"enable_dbo": False, "ubatch_size": 0},
    "compilation_config": {"use_inductor": False},
}


def _fix_incompatible_config(vllm_config: Any) -> None:
    for section, attrs in _RESET_ATTRS.items():
        obj = getattr(vllm_config, section, None)
        if obj is None:
            continue
        for k, v in attrs.items():
            if hasattr(obj, k) and getattr(obj, k) != v:
                logger.info("resetting %s.%s to %r (not supported by the B200 runtime)", section, k, v)
                try:
                    setattr(obj, k, v)
                except Exception:
                    pass
    ktc = getattr(vllm_config, "kv_transfer_config", None)
    if ktc is not None and getattr(ktc, "engine_id", None):
        # instances launched from one command line would otherwise share an engine id
        dp = getattr(getattr(vllm_config, "parallel_config", None), "data_parallel_rank", 0) or 0
        if not str(ktc.engine_id).endswith(f"-dp{dp}") and dp:
            ktc.engine_id = f"{ktc.engine_id}-dp{dp}"


def _validate_parallel_config(vllm_config: Any) -> None:
    """Parallel layouts the worker behind a host engine cannot run are refused before any process
    starts (the reference refuses prefill context parallelism on its first-generation runner and
    ties sparse-attention DCP to the TP size, platform.py:1381-1398; dynamic speculative lengths
    with DCP, platform.py:1401-1418)."""
    pc = getattr(vllm_config, "parallel_config", None)
    if pc is None:
        return
    tp = getattr(pc, "tensor_parallel_size", 1) or 1
    pcp = getattr(pc, "prefill_context_parallel_size", 1) or 1
    dcp = getattr(pc, "decode_context_parallel_size", 1) or 1
    if pcp > 1:
        raise ValueError("prefill context parallelism is offered by this package's own engine "
                         "(LLM(prefill_context_parallel_size=...)), not behind a host engine: "
                         f"set --prefill-context-parallel-size 1 (got {pcp})")
    if dcp > 1 and tp % dcp:
        raise ValueError(f"decode_context_parallel_size ({dcp}) must divide tensor_parallel_size ({tp})")
    spec = getattr(vllm_config, "speculative_config", None)
    if spec is not None and dcp > 1 and getattr(spec, "num_speculative_tokens_per_batch_size", None):
        raise ValueError("per-batch-size speculative lengths cannot be combined with decode context "
                         "parallelism: set --decode-context-parallel-size 1 or drop "
                         "num_speculative_tokens_per_batch_size")


def _auto_detect_quantization(vllm_config: Any) -> None:
    """A checkpoint directory that carries a quantization description selects the quantization
    method when the user gave none (platform.py:365-366, utils.py maybe_auto_detect_quantization)."""
    mc = getattr(vllm_config, "model_config", None)
    if mc is None or getattr(mc, "quantization", None):
        return
    path = getattr(mc, "model", None)
    if not isinstance(path, str) or not os.path.isdir(path):
        return
    from .quantization import detect_quantization
    found = detect_quantization(path, getattr(mc, "hf_config", None))
    if found:
        logger.info("quantization method %r detected from %s", found, path)
        try:
            mc.quantization = found
        except Exception:
            pass


def _validate_cp_kv(vllm_config: Any) -> None:
    """Context parallelism with KV transfer moves whole pages between instances: the interleave
    granule of the context-parallel KV layout has to be the page size (platform.py:1167-1184)."""
    pc = getattr(vllm_config, "parallel_config", None)
    cache = getattr(vllm_config, "cache_config", None)
    if pc is None or cache is None or getattr(vllm_config, "kv_transfer_config", None) is None:
        return
    cp = (getattr(pc, "prefill_context_parallel_size", 1) or 1) * (getattr(pc, "decode_context_parallel_size", 1) or 1)
    inter = getattr(pc, "cp_kv_cache_interleave_size", None)
    if cp > 1 and inter is not None and inter != getattr(cache, "block_size", inter):
        raise ValueError(f"cp_kv_cache_interleave_size ({inter}) must equal block_size ({cache.block_size}) "
                         "when context parallelism is combined with KV transfer or a KV pool")


def _set_allocator_env() -> None:
    """Expandable segments keep the caching allocator from fragmenting under changing batch
    shapes; not combined with the sleep-mode pluggable allocator (platform.py:1208-1244)."""
    conf = os.environ.get("PYTORCH_CUDA_ALLOC_CONF", "")
    if "expandable_segments" not in conf:
        os.environ["PYTORCH_CUDA_ALLOC_CONF"] = (conf + "," if conf else "") + "expandable_segments:True"
