"""Typed view over ``additional_config`` plus the config finalisation pipeline.

Key names follow the reference's user API
(docs/source/user_guide/configuration/additional_config.md:48-224, parsed by
vllm_ascend/ascend_config.py:30-328); Ascend-only keys (NZ weight format, torchair
graph backend, xlite) are rejected with an explanatory error instead of being
silently ignored.  Precedence: ``additional_config`` > ``VLLM_B200_*`` env vars
> defaults (vllm_ascend/ascend_config.py:360-372).
"""
from __future__ import annotations

from dataclasses import MISSING, dataclass, field, fields, is_dataclass
from typing import Any, Optional

from . import envs

_ASCEND_ONLY_KEYS = {"weight_nz_mode", "enable_kv_nz", "pa_shape_list", "xlite_graph_config",
                     "torchair_graph_config"}


def _from_dict(cls, d: Optional[dict], path: str):
    d = dict(d or {})
    kw = {}
    for f in fields(cls):
        if f.name not in d:
            continue
        v = d.pop(f.name)
        if f.default_factory is not MISSING:
            proto = f.default_factory()
            if is_dataclass(proto) and isinstance(v, dict):
                v = _from_dict(type(proto), v, f"{path}.{f.name}")
        kw[f.name] = v
    if d:
        raise ValueError(f"unknown keys in {path}: {sorted(d)}")
    return cls(**kw)


@dataclass
class FinegrainedTPConfig:
    lmhead_tensor_parallel_size: int = 0
    oproj_tensor_parallel_size: int = 0
    embedding_tensor_parallel_size: int = 0
    mlp_tensor_parallel_size: int = 0


@dataclass
class FusionConfig:
    """Kernel-fusion switches (the reference's ``ascend_compilation_config`` /
    ``ascend_fusion_config`` toggles, implemented as hand-fused kernels)."""
    fuse_norm_quant: bool = True
    fuse_qknorm_rope: bool = True
    fuse_muls_add: bool = True
    fuse_gemm_comm: bool = True          # AG->GEMM / GEMM->RS over peer memory


@dataclass
class EplbConfig:
    dynamic_eplb: bool = False
    expert_map_path: Optional[str] = None
    expert_map_record_path: Optional[str] = None
    expert_heat_collection_interval: int = 600
    algorithm_execution_interval: int = 50
    num_redundant_experts: int = 0
    eplb_policy_type: int = 2
    eplb_heat_collection_stage: str = "all"      # all | prefill | decode
    load_collection_phase: str = "all"


@dataclass
class ShortRequestFirstConfig:
    enabled: bool = False
    threshold: int = 256
    long_max_wait_ms: float = 2000.0


@dataclass
class ProfilingChunkConfig:
    enabled: bool = False
    smooth_factor: float = 0.8
    min_chunk: int = 512
    need_timing: bool = True
    max_fit_chunk: int = 16384


@dataclass
class BatchJobSchedConfig:
    enabled: bool = False
    max_jobs: int = 20                          # 0 = no limit
    reserve_margin_blocks: int = 2
    reserve_max_blocks: int = 8                 # 0 = no cap
    low_available_tokens_threshold: int = 4096  # above: long-decode jobs first; at or below: short ones
    short_decode_token_threshold: int = 32      # predicted decode length that separates short from long jobs
    max_samples_per_job: int = 10               # the estimate of a job is frozen after this many samples (0 = never)
    cold_start_requests: int = 3                # first requests of a job admitted ahead of the job ordering


@dataclass
class DyntraLBConfig:
    enabled: bool = False
    mode: str = "kv_load"
    start_step: int = 0
    end_step: int = 0
    bubble_threshold: float = 0.1
    long_req_block_threshold: int = 64
    dynamic_max_step: int = 0
    enable_diagnostics: bool = False
    imbalance_threshold: float = 0.15           # pressure gap that triggers a hand-over
    max_migrations_per_step: int = 4


@dataclass
class SchedulerExtConfig:
    enable_balance_scheduling: bool = False
    recompute_scheduler_enable: bool = False
    short_request_first_config: ShortRequestFirstConfig = field(default_factory=ShortRequestFirstConfig)
    profiling_chunk_config: ProfilingChunkConfig = field(default_factory=ProfilingChunkConfig)
    batch_job_sched_config: BatchJobSchedConfig = field(default_factory=BatchJobSchedConfig)
    dyntra_lb_config: DyntraLBConfig = field(default_factory=DyntraLBConfig)


@dataclass
class RejectionSamplerConfig:
    enable_block_verify: bool = False
    enable_entropy_verify: bool = False
    posterior_threshold: float = 0.95
    posterior_alpha: float = 0.4


@dataclass
class DynamicSpecConfig:
    """``method``: None (fixed speculation length) or "acceptance" (per-request length from the measured
    acceptance rate; the reference's "dspark" / "dflash" names select the same controller here, their
    confidence heads are not part of this build).  ``method_params``: min_tokens, budget_threshold,
    ema_alpha, initial_acceptance."""
    method: Optional[str] = None
    method_params: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.method is not None and self.method not in ("acceptance", "dspark", "dflash"):
            raise ValueError("dynamic_spec_config.method must be one of acceptance, dspark, dflash or None")


@dataclass
class RlConfig:
    enabled: bool = False
    sleep_mode_extra_cleanup: bool = False
    enable_training_consistency: bool = False
    enable_batch_invariant: bool = False


@dataclass
class WeightOffloadConfig:
    """Layers i with i % group_size < num_in_group keep their weights on the host and are
    prefetched ``prefetch_step`` layers ahead."""
    enabled: bool = False
    group_size: int = 2
    num_in_group: int = 1
    prefetch_step: int = 1


@dataclass
class SparseKVOffloadConfig:
    """Sparse-attention models: the latent KV of every sequence lives in pinned host memory, the GPU
    keeps ``device_slots_per_seq`` recently selected tokens per sequence (0: 4 x index_topk).  Index
    keys stay on the device (the indexer scores every key each step)."""
    enabled: bool = False
    device_slots_per_seq: int = 0
    num_threads: int = 4


@dataclass
class B200Config:
    finegrained_tp_config: FinegrainedTPConfig = field(default_factory=FinegrainedTPConfig)
    fusion_config: FusionConfig = field(default_factory=FusionConfig)
    eplb_config: EplbConfig = field(default_factory=EplbConfig)
    scheduler_config: SchedulerExtConfig = field(default_factory=SchedulerExtConfig)
    rejection_sampler_config: RejectionSamplerConfig = field(default_factory=RejectionSamplerConfig)
    dynamic_spec_config: DynamicSpecConfig = field(default_factory=DynamicSpecConfig)
    rl_config: RlConfig = field(default_factory=RlConfig)
    weight_offload_config: WeightOffloadConfig = field(default_factory=WeightOffloadConfig)
    sparse_kv_offload_config: SparseKVOffloadConfig = field(default_factory=SparseKVOffloadConfig)
    enable_shared_expert_dp: bool = False
    multistream_overlap_shared_expert: bool = False
    enable_prefill_fused_moe: bool = True        # reference: enable_prefill_mc2
    fused_moe_pool_limit_gb: float = 12.0        # largest packed receive/combine pools the fused path may allocate
    enable_fused_moe_comm: bool = True           # reference: enable_fused_mc2
    fused_moe_max_tokens: int = 512              # reference: mega_moe_max_tokens / MC2 capacity
    enable_mlapo: bool = True
    enable_reduce_sample: bool = False
    enable_transpose_kv_cache_by_block: bool = True
    enable_cpu_binding: bool = True
    kv_load_failure_policy: str = "recompute"    # recompute | fail
    cp_kv_cache_interleave_size: int = 1         # tokens per run when the KV of a sequence is spread over DCP ranks
    dump_config: bool = False
    dump_config_path: Optional[str] = None
    log_path: Optional[str] = None
    refresh: bool = False


_CONFIG: Optional[B200Config] = None


def init_b200_config(additional_config: Optional[dict], refresh: bool = False) -> B200Config:
    """Singleton like ``init_ascend_config`` (vllm_ascend/ascend_config.py:1313-1327)."""
    global _CONFIG
    ac = dict(additional_config or {})
    if _CONFIG is not None and not (refresh or ac.get("refresh")):
        return _CONFIG
    bad = _ASCEND_ONLY_KEYS & set(ac)
    if bad:
        raise ValueError(f"additional_config keys {sorted(bad)} are Ascend-only and have no "
                         "meaning on B200")
    # reference spellings accepted as aliases
    alias = {"ascend_compilation_config": "fusion_config", "ascend_fusion_config": "fusion_config",
             "enable_fused_mc2": "enable_fused_moe_comm", "enable_prefill_mc2": "enable_prefill_fused_moe",
             "mega_moe_max_tokens": "fused_moe_max_tokens", "ascend_log_path": "log_path"}
    for old, new in alias.items():
        if old in ac:
            v = ac.pop(old)
            if old.endswith("compilation_config") and isinstance(v, dict):
                v = {k: x for k, x in v.items() if k in {f.name for f in fields(FusionConfig)}}
            ac.setdefault(new, v)
    cfg = _from_dict(B200Config, ac, "additional_config")
    if "enable_fused_moe_comm" not in ac:
        cfg.enable_fused_moe_comm = envs.VLLM_B200_ENABLE_FUSED_MOE_COMM
    if "enable_cpu_binding" not in ac:
        cfg.enable_cpu_binding = envs.VLLM_B200_ENABLE_CPU_BINDING
    if not cfg.eplb_config.dynamic_eplb and "eplb_config" not in ac:
        cfg.eplb_config.dynamic_eplb = envs.DYNAMIC_EPLB
    if cfg.scheduler_config.enable_balance_scheduling is False and envs.VLLM_B200_BALANCE_SCHEDULING:
        cfg.scheduler_config.enable_balance_scheduling = True
    _CONFIG = cfg
    return cfg


def get_b200_config() -> B200Config:
    if _CONFIG is None:
        return init_b200_config({})
    return _CONFIG


def clear_b200_config() -> None:
    global _CONFIG
    _CONFIG = None


def finegrained_sizes(additional_config: Optional[dict]) -> dict[str, int]:
    fg = (additional_config or {}).get("finegrained_tp_config") or {}
    m = {"otp": "oproj_tensor_parallel_size", "lmtp": "lmhead_tensor_parallel_size",
         "embed_tp": "embedding_tensor_parallel_size", "mlp_tp": "mlp_tensor_parallel_size"}
    return {k: int(fg.get(v, 0) or 0) for k, v in m.items()}


# ---------------------------------------------------------------- validation
def _validate_finegrained(cfg: B200Config, tp: int, dp: int) -> None:
    """Constraints of vllm_ascend/ascend_config.py:641-712: each fine-grained TP size
    must be a multiple of tp whose span divides the DP size (or divide tp)."""
    for name in ("lmhead", "oproj", "embedding", "mlp"):
        size = getattr(cfg.finegrained_tp_config, f"{name}_tensor_parallel_size")
        if not size:
            continue
        if size < 0:
            raise ValueError(f"{name}_tensor_parallel_size must be positive")
        if size <= tp:
            if tp % size:
                raise ValueError(f"{name}_tensor_parallel_size={size} must divide tp={tp}")
        elif size % tp or dp % (size // tp):
            raise ValueError(f"{name}_tensor_parallel_size={size} must be tp ({tp}) times a "
                             f"divisor of dp ({dp})")


def _validate_eplb(e: EplbConfig, is_moe: bool, ep: bool) -> None:
    """vllm_ascend/platform.py:749-795."""
    if e.dynamic_eplb or e.expert_map_path or e.num_redundant_experts:
        if not is_moe:
            raise ValueError("eplb_config requires a MoE model")
        if not ep:
            raise ValueError("eplb_config requires expert parallelism")
    if e.eplb_policy_type not in (0, 1, 2, 3):
        raise ValueError("eplb_policy_type must be 0 (random), 1 (greedy), 2 (swift) or 3 (flashlb)")
    if e.expert_heat_collection_interval <= 0 or e.algorithm_execution_interval <= 0:
        raise ValueError("EPLB intervals must be positive")
    if e.num_redundant_experts < 0:
        raise ValueError("num_redundant_experts must be non-negative")
    if e.dynamic_eplb and e.expert_map_path:
        raise ValueError("dynamic_eplb and a static expert_map_path are mutually exclusive")


def _validate_scheduler_ext(s: SchedulerExtConfig, engine_cfg, dp_size: int = 1) -> None:
    """vllm_ascend/platform.py:798-925: at most one queue policy; option sanity."""
    chosen = [n for n, on in (("short_request_first", s.short_request_first_config.enabled),
                              ("batch_job", s.batch_job_sched_config.enabled),
                              ("profiling_chunk", s.profiling_chunk_config.enabled),
                              ("dyntra_lb", s.dyntra_lb_config.enabled)) if on]
    if len(chosen) > 1:
        raise ValueError(f"scheduler extensions are mutually exclusive, got {chosen}")
    b = s.batch_job_sched_config
    for name in ("max_jobs", "reserve_margin_blocks", "reserve_max_blocks", "max_samples_per_job",
                 "cold_start_requests"):
        if getattr(b, name) < 0:
            raise ValueError(f"batch_job_sched_config.{name} must be non-negative, got {getattr(b, name)}")
    if b.low_available_tokens_threshold <= 0 or b.short_decode_token_threshold <= 0:
        raise ValueError("batch_job_sched_config thresholds must be positive")
    if s.short_request_first_config.enabled and s.short_request_first_config.threshold <= 0:
        raise ValueError("short_request_first_config.threshold must be positive")
    if s.profiling_chunk_config.enabled:
        p = s.profiling_chunk_config
        if not (0 < p.smooth_factor <= 1) or p.min_chunk <= 0 or p.max_fit_chunk < p.min_chunk:
            raise ValueError("invalid profiling_chunk_config")
        if not engine_cfg.scheduler.enable_chunked_prefill:
            raise ValueError("profiling_chunk_config requires chunked prefill")
    if s.recompute_scheduler_enable and not engine_cfg.kv_transfer_config:
        raise ValueError("recompute_scheduler_enable requires a kv_transfer_config (decode node)")
    if s.dyntra_lb_config.enabled and max(dp_size, engine_cfg.parallel.data_parallel_size) <= 1:
        raise ValueError("dyntra_lb_config requires data parallelism")


GRAPH_MODES = ("NONE", "PIECEWISE", "FULL", "FULL_DECODE_ONLY", "FULL_AND_PIECEWISE")


def check_and_update_config(engine_cfg) -> B200Config:
    """Finalisation pipeline (steps of vllm_ascend/platform.py:343-395 that apply)."""
    cfg = init_b200_config(engine_cfg.additional_config, refresh=True)
    pc, sc, cc, mc = engine_cfg.parallel, engine_cfg.scheduler, engine_cfg.compilation, engine_cfg.model
    # 1 parallel sanity
    if pc.tensor_parallel_size < 1 or pc.pipeline_parallel_size < 1:
        raise ValueError("parallel sizes must be >= 1")
    if mc.num_attention_heads % pc.tensor_parallel_size:
        raise ValueError(f"num_attention_heads={mc.num_attention_heads} not divisible by "
                         f"tp={pc.tensor_parallel_size}")
    if pc.prefill_context_parallel_size > 1:
        if engine_cfg.speculative_config:
            raise ValueError("prefill context parallelism cannot be combined with speculative decoding")
        if pc.pipeline_parallel_size > 1:
            raise ValueError("prefill context parallelism cannot be combined with pipeline parallelism")
    if pc.decode_context_parallel_size > 1 and pc.tensor_parallel_size % pc.decode_context_parallel_size:
        raise ValueError("decode_context_parallel_size must divide tensor_parallel_size")
    if pc.enable_expert_parallel and not mc.is_moe:
        pc.enable_expert_parallel = False
    # 2 quantization auto-detect is done by ModelConfig.from_hf_dict
    # 3 knobs that cannot work together
    if cfg.rl_config.enabled:
        engine_cfg.enable_sleep_mode = True
        if cfg.rl_config.enable_training_consistency and (mc.use_mla or mc.sliding_window):
            raise ValueError("training-consistent attention supports neither MLA nor sliding windows")
        if cfg.rl_config.enable_batch_invariant:
            cc.cudagraph_mode = "NONE"
            from .batch_invariant import enable_batch_invariant_mode
            enable_batch_invariant_mode()
    from .attention.backend import set_training_consistent_attention
    set_training_consistent_attention(cfg.rl_config.enabled and cfg.rl_config.enable_training_consistency)
    dp_size = max(1, pc.data_parallel_size)
    if dp_size == 1:      # under a launcher the DP size follows from the world size
        import os
        world = int(os.environ.get("WORLD_SIZE", "1"))
        dp_size = max(1, world // (pc.tensor_parallel_size * pc.pipeline_parallel_size
                                   * max(1, pc.prefill_context_parallel_size)))
    _validate_finegrained(cfg, pc.tensor_parallel_size, dp_size)
    if any(finegrained_sizes(engine_cfg.additional_config).values()):
        if pc.tensor_parallel_size != 1:
            raise ValueError("fine-grained tensor parallelism shards replicated modules of tp=1 replicas")
        cc.cudagraph_mode = "NONE"        # token counts differ per replica and are padded per step
    _validate_eplb(cfg.eplb_config, mc.is_moe, pc.enable_expert_parallel)
    _validate_scheduler_ext(cfg.scheduler_config, engine_cfg, dp_size)
    if mc.is_hybrid and engine_cfg.speculative_config:
        # a rejected draft token has already advanced the recurrent state and cannot be taken back
        raise ValueError("speculative decoding is not supported for models with recurrent (linear-attention) layers")
    if mc.is_hybrid and engine_cfg.cache.enable_prefix_caching:
        # a recurrent state is not addressable by block: a cached prefix could not restore it
        engine_cfg.cache.enable_prefix_caching = False
    if cfg.weight_offload_config.enabled:
        cc.cudagraph_mode = "NONE"        # offloaded weights rotate through device buffers
    if cfg.sparse_kv_offload_config.enabled:
        if not mc.use_sparse:
            raise ValueError("sparse_kv_offload_config needs a sparse-attention (index_topk) model")
        if pc.tensor_parallel_size > 1 and pc.decode_context_parallel_size > 1:
            raise ValueError("sparse KV offload cannot be combined with decode context parallelism")
        cc.cudagraph_mode = "NONE"        # every layer reads the selection back to maintain the host-side LRU
        engine_cfg.cache.enable_prefix_caching = False
        engine_cfg.async_scheduling = False
    if (engine_cfg.speculative_config or {}).get("method") in ("eagle3", "extract_hidden_states"):
        cc.cudagraph_mode = "NONE"        # the head reads intermediate residual streams of eager forwards
    # 4 graph mode normalisation + capture sizes (platform.py:937-1117, 1275-1309)
    cc.cudagraph_mode = cc.cudagraph_mode.upper()
    if cc.cudagraph_mode not in GRAPH_MODES:
        raise ValueError(f"cudagraph_mode must be one of {GRAPH_MODES}")
    if engine_cfg.device != "cuda" or pc.pipeline_parallel_size > 1:
        cc.cudagraph_mode = "NONE"
    if cc.max_cudagraph_capture_size is None:
        cc.max_cudagraph_capture_size = min(sc.max_num_seqs, 1024)
    if pc.enable_sequence_parallel and cc.cudagraph_capture_sizes:
        tp = pc.tensor_parallel_size
        cc.cudagraph_capture_sizes = sorted({((s + tp - 1) // tp) * tp for s in cc.cudagraph_capture_sizes})
    # 5 scheduler selection
    s = cfg.scheduler_config
    if s.recompute_scheduler_enable:
        sc.policy = "recompute"
    elif s.short_request_first_config.enabled:
        sc.policy = "short_request_first"
    elif s.batch_job_sched_config.enabled:
        sc.policy = "batch_job"
    elif s.profiling_chunk_config.enabled:
        sc.policy = "profiling_chunk"
    elif s.enable_balance_scheduling:
        sc.policy = "balance"
    elif s.dyntra_lb_config.enabled:
        sc.policy = "dyntra_lb"
    if sc.max_num_batched_tokens < 1 or sc.max_num_seqs < 1:
        raise ValueError("scheduler limits must be positive")
    if not sc.enable_chunked_prefill and sc.max_num_batched_tokens < sc.max_model_len:
        sc.max_num_batched_tokens = sc.max_model_len
    if engine_cfg.cache.block_size & (engine_cfg.cache.block_size - 1):
        raise ValueError("block_size must be a power of two")
    if cfg.dump_config:
        import json, dataclasses
        path = cfg.dump_config_path or "b200_config_dump.json"
        with open(path, "w") as f:
            json.dump(dataclasses.asdict(cfg), f, indent=1)
    return cfg
