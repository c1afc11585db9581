"""Fusion plan: which hand-fused kernels replace which op sequences.

The reference rewrites FX graphs with pattern-matching passes
(vllm_ascend/compilation/passes/norm_quant_fusion_pass.py:29-403,
qknorm_rope_fusion_pass.py:31-244, muls_add_pass.py, manager
graph_fusion_pass_manager.py:25-67).  Here there is no tracing compiler on the hot path:
every fusion is a CUDA kernel the model code calls directly, and this table only records
which of them are switched on (``additional_config["fusion_config"]``).  The layers ask
``get_plan().enabled(...)``: with a fusion off they run the op sequence it replaces (residual add then
RMSNorm; q/k norm, rotary and cache write as three passes; gate_up GEMM then SiLU-mul; NCCL
collectives around plain GEMMs), which is what tests use as the oracle of the fused kernels.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from ..platform_config import get_b200_config


@dataclass(frozen=True)
class Fusion:
    name: str
    replaces: str          # the op sequence the reference's pass matches
    kernel: str            # the kernel entry point that implements the fused form
    flag: str              # attribute of FusionConfig that switches it


FUSIONS = (
    Fusion("add_rmsnorm", "residual add -> RMSNorm (+bias)", "b200_rms_norm", "fuse_norm_quant"),
    Fusion("add_rmsnorm_quant", "residual add -> RMSNorm -> 1x128 fp8 quant", "b200_rms_norm + b200_quant_fp8_group128",
           "fuse_norm_quant"),
    Fusion("qknorm_rope", "split qkv -> q/k RMSNorm -> RoPE -> paged KV write", "b200_qknorm_rope_kvwrite",
           "fuse_qknorm_rope"),
    Fusion("gemm_swiglu", "gate_up GEMM -> SiLU*mul", "b200_gemm_swiglu_bf16", "fuse_muls_add"),
    Fusion("gemm_reduce_scatter", "row-parallel GEMM -> reduce-scatter", "b200_gemm_rs_bf16", "fuse_gemm_comm"),
    Fusion("allgather_gemm", "all-gather -> column-parallel GEMM", "b200_gemm_ag_bf16", "fuse_gemm_comm"),
    Fusion("reduce_add_rmsnorm", "reduce-scatter tail -> add -> RMSNorm -> all-gather push",
           "b200_reduce_add_norm_push", "fuse_gemm_comm"),
)


class FusionPlan:
    """Plays the role of the pass manager: holds the active fusions for this process."""

    def __init__(self):
        cfg = get_b200_config().fusion_config
        self.active = {f.name: bool(getattr(cfg, f.flag, True)) for f in FUSIONS}

    def enabled(self, name: str) -> bool:
        return self.active.get(name, False)

    def describe(self) -> list[str]:
        return [f"{f.name}: {f.replaces} => {f.kernel} [{'on' if self.active[f.name] else 'off'}]"
                for f in FUSIONS]

    # pass-manager call shape: a graph goes in, the same graph comes out
    def __call__(self, graph):
        return graph


_PLAN = None


def get_plan() -> FusionPlan:
    """The process-wide plan, built from the configuration on first use."""
    global _PLAN
    cfg = get_b200_config().fusion_config
    if _PLAN is None or _PLAN._cfg is not cfg:
        _PLAN = FusionPlan()
        _PLAN._cfg = cfg
    return _PLAN


class EagerFusedBackend:
    """Compile-backend stand-in for a host framework that insists on one: returns the module's
    own forward, whose ops already are the fused kernels."""

    def __call__(self, graph_module, example_inputs=None) -> Callable:
        return graph_module.forward if hasattr(graph_module, "forward") else graph_module
