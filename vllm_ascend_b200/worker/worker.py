"""Process-per-GPU worker.

Owns the device, the distributed groups, the model runner and the memory pools of one
rank, and exposes the worker surface an engine (this package's, or a host vLLM's executor)
drives: init_device → load_model → determine_num_blocks → initialize_cache →
compile_or_warm_up_model → execute_model, plus sleep/wake_up, weight updates, profiling,
LoRA passthroughs and a health check.  Role of ``NPUWorker``
(vllm_ascend/worker/worker.py:99-1116).
"""
from __future__ import annotations

import time
from typing import Optional

import torch

from .. import _native, envs
from ..logger import logger
from ..parallel import state as pstate


class B200Worker:
    def __init__(self, cfg, local_rank: Optional[int] = None, rank: Optional[int] = None,
                 distributed_init_method: Optional[str] = None, is_driver_worker: bool = True):
        self.cfg = cfg
        self.local_rank, self.rank = local_rank, rank
        self.distributed_init_method = distributed_init_method
        self.is_driver_worker = is_driver_worker
        self.device: Optional[torch.device] = None
        self.runner = None
        self.moe_runtime = None
        self.num_blocks = 0
        self.sleep_level = 0
        self._weight_update_state = "idle"
        self._profiler = None
        self._mem_before_load = 0
        self.offloader = None

    # ------------------------------------------------------------------ device / groups
    def init_device(self) -> None:
        cfg = self.cfg
        rank, local, world = pstate.init_distributed(backend=None if cfg.device == "cuda" else "gloo")
        pc = cfg.parallel
        pc.rank, pc.local_rank, pc.world_size = rank, local, world
        self.rank, self.local_rank, self.world_size = rank, local, world
        if cfg.device == "cuda":
            if not torch.cuda.is_available():
                raise RuntimeError("device='cuda' requested but no GPU is visible")
            # a single-process engine may be pinned to any GPU ("cuda:1"); under torchrun
            # the local rank decides
            idx = cfg.device_index if (world == 1 and cfg.device_index is not None) else local
            self.device = torch.device("cuda", idx)
            torch.cuda.set_device(self.device)
            _native.load(required=True)
            free, total = torch.cuda.mem_get_info(self.device)
            self._mem_before_load = total - free
            if envs.VLLM_B200_ENABLE_CPU_BINDING:
                try:
                    from ..cpu_binding import bind_cpus
                    bind_cpus(idx, local_world=max(1, min(world, torch.cuda.device_count())))
                except Exception as e:     # binding is an optimisation, never a reason to fail
                    logger.debug("cpu binding skipped: %s", e)
        else:
            self.device = torch.device("cpu")
        if world > 1:
            pcp = max(1, pc.prefill_context_parallel_size)
            dp = max(1, world // (pc.tensor_parallel_size * pc.pipeline_parallel_size * pcp))
            pc.data_parallel_size = dp
            from ..platform_config import finegrained_sizes
            pstate.initialize_model_parallel(pc.tensor_parallel_size, pc.pipeline_parallel_size, dp,
                                             pc.decode_context_parallel_size,
                                             finegrained=finegrained_sizes(cfg.additional_config), pcp=pcp)
        else:
            pstate.initialize_model_parallel()
        from ..parallel import finegrained
        finegrained.init_from_groups()
        from ..engine.model_runner import ModelRunner
        self.runner = ModelRunner(cfg, self.device)

    # ------------------------------------------------------------------ model / memory
    def _pool(self, tag: str):
        import contextlib
        if self.cfg.enable_sleep_mode and self.cfg.device == "cuda":
            from ..device_allocator.vmm import VmmAllocator
            return VmmAllocator.get_instance().use_memory_pool(tag)
        return contextlib.nullcontext()

    def load_model(self) -> None:
        cfg, pc = self.cfg, self.cfg.parallel
        if cfg.model.is_moe and pc.enable_expert_parallel and self.world_size > 1:
            from ..ops.moe_comm import MoERuntime
            self.moe_runtime = MoERuntime(cfg, self.device)
        with self._pool("weights"):
            self.runner.load_model(moe_runtime=self.moe_runtime)
        if cfg.enable_lora:
            self.runner.init_lora()
        if self.world_size == 1 and cfg.device == "cuda":
            from ..models import folded
            if folded.attach(self.runner.model, cfg):
                logger.info("RMSNorm folded into the neighbouring GEMMs (%d layers)", len(self.runner.model.layers))
        from ..platform_config import get_b200_config
        oc = get_b200_config().weight_offload_config
        if oc.enabled:
            from ..offloader import PrefetchOffloader
            self.offloader = PrefetchOffloader(self.runner.model, oc.group_size, oc.num_in_group, oc.prefetch_step)
        # the fused sequence-sharded TP path has no adapter hook: LoRA engines use the NCCL path
        self.tp_comm_calibration = None
        from ..compilation.fusion import get_plan
        if self.world_size > 1 and cfg.device == "cuda" and envs.VLLM_B200_TP_COMM in ("fused", "auto") \
                and get_plan().enabled("gemm_reduce_scatter") \
                and pc.tensor_parallel_size > 1 and not cfg.enable_lora \
                and pc.prefill_context_parallel_size == 1:
            from ..parallel import fused_linear
            fused_linear.attach(self.runner.model, cfg, self.device)

    def determine_num_blocks(self) -> int:
        """Blocks that fit next to weights and peak activations; every rank must agree."""
        n = self.runner.determine_num_blocks()
        if self.world_size > 1:
            n = min(pstate.get_world_group().all_gather_object(n))
        return n

    def determine_available_memory(self) -> int:
        return self.determine_num_blocks() * self.runner.kv_bytes_per_block()

    def initialize_cache(self, num_blocks: int) -> None:
        self.num_blocks = num_blocks
        with self._pool("kv_cache"):
            self.runner.init_kv_cache(num_blocks)

    def compile_or_warm_up_model(self) -> None:
        self.runner.warmup()
        if envs.VLLM_B200_TP_COMM == "auto" and getattr(self.runner.model, "sp_ctx", None) is not None:
            from ..parallel import fused_linear
            try:
                self.tp_comm_calibration = fused_linear.calibrate(self.runner, pstate.get_tp_group())
            except Exception as e:          # calibration is an optimisation: keep the fused default
                logger.warning("TP communication calibration failed: %s", e)
            logger.info("TP communication path per step class: %s", self.tp_comm_calibration)

    def capture_model(self) -> None:
        self.runner.capture_graphs()

    # ------------------------------------------------------------------ stepping
    def execute_model(self, scheduler_output) -> dict:
        return self.runner.execute(scheduler_output)

    def execute_dummy_batch(self) -> None:
        self.runner.execute_dummy()

    def profile_prefill_latency(self, lengths=(256, 512, 1024, 2048), repeats: int = 2) -> list[tuple[int, float]]:
        """(chunk length, seconds) samples for the chunk-size predictor of the profiling
        scheduler (worker.py:830-891)."""
        out = []
        for n in lengths:
            n = min(n, self.runner.max_tokens, self.runner.max_model_len - 1)
            best = float("inf")
            for _ in range(repeats):
                meta, T, Tp, _, _ = self.runner._dummy_meta(1, n)
                meta.slot_mapping.fill_(-1)
                if self.device.type == "cuda":
                    torch.cuda.synchronize()
                t0 = time.perf_counter()
                with torch.inference_mode():
                    self.runner._forward(Tp, meta)
                if self.device.type == "cuda":
                    torch.cuda.synchronize()
                best = min(best, time.perf_counter() - t0)
            out.append((n, best))
        return out

    # ------------------------------------------------------------------ RL: sleep / weights
    def start_weight_update(self) -> None:
        if self._weight_update_state != "idle":
            raise RuntimeError(f"weight update already {self._weight_update_state}")
        self._weight_update_state = "updating"

    def update_weights(self, named_tensors) -> int:
        """Copy new values into the live parameters (same shapes, any device)."""
        if self._weight_update_state != "updating":
            raise RuntimeError("call start_weight_update() first")
        loaded = self.runner.model.load_weights(named_tensors)
        self._updated_names = getattr(self, "_updated_names", set()) | set(loaded)
        return len(loaded)

    def finish_weight_update(self) -> None:
        if self._weight_update_state != "updating":
            raise RuntimeError("no weight update in progress")
        self._weight_update_state = "idle"
        names, self._updated_names = getattr(self, "_updated_names", set()), set()
        model = self.runner.model
        if getattr(model, "norm_folded", False):
            # a norm weight lives inside the GEMM weight that follows it: both must arrive together
            for L in model.layers:
                p = f"model.layers.{L.idx}"
                for norm, parts in ((f"{p}.input_layernorm.weight", ("q_proj", "k_proj", "v_proj", "qkv_proj")),
                                    (f"{p}.post_attention_layernorm.weight", ("gate_proj", "up_proj", "gate_up_proj"))):
                    got_w = any(f".{x}.weight" in n and n.startswith(p + ".") for n in names for x in parts)
                    if got_w != (norm in names):
                        raise RuntimeError(f"weight update of layer {L.idx} replaced a projection without its "
                                           "norm weight (or the reverse); with folded norms send both")
            from ..models.folded import fold_norms
            fold_norms(model)
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    # ------------------------------------------------------------------ profiling / health
    def profile(self, is_start: bool = True, out_dir: Optional[str] = None) -> Optional[str]:
        from ..profiler.torch_profiler import TorchProfilerSession
        if is_start:
            if self._profiler is not None:
                raise RuntimeError("profiler already running")
            self._profiler = TorchProfilerSession(out_dir or envs.VLLM_B200_LOG_PATH or ".", self.rank or 0)
            self._profiler.start()
            return None
        if self._profiler is None:
            raise RuntimeError("profiler is not running")
        path = self._profiler.stop()
        self._profiler = None
        return path

    def check_health(self) -> None:
        """Raises when a kernel reported a timeout / bad index, or when NVML reports the GPU
        lost or with uncorrectable errors (worker.py:1083-1106 asks the vendor tool)."""
        if self.device is None or self.device.type != "cuda":
            return
        _native.check_status(self.device)
        from ..observability.health import gpu_health
        h = gpu_health(self.device.index or 0)
        if not h["ok"]:
            raise RuntimeError(f"GPU {self.device.index} unhealthy: {h['reason']}")

    # ------------------------------------------------------------------ LoRA passthroughs
    def add_lora(self, lora_request) -> bool:
        return self.runner.lora_manager.add(lora_request) if getattr(self.runner, "lora_manager", None) else False

    def remove_lora(self, lora_id: int) -> bool:
        return self.runner.lora_manager.remove(lora_id) if getattr(self.runner, "lora_manager", None) else False

    def list_loras(self) -> set:
        return self.runner.lora_manager.list() if getattr(self.runner, "lora_manager", None) else set()

    def pin_lora(self, lora_id: int) -> bool:
        return self.runner.lora_manager.pin(lora_id) if getattr(self.runner, "lora_manager", None) else False

    def shutdown(self) -> None:
        if self.device is not None and self.device.type == "cuda":
            torch.cuda.synchronize()
