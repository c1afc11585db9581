"""Worker that upstream vLLM's executors construct when this package is the active platform.

``vllm.LLM`` / ``vllm serve`` stay the entry points: vLLM's engine core, scheduler and KV-cache
manager run unchanged and drive this class through the ``WorkerBase`` surface
(init_device -> load_model -> get_kv_cache_spec -> determine_available_memory ->
initialize_from_config -> compile_or_warm_up_model -> execute_model / sample_tokens).  Inside, the
device, the process groups, the model, the paged KV cache, the CUDA graphs and every kernel are this
package's: the class hosts a ``B200Worker`` and translates vLLM's per-step ``SchedulerOutput``
(new / cached / finished / preempted requests, block ids chosen by vLLM's block pool, token counts)
into the runner's own step description, and the sampled tokens back into a ``ModelRunnerOutput``.

Role of ``NPUWorker(WorkerBase)`` + ``NPUModelRunner`` (vllm_ascend/worker/worker.py:98-187,
625-695; vllm_ascend/worker/model_runner_v1.py:291).  The reference subclasses vLLM's GPU runner
and patches it; here the runner is independent of vLLM's, so the adapter is the only code that
knows both vocabularies.

Both of vLLM's stepping modes are served.  Synchronous: ``execute_model`` enqueues the step and
``sample_tokens`` waits for it.  Asynchronous scheduling: ``sample_tokens`` returns a handle whose
``get_output`` waits, so vLLM schedules step N+1 while step N runs; the token a request is still
sampling is forwarded on the device from step N's output into step N+1's input ids.
"""
from __future__ import annotations

import os
from typing import Any, Optional

import numpy as np
import torch

from ..config import (CacheConfig, CompilationConfig, EngineConfig, ModelConfig, ParallelConfig,
                      SchedulerConfig)
from ..engine.request import Request, RequestStatus, SamplingParams
from ..engine.scheduler import SchedulerOutput as StepPlan
from ..logger import logger

try:
    from vllm.v1.worker.worker_base import WorkerBase as _WorkerBase
    _HAVE_VLLM = True
except Exception:          # pragma: no cover - only without vLLM installed
    _HAVE_VLLM = False

    class _WorkerBase:      # type: ignore
        def __init__(self, vllm_config, local_rank, rank, distributed_init_method, is_driver_worker=False):
            self.vllm_config = vllm_config
            self.local_rank, self.rank = local_rank, rank
            self.distributed_init_method = distributed_init_method
            self.is_driver_worker = is_driver_worker


def engine_config_from_vllm(vllm_config: Any, device: str) -> EngineConfig:
    """The part of a ``VllmConfig`` this runtime honours, as an ``EngineConfig``."""
    mc, cc, sc, pc = (vllm_config.model_config, vllm_config.cache_config, vllm_config.scheduler_config,
                      vllm_config.parallel_config)
    hf = mc.hf_config.to_dict() if hasattr(mc.hf_config, "to_dict") else dict(mc.hf_config)
    if "text_config" in hf and isinstance(hf["text_config"], dict) and "hidden_size" not in hf:
        hf = {**hf["text_config"], **{k: v for k, v in hf.items() if k != "text_config"}}
    dtype = str(mc.dtype).replace("torch.", "")
    model = ModelConfig.from_hf_dict(hf, dtype=dtype)
    load_format = str(getattr(vllm_config.load_config, "load_format", "auto"))
    if load_format != "dummy" and os.path.isdir(str(mc.model)):
        model.model_path = str(mc.model)
    model.name = os.path.basename(os.path.normpath(str(mc.model)))
    model.seed = int(mc.seed or 0)
    comp = vllm_config.compilation_config
    mode = getattr(getattr(comp, "cudagraph_mode", None), "name", "FULL_DECODE_ONLY")
    eager = bool(getattr(mc, "enforce_eager", False)) or mode == "NONE"
    sizes = list(getattr(comp, "cudagraph_capture_sizes", None) or []) or None
    cfg = EngineConfig(
        model=model,
        cache=CacheConfig(block_size=int(cc.block_size), gpu_memory_utilization=float(cc.gpu_memory_utilization),
                          enable_prefix_caching=False),     # vLLM's block pool owns prefix caching
        scheduler=SchedulerConfig(max_num_seqs=int(sc.max_num_seqs),
                                  max_num_batched_tokens=int(sc.max_num_batched_tokens),
                                  max_model_len=int(mc.max_model_len)),
        parallel=ParallelConfig(tensor_parallel_size=int(pc.tensor_parallel_size),
                                pipeline_parallel_size=int(pc.pipeline_parallel_size),
                                enable_expert_parallel=bool(getattr(pc, "enable_expert_parallel", False))),
        compilation=CompilationConfig(cudagraph_mode="NONE" if eager else "FULL_DECODE_ONLY",
                                      cudagraph_capture_sizes=sizes),
        additional_config=dict(getattr(vllm_config, "additional_config", None) or {}),
        device=device, seed=int(mc.seed or 0), load_format="auto",
        enable_sleep_mode=bool(getattr(mc, "enable_sleep_mode", False)))
    if device == "cuda":
        cfg.scheduler.decode_batch_alignment = 256
    cfg.async_scheduling = False          # vLLM's scheduler decides; the adapter serves both modes
    return cfg


def to_sampling_params(sp: Any) -> SamplingParams:
    """vLLM ``SamplingParams`` -> this package's.  Stop strings, stop tokens and max_tokens are
    enforced by vLLM's scheduler; the worker only needs what shapes the distribution."""
    if sp is None:
        return SamplingParams(temperature=0.0, max_tokens=1 << 30)
    bad = getattr(sp, "_bad_words_token_ids", None) or getattr(sp, "bad_words_token_ids", None)
    stops = list(getattr(sp, "all_stop_token_ids", None) or getattr(sp, "stop_token_ids", None) or [])
    return SamplingParams(
        temperature=float(sp.temperature), top_p=float(sp.top_p), top_k=int(sp.top_k or 0),
        min_p=float(getattr(sp, "min_p", 0.0) or 0.0),
        presence_penalty=float(sp.presence_penalty), frequency_penalty=float(sp.frequency_penalty),
        repetition_penalty=float(sp.repetition_penalty), max_tokens=int(sp.max_tokens or (1 << 30)),
        min_tokens=int(getattr(sp, "min_tokens", 0) or 0), stop_token_ids=stops or None,
        ignore_eos=True,                  # the scheduler of the host checks EOS / stops
        seed=getattr(sp, "seed", None),
        logprobs=getattr(sp, "logprobs", None),
        logit_bias=dict(sp.logit_bias) if getattr(sp, "logit_bias", None) else None,
        allowed_token_ids=list(sp.allowed_token_ids) if getattr(sp, "allowed_token_ids", None) else None,
        bad_words_token_ids=[list(w) for w in bad] if bad else None)


class _AsyncStepOutput:
    """What ``sample_tokens`` returns under asynchronous scheduling: ``get_output`` blocks until the
    step's tokens are on the host (vllm/v1/outputs.py ``AsyncModelRunnerOutput`` contract)."""

    def __init__(self, worker: "B200VllmWorker", pending):
        self._worker, self._pending = worker, pending

    def get_output(self):
        return self._worker._finish(self._pending)


if _HAVE_VLLM:
    from vllm.v1.outputs import AsyncModelRunnerOutput as _AsyncBase

    class _AsyncStepOutput(_AsyncStepOutput, _AsyncBase):   # type: ignore[no-redef]
        pass


class B200VllmWorker(_WorkerBase):
    def __init__(self, vllm_config, local_rank: int, rank: int, distributed_init_method: str,
                 is_driver_worker: bool = False, **unused):
        super().__init__(vllm_config=vllm_config, local_rank=local_rank, rank=rank,
                         distributed_init_method=distributed_init_method, is_driver_worker=is_driver_worker)
        self.inner = None                      # B200Worker
        self.runner = None
        self.reqs: dict[str, Request] = {}
        self._free_rows: list[int] = []
        self._pending = None                   # (handle, plan, order) enqueued by execute_model
        self._uncollected = None               # handle of the newest step whose tokens were not read yet
        self._async = bool(getattr(vllm_config.scheduler_config, "async_scheduling", False))
        self.stats = {"steps": 0, "resumed": 0, "preempted": 0}

    # ------------------------------------------------------------------ set-up
    def init_device(self) -> None:
        from .worker import B200Worker
        device = "cuda" if torch.cuda.is_available() else "cpu"
        pc = self.vllm_config.parallel_config
        world = int(pc.world_size) if hasattr(pc, "world_size") else 1
        if world > 1:
            # ranks spawned by a vLLM executor get their identity as arguments; the process group
            # is joined from torchrun-style variables
            os.environ.setdefault("RANK", str(self.rank))
            os.environ.setdefault("LOCAL_RANK", str(self.local_rank))
            os.environ.setdefault("WORLD_SIZE", str(world))
            m = str(self.distributed_init_method or "")
            if m.startswith("tcp://"):
                host, port = m[len("tcp://"):].rsplit(":", 1)
                os.environ.setdefault("MASTER_ADDR", host.strip("[]"))
                os.environ.setdefault("MASTER_PORT", port)
        cfg = engine_config_from_vllm(self.vllm_config, device)
        if device == "cuda" and world == 1:
            cfg.device_index = int(self.local_rank)
        from ..platform_config import check_and_update_config
        check_and_update_config(cfg)
        self.cfg = cfg
        self.inner = B200Worker(cfg, local_rank=self.local_rank, rank=self.rank,
                                distributed_init_method=self.distributed_init_method,
                                is_driver_worker=self.is_driver_worker)
        self.inner.init_device()
        self.device = self.inner.device
        self.runner = self.model_runner = self.inner.runner
        self._free_rows = list(range(cfg.scheduler.max_num_seqs - 1, -1, -1))

    def load_model(self, *, load_dummy_weights: bool = False) -> None:
        self.inner.load_model()

    def get_model(self):
        return self.runner.model

    def update_max_model_len(self, max_model_len: int) -> None:
        self.cfg.scheduler.max_model_len = int(max_model_len)

    def get_supported_tasks(self) -> tuple:
        return ("generate",)

    # ------------------------------------------------------------------ KV cache
    def get_kv_cache_spec(self) -> dict:
        """One spec per attention layer, in vLLM's terms: vLLM sizes the pool (number of blocks) from
        these; the cache tensors themselves are allocated by this package's runner."""
        from vllm.v1.kv_cache_interface import FullAttentionSpec
        m, r = self.cfg.model, self.runner
        if m.is_hybrid:
            raise NotImplementedError("hybrid linear-attention models run on the standalone engine "
                                      "(vllm_ascend_b200.LLM), not yet under a host vLLM")
        bs = self.cfg.cache.block_size
        specs = {}
        if m.use_mla:
            from vllm.v1.kv_cache_interface import MLAAttentionSpec
            width = m.kv_lora_rank + m.qk_rope_head_dim
            mk = lambda: MLAAttentionSpec(block_size=bs, num_kv_heads=1, head_size=width, dtype=r.kv_dtype)
        else:
            a = r._attn_layer()
            mk = lambda: FullAttentionSpec(block_size=bs, num_kv_heads=int(a.Hkv), head_size=int(a.D),
                                           dtype=r.kv_dtype)
        for i in range(m.num_hidden_layers):
            specs[f"model.layers.{i}.self_attn.attn"] = mk()
        self._spec_page_bytes = next(iter(specs.values())).page_size_bytes * len(specs)
        return specs

    def get_cache_block_size_bytes(self) -> int:
        return int(self.runner.kv_bytes_per_block())

    def determine_available_memory(self) -> int:
        """Bytes vLLM may hand to the KV cache.  Expressed in vLLM's page size so that the block
        count it derives is the one this runner would have chosen."""
        n = self.inner.determine_num_blocks()
        per_block = getattr(self, "_spec_page_bytes", None) or self.runner.kv_bytes_per_block()
        return int(n) * int(per_block)

    def initialize_from_config(self, kv_cache_config) -> None:
        cfgs = kv_cache_config if isinstance(kv_cache_config, (list, tuple)) else [kv_cache_config]
        num_blocks = int(cfgs[0].num_blocks)
        self.inner.initialize_cache(num_blocks)

    def initialize_cache(self, num_gpu_blocks: int, num_cpu_blocks: int = 0) -> None:
        self.vllm_config.cache_config.num_gpu_blocks = num_gpu_blocks
        self.vllm_config.cache_config.num_cpu_blocks = num_cpu_blocks

    def compile_or_warm_up_model(self):
        self.inner.compile_or_warm_up_model()
        self.inner.capture_model()
        try:
            from vllm.v1.worker.worker_base import CompilationTimes
            return CompilationTimes(0.0, 0.0)
        except Exception:
            return 0.0

    # ------------------------------------------------------------------ per-step translation
    def _take_row(self, req: Request) -> None:
        if req.row < 0:
            if not self._free_rows:
                raise RuntimeError("more concurrent requests than max_num_seqs rows")
            req.row = self._free_rows.pop()

    def _drop(self, rid: str) -> None:
        req = self.reqs.pop(rid, None)
        if req is not None and req.row >= 0:
            self._free_rows.append(req.row)
            req.row = -1

    def _update_states(self, so) -> list:
        """Mirror vLLM's request bookkeeping; returns the requests whose block lists changed."""
        for rid in so.finished_req_ids:
            self._drop(rid)
        for rid in (so.preempted_req_ids or ()):
            req = self.reqs.get(rid)
            if req is not None:           # the blocks are gone; the row is kept for the resume
                req.block_ids = []
                req.num_computed_tokens = 0
                req.num_inflight = 0
                self.stats["preempted"] += 1
        changed = []
        for nr in so.scheduled_new_reqs:
            # a request that resumes after a preemption arrives here again with every token it had
            # (``prefill_token_ids`` = prompt + generated so far)
            every = getattr(nr, "prefill_token_ids", None) or nr.prompt_token_ids
            prompt = nr.prompt_token_ids if nr.prompt_token_ids is not None else every
            if getattr(nr, "mm_features", None):
                raise NotImplementedError("multimodal requests run on the standalone engine")
            mm_items = []
            embeds = getattr(nr, "prompt_embeds", None)
            if embeds is not None:
                # the caller supplied input embeddings: placeholder ids, rows merged in like encoder outputs
                from ..multimodal.inputs import MMInput
                pe = torch.as_tensor(embeds)
                if pe.dim() != 2 or pe.shape[1] != self.runner.mcfg.hidden_size:
                    raise ValueError(f"prompt_embeds must be [num_tokens, {self.runner.mcfg.hidden_size}]")
                if self.runner.mm is None:
                    from ..engine.mm_runner import MultimodalState
                    self.runner.mm = MultimodalState(self.runner)
                n_emb = pe.shape[0]
                mm_items = [MMInput("embeds", 0, n_emb, (0, 0, 0), None, f"embeds-{nr.req_id}", embeds=pe)]
                tail = [int(t) for t in (every[n_emb:] if every is not None else [])]
                prompt = [0] * n_emb
                every = prompt + tail
            if every is None:
                raise ValueError(f"request {nr.req_id} carries neither token ids nor embeddings")
            old = self.reqs.pop(nr.req_id, None)
            req = Request(nr.req_id, np.asarray(prompt, dtype=np.int32), to_sampling_params(nr.sampling_params),
                          lora_request=nr.lora_request, mm_inputs=mm_items)
            if old is not None:
                req.row = old.row
                self.runner.row_owner[req.row] = None      # the row's cached ids are rebuilt
                self.stats["resumed"] += 1
            vsp = nr.sampling_params
            # structured outputs: the host computes a token bitmask per step after scheduling; steps of
            # such requests sample only once the bitmask has arrived (sample_tokens)
            req.structured = vsp is not None and (getattr(vsp, "structured_outputs", None) is not None
                                                   or getattr(vsp, "guided_decoding", None) is not None)
            req.status = RequestStatus.RUNNING
            req.block_ids = list(nr.block_ids[0])
            req.num_computed_tokens = int(nr.num_computed_tokens)
            req.output_token_ids = [int(t) for t in every[len(prompt):]]
            req.num_output_tokens = len(req.output_token_ids)
            self._take_row(req)
            self.reqs[nr.req_id] = req
            changed.append(req)
        cached = so.scheduled_cached_reqs
        for i, rid in enumerate(cached.req_ids):
            req = self.reqs[rid]
            resumed = rid in cached.resumed_req_ids
            new_blocks = cached.new_block_ids[i]
            if resumed:
                self.stats["resumed"] += 1
                req.block_ids = list(new_blocks[0]) if new_blocks is not None else []
                toks = cached.all_token_ids.get(rid)
                if toks is not None:
                    n_prompt = req.num_prompt_tokens
                    req.output_token_ids = [int(t) for t in toks[n_prompt:]]
                    req.num_output_tokens = len(req.output_token_ids)
                # the row's cached token ids / block list are rebuilt from the request
                self.runner.row_owner[req.row] = None
                changed.append(req)
            elif new_blocks is not None and new_blocks[0]:
                req.block_ids.extend(new_blocks[0])
                changed.append(req)
            if cached.new_token_ids and i < len(cached.new_token_ids) and cached.new_token_ids[i]:
                # tokens the host already knows and this worker has not produced itself
                # (pipeline parallelism: sampled on the last stage)
                known = req.num_prompt_tokens + req.num_output_tokens
                want = int(cached.num_computed_tokens[i]) + int(so.num_scheduled_tokens[rid])
                for t in cached.new_token_ids[i][max(0, known - want):] if known < want else ():
                    req.output_token_ids.append(int(t))
                    req.num_output_tokens += 1
            req.num_computed_tokens = int(cached.num_computed_tokens[i])
        return changed

    def _plan(self, so) -> tuple:
        changed = self._update_states(so)
        decodes, prefills = [], []
        for rid, n in so.num_scheduled_tokens.items():
            req = self.reqs[rid]
            spec = so.scheduled_spec_decode_tokens.get(rid) if so.scheduled_spec_decode_tokens else None
            req.spec_token_ids = [int(t) for t in spec] if spec else []
            (decodes if (n == 1 and req.num_computed_tokens > 0) else prefills).append((req, int(n)))
        plan = StepPlan(scheduled=decodes + prefills)
        plan.num_scheduled_tokens = int(so.total_num_scheduled_tokens)
        plan.new_block_rows = changed
        self.stats["steps"] += 1
        plan.step_id = self.stats["steps"]
        order = list(so.num_scheduled_tokens.keys())
        return plan, order

    # ------------------------------------------------------------------ stepping
    @torch.inference_mode()
    def execute_model(self, scheduler_output):
        so = scheduler_output
        if so.total_num_scheduled_tokens == 0:
            self._update_states(so)
            from vllm.v1.outputs import EMPTY_MODEL_RUNNER_OUTPUT
            return EMPTY_MODEL_RUNNER_OUTPUT
        plan, order = self._plan(so)
        defer = any(getattr(r, "structured", False) for r, _ in plan.scheduled)
        handle = self.runner.execute_async(plan, self._uncollected, defer_sampling=defer)
        # account for the step at launch (the runner's own scheduler does the same): a request whose
        # step samples has one more token in flight until the step is collected
        for req, n in plan.scheduled:
            if req.num_computed_tokens + n >= req.num_tokens + req.num_inflight:
                req.num_inflight += 1
        if handle is not None and handle.tokens is not None:
            self._uncollected = handle
        self._pending = (handle, plan, order)
        return None

    def sample_tokens(self, grammar_output=None):
        pending, self._pending = self._pending, None
        if pending is None:
            return None
        handle = pending[0]
        bitmask = getattr(grammar_output, "grammar_bitmask", None) if grammar_output is not None else None
        if handle is not None and handle.h_sel is not None:
            # the forward pass ran without sampling: apply the host's grammar bitmask (bit t of word
            # t // 32 set = token t allowed) to the rows of the structured requests, then sample
            allowed = None
            if bitmask is not None:
                allowed = self._unpack_bitmask(grammar_output.structured_output_request_ids, bitmask)
            self.runner.finish_sampling(handle, allowed)
            if handle.tokens is not None:
                self._uncollected = handle
        elif bitmask is not None and len(grammar_output.structured_output_request_ids):
            raise RuntimeError("a grammar bitmask arrived for a step that was sampled without it")
        if self._async:
            return _AsyncStepOutput(self, pending)
        return self._finish(pending)

    def _unpack_bitmask(self, req_ids, bitmask) -> dict:
        vocab = self.runner.mcfg.vocab_size
        bm = torch.from_numpy(np.ascontiguousarray(bitmask)).to(torch.int32)
        if self.device is not None and self.device.type == "cuda":
            bm = bm.to(self.device, non_blocking=True)
        shifts = torch.arange(32, dtype=torch.int32, device=bm.device)
        bits = ((bm.unsqueeze(-1) >> shifts) & 1).bool().reshape(bm.shape[0], -1)
        if bits.shape[1] < vocab:                # tokens beyond the grammar's vocabulary are not allowed
            bits = torch.nn.functional.pad(bits, (0, vocab - bits.shape[1]))
        return {rid: bits[i, :vocab] for i, rid in enumerate(req_ids)}

    def _finish(self, pending):
        from vllm.v1.outputs import ModelRunnerOutput
        handle, plan, order = pending
        dev_lp = getattr(handle, "logprobs", None) if handle is not None else None
        sampled = self.runner.collect(handle) if handle is not None else {}
        lp_lists = self._logprobs_lists(handle, dev_lp, order, sampled) if dev_lp is not None else None
        self.runner.take_logprobs()           # the per-request dictionaries are the own engine's format
        if handle is self._uncollected:
            self._uncollected = None
        from .. import _native
        if self.device is not None and self.device.type == "cuda" and (self.stats["steps"] & 63) == 0:
            _native.check_status(self.device)
        for req, _ in plan.scheduled:
            toks = sampled.get(req.request_id)
            if toks:
                req.num_inflight = max(0, req.num_inflight - 1)
                if self.reqs.get(req.request_id) is req:
                    req.output_token_ids.extend(int(t) for t in toks)
                    req.num_output_tokens += len(toks)
                req.spec_token_ids = []
        out_tokens = [[int(t) for t in (sampled.get(rid) or ())] for rid in order]
        return ModelRunnerOutput(req_ids=order, req_id_to_index={rid: i for i, rid in enumerate(order)},
                                 sampled_token_ids=out_tokens, logprobs=lp_lists, prompt_logprobs_dict={},
                                 pooler_output=None)

    @staticmethod
    def _logprobs_lists(handle, dev_lp, order, sampled):
        """Log-probabilities of the step in vLLM's layout: per generated token one row holding the
        sampled token followed by the top-k tokens, their log-probabilities, and the sampled
        token's rank (exact while it is among the top-k, else k + 1)."""
        from vllm.v1.outputs import LogprobsLists
        tok_lp, ids, vals = (t.float().cpu().numpy() if t.is_floating_point() else t.cpu().numpy() for t in dev_lp)
        k = ids.shape[1]
        row_of = {r.request_id: i for i, r in enumerate(handle.reqs)}
        out_ids, out_lp, ranks, cu = [], [], [], [0]
        for rid in order:
            toks = sampled.get(rid)
            i = row_of.get(rid)
            if toks and i is not None:
                out_ids.append([int(toks[0])] + [int(x) for x in ids[i]])
                out_lp.append([float(tok_lp[i])] + [float(x) for x in vals[i]])
                ranks.append(1 + int((vals[i] > tok_lp[i]).sum()))
            cu.append(len(out_ids))
        return LogprobsLists(np.asarray(out_ids, dtype=np.int32).reshape(-1, k + 1),
                             np.asarray(out_lp, dtype=np.float32).reshape(-1, k + 1),
                             np.asarray(ranks, dtype=np.int32), cu[:-1])

    def take_draft_token_ids(self):
        return None

    def execute_dummy_batch(self) -> None:
        self.inner.execute_dummy_batch()

    # ------------------------------------------------------------------ lifecycle passthroughs
    def _engine_view(self):
        """The handful of attributes ``device_allocator.sleep`` reads from an engine."""
        from types import SimpleNamespace
        if getattr(self, "_view", None) is None:
            self._view = SimpleNamespace(
                cfg=self.cfg, runner=self.runner, sleep_level=0,
                scheduler=SimpleNamespace(pool=SimpleNamespace(reset_prefix_cache=lambda: True)))
        return self._view

    def sleep(self, level: int = 1) -> None:
        from ..device_allocator.sleep import sleep
        sleep(self._engine_view(), level)

    def wake_up(self, tags: Optional[list] = None) -> None:
        from ..device_allocator.sleep import wake_up
        wake_up(self._engine_view(), tags)

    def profile(self, is_start: bool = True, profile_prefix: Optional[str] = None):
        return self.inner.profile(is_start)

    def check_health(self) -> None:
        self.inner.check_health()

    def add_lora(self, lora_request) -> bool:
        return self.inner.add_lora(lora_request)

    def remove_lora(self, lora_id: int) -> bool:
        return self.inner.remove_lora(lora_id)

    def pin_lora(self, lora_id: int) -> bool:
        return self.inner.pin_lora(lora_id)

    def list_loras(self) -> set:
        return self.inner.list_loras()

    def reset_mm_cache(self) -> None:
        return None

    def reset_encoder_cache(self) -> None:
        return None

    def get_kv_connector_handshake_metadata(self):
        return None

    def save_sharded_state(self, path: str, pattern: Optional[str] = None, max_size: Optional[int] = None) -> None:
        from ..model_loader.sharded_state import save_sharded_state
        save_sharded_state(self.runner.model, path, int(self.rank), max_size or (5 << 30))

    def shutdown(self) -> None:
        if self.runner is not None:
            try:
                if self.device is not None and self.device.type == "cuda":
                    torch.cuda.synchronize()
                self.runner.drop_graphs()
            except Exception as e:      # teardown must not mask the caller's error
                logger.debug("shutdown: %s", e)
