"""Public offline entry point: ``LLM(...).generate(prompts, sampling_params)``.

The class keeps the upstream vLLM ``LLM`` call shape (the reference exposes no
entry point of its own; its users call ``vllm.LLM`` / ``vllm serve``).  One
process drives one GPU; under ``torchrun`` every rank constructs the same ``LLM``
and calls ``generate`` with the same prompts (SPMD), the ranks meeting in the
model's collectives.
"""
from __future__ import annotations

import itertools
import time
from typing import Optional, Sequence, Union

import numpy as np
import torch

from .. import _native, envs
from ..config import (CacheConfig, CompilationConfig, EngineConfig, ModelConfig, ParallelConfig,
                      SchedulerConfig, get_model_config)
from ..parallel import state as pstate
from .model_runner import ModelRunner
from .request import (CompletionOutput, Request, RequestMetrics, RequestOutput, RequestStatus,
                      SamplingParams)
from .scheduler import Scheduler

_FINISH_REASON = {RequestStatus.FINISHED_STOPPED: "stop", RequestStatus.FINISHED_LENGTH: "length",
                  RequestStatus.FINISHED_ABORTED: "abort"}


class LLMEngine:
    def __init__(self, cfg: EngineConfig):
        self.cfg = cfg
        from ..worker.worker import B200Worker
        self.worker = B200Worker(cfg)
        self.worker.init_device()
        pc = cfg.parallel
        world = self.worker.world_size
        self.device = self.worker.device
        self.runner = self.worker.runner
        self.dp = pstate.get_dp_group()
        self.sleep_level = 0
        self.worker.load_model()
        self.moe_runtime = self.worker.moe_runtime
        num_blocks = self.worker.determine_num_blocks()
        self.worker.initialize_cache(num_blocks)
        self.worker.compile_or_warm_up_model()
        self.eplb = None
        from ..platform_config import get_b200_config
        ecfg = get_b200_config().eplb_config
        if cfg.model.is_moe and pc.enable_expert_parallel and world > 1 and \
                (ecfg.dynamic_eplb or ecfg.expert_map_path or ecfg.num_redundant_experts):
            from ..eplb.updater import EplbAdaptor, EplbUpdater
            self.eplb = EplbUpdater(EplbAdaptor(self.runner.model, pstate.get_ep_group(),
                                                ecfg.num_redundant_experts), ecfg)
        self.kv_connector = None
        if cfg.kv_transfer_config:
            from ..distributed.kv_transfer import create_connector
            self.kv_connector = create_connector(cfg, self.runner)
        if cfg.ec_transfer_config and self.runner.mm is not None:
            from ..distributed.ec_transfer import create_ec_connector
            self.runner.mm.ec_connector = create_ec_connector(cfg.ec_transfer_config)
        self.scheduler = self._make_scheduler(num_blocks)
        if cfg.enable_lora:
            self.scheduler.max_loras = cfg.max_loras
        if cfg.speculative_config:
            from ..spec_decode import get_spec_decode_method
            self.runner.proposer = get_spec_decode_method(cfg.speculative_config, self.runner)
            self.scheduler.spec_slack = int(cfg.speculative_config.get("num_speculative_tokens", 3))
            dsc = get_b200_config().dynamic_spec_config
            if dsc.method:
                from ..spec_decode.dynamic import DynamicSpecController
                self.runner.dynamic_spec = DynamicSpecController(self.scheduler.spec_slack, dsc.method_params)
        self._model_proposer = hasattr(self.runner.proposer, "propose_step")
        # asynchronous scheduling needs nothing between two steps that depends on the sampled
        # token values: no proposer, no connector bookkeeping, no lock-step groups
        self._inflight = None
        self._sync_reqs: set = set()
        self.guided = None                 # sample.guided.GuidedDecodingManager once a vocabulary is set
        want_async = cfg.async_scheduling if cfg.async_scheduling is not None else (cfg.device == "cuda")
        # (TP ranks take identical decisions from identical tokens, so they stay in lock-step;
        # DP / PP engines exchange host-side state every step and run synchronously)
        self.async_scheduling = bool(want_async and self.runner.proposer is None and self.kv_connector is None
                                     and self.eplb is None and self.dp.world_size == 1
                                     and pc.pipeline_parallel_size == 1
                                     and pc.prefill_context_parallel_size == 1)
        self.runner.capture_graphs()
        self._req_counter = itertools.count()
        self.eos_token_id: Optional[int] = None
        self.step_times: list[float] = []
        self.host_times = {"schedule": 0.0, "execute": 0.0, "update": 0.0}
        # schedulers that learn from step durations (profiling chunk): start-up profile + online samples
        self._record_step = None
        if hasattr(self.scheduler, "run_profiling"):
            # Every rank of a replica runs its own copy of the scheduler and all copies must decide alike, so
            # a duration is agreed on (the slowest rank's) before the predictor sees it.
            from ..parallel import state as _ps
            groups = [g for g in (_ps.get_tp_group(), _ps.get_pp_group()) if g.world_size > 1]

            def agreed(seconds: float) -> float:
                for g in groups:
                    seconds = max(g.all_gather_object(float(seconds)))
                return seconds
            if getattr(self.scheduler, "need_timing", True):
                self._record_step = lambda so, sec: self.scheduler.record_step(so, agreed(sec))
            if cfg.parallel.data_parallel_size == 1:
                # pipeline stages take part too: the dummy forward passes activations from stage to stage
                self.scheduler.run_profiling(lambda n: agreed(self.runner.profile_prefill_latency(n)))

    def _make_scheduler(self, num_blocks: int) -> Scheduler:
        from ..core import make_scheduler
        return make_scheduler(self.cfg, num_blocks, self.kv_connector)

    # ------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], sampling_params: SamplingParams,
                    request_id: Optional[str] = None, kv_transfer_params: Optional[dict] = None,
                    job_id: Optional[str] = None, lora_request=None,
                    multi_modal_data: Optional[dict] = None, prompt_embeds=None) -> str:
        if request_id:
            rid = request_id
        elif self.dp.world_size > 1:
            # unique across replicas: a request may move to another replica (load balancing)
            rid = f"req-d{self.dp.rank_in_group}-{next(self._req_counter)}"
        else:
            rid = f"req-{next(self._req_counter)}"
        sampling_params.validate_for_vocab(self.cfg.model.vocab_size)
        if lora_request is not None and self.runner.lora_manager is None:
            raise ValueError("a LoRA request needs an engine built with enable_lora=True")
        mm_items, mrope, delta = [], None, 0
        mcfg = self.cfg.model
        if multi_modal_data:
            if not mcfg.is_multimodal:
                raise ValueError(f"{mcfg.architecture} takes no multimodal inputs")
            from ..multimodal import build_mm_request, mrope_positions
            from ..models.vision import VisionConfig
            prompt_token_ids, mm_items = build_mm_request(prompt_token_ids, multi_modal_data, mcfg)
            if mcfg.mrope_section:
                mrope, delta = mrope_positions(prompt_token_ids, mm_items,
                                               VisionConfig.from_hf(mcfg.vision_config).spatial_merge_size,
                                               mcfg.tokens_per_second)
        if prompt_embeds is not None:
            # the caller supplies the input embeddings: the ids are placeholders, the rows are merged in
            # the way encoder outputs are
            from ..multimodal.inputs import MMInput
            pe = torch.as_tensor(prompt_embeds)
            if pe.dim() != 2 or pe.shape[1] != mcfg.hidden_size:
                raise ValueError(f"prompt_embeds must be [num_tokens, {mcfg.hidden_size}]")
            if self.runner.mm is None:
                from .mm_runner import MultimodalState
                self.runner.mm = MultimodalState(self.runner)
            prompt_token_ids = [0] * pe.shape[0]
            mm_items = [MMInput("embeds", 0, pe.shape[0], (0, 0, 0), None, f"embeds-{rid}", embeds=pe)]
        req = Request(rid, np.asarray(prompt_token_ids, dtype=np.int32), sampling_params,
                      eos_token_id=self.eos_token_id, kv_transfer_params=kv_transfer_params,
                      job_id=job_id, lora_request=lora_request, mm_inputs=mm_items,
                      mrope_positions=mrope, mrope_delta=delta)
        sp_ = sampling_params
        if sp_.prompt_logprobs is not None:
            self.runner.plp_enabled = True
        if sp_.guided_decoding is not None:
            if self.guided is None:
                raise ValueError("guided decoding needs the token strings: call set_guided_vocabulary() first")
            if self.cfg.speculative_config:
                raise ValueError("guided decoding and speculative decoding cannot be combined")
            req.guided = self.guided.new_state(sp_.guided_decoding)
        if sp_.guided_decoding is not None or sp_.has_penalties \
                or any(len(w) > 1 for w in (sp_.bad_words_token_ids or ())):
            self._sync_reqs.add(rid)
        self.scheduler.add_request(req)
        return rid

    def _propose(self, so, sampled: dict) -> None:
        p = self.runner.proposer
        if p is None:
            return
        if self._model_proposer:
            hidden = self.runner.model.aux_hidden if getattr(p, "method", "") == "eagle3" else self.runner.last_hidden
            p.propose_step(so, sampled, hidden, self.scheduler)
        else:
            self.runner.propose_draft_tokens([r for r, _ in so.scheduled
                                              if r.status == RequestStatus.RUNNING and r.request_id in sampled])

    def set_guided_vocabulary(self, tokens, eos_token_id: Optional[int] = None) -> None:
        """``tokens``: the string of every token id (list), or a tokenizer with ``decode``.  Needed
        once before requests with ``guided_decoding`` are accepted."""
        from ..sample.guided import GuidedDecodingManager, TokenVocabulary
        if hasattr(tokens, "decode"):
            vocab = TokenVocabulary.from_tokenizer(tokens, self.cfg.model.vocab_size)
            if eos_token_id is not None:
                vocab.eos_token_id = eos_token_id
        else:
            vocab = TokenVocabulary(list(tokens), eos_token_id if eos_token_id is not None else self.eos_token_id)
        if self.eos_token_id is None and vocab.eos_token_id is not None:
            self.eos_token_id = vocab.eos_token_id
        self.guided = GuidedDecodingManager(vocab)

    def _attach_logprobs(self) -> None:
        for rid, entries in self.runner.take_prompt_logprobs().items():
            req = self.scheduler.requests.get(rid)
            if req is not None:
                if getattr(req, "prompt_logprobs", None) is None:
                    req.prompt_logprobs = [None] * req.num_prompt_tokens
                for pos, entry in entries:
                    req.prompt_logprobs[pos] = entry
        for rid, entries in self.runner.take_logprobs().items():
            req = self.scheduler.requests.get(rid)
            if req is not None:
                if req.logprobs is None:
                    req.logprobs = []
                room = len(req.output_token_ids or []) - len(req.logprobs)
                req.logprobs.extend(entries[:max(room, 0)])

    def _release_mm(self, finished) -> None:
        if self.runner.dynamic_spec is not None:
            for r in finished:
                self.runner.dynamic_spec.forget(r.request_id)
        mm = self.runner.mm
        if mm is not None:
            for r in finished:
                mm.release(r)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._inflight is not None

    def _step_async(self) -> list[Request]:
        """One iteration with asynchronous scheduling: plan and enqueue step N+1 while step N
        runs on the GPU, then read step N's tokens.  The host work of a step (scheduling, input
        preparation, launches) overlaps the previous step's kernels."""
        t0 = time.perf_counter()
        prev = self._inflight
        so = self.scheduler.schedule()
        t1 = time.perf_counter()
        handle = None
        if not so.is_empty:
            handle = self.runner.execute_async(so, prev[1] if prev else None)
            self.scheduler.advance(so)
        t2 = time.perf_counter()
        finished: list[Request] = []
        if prev is not None:
            so_prev, h_prev = prev
            sampled = self.runner.collect(h_prev)
            now = time.monotonic()
            for req, _ in so_prev.scheduled:
                if req.first_token_time is None and req.request_id in sampled:
                    req.first_token_time = now
            finished = self.scheduler.update_from_output(so_prev, sampled)
            self._attach_logprobs()
            self._release_mm(finished)
        self._inflight = (so, handle) if handle is not None else None
        t3 = time.perf_counter()
        self.host_times["schedule"] += t1 - t0
        self.host_times["execute"] += t2 - t1
        self.host_times["update"] += t3 - t2
        return finished

    def _needs_sync(self) -> bool:
        """Requests whose next-token distribution depends on the token sampled one step earlier
        (penalties, multi-token bad words) need that token on the host before the next step is built:
        while one is alive the engine steps synchronously."""
        if not self._sync_reqs:
            return False
        reqs = self.scheduler.requests
        self._sync_reqs = {r for r in self._sync_reqs if r in reqs and not reqs[r].is_finished}
        return bool(self._sync_reqs)

    def _drain_async(self) -> list[Request]:
        so_prev, h_prev = self._inflight
        self._inflight = None
        sampled = self.runner.collect(h_prev)
        now = time.monotonic()
        for req, _ in so_prev.scheduled:
            if req.first_token_time is None and req.request_id in sampled:
                req.first_token_time = now
        finished = self.scheduler.update_from_output(so_prev, sampled)
        self._attach_logprobs()
        self._release_mm(finished)
        return finished

    def step(self) -> list[Request]:
        if self.async_scheduling and not self._needs_sync():
            return self._step_async()
        if self._inflight is not None:          # switch to synchronous stepping: finish the step in flight
            return self._drain_async()
        t0 = time.perf_counter()
        so = self.scheduler.schedule()
        t1 = time.perf_counter()
        if self.kv_connector is not None:
            self.kv_connector.start_load_kv(so)
        if self._model_proposer:
            self.runner.proposer.note_step_start(so)
        sampled = self.runner.execute(so)
        t2 = time.perf_counter()
        self.host_times["schedule"] += t1 - t0
        self.host_times["execute"] += t2 - t1
        now = time.monotonic()
        for req, _ in so.scheduled:
            if req.first_token_time is None and req.request_id in sampled:
                req.first_token_time = now
        finished = self.scheduler.update_from_output(so, sampled)
        if self._record_step is not None and so.scheduled:
            self._record_step(so, t2 - t1)              # chunk-size predictor: duration of this step
        self._attach_logprobs()
        self._release_mm(finished)
        self._propose(so, sampled)
        if self.kv_connector is not None:
            self.kv_connector.step_finished(so, self.scheduler)
        if self.eplb is not None:
            self.eplb.step()
        self.host_times["update"] += time.perf_counter() - t2
        return finished

    def step_dp(self) -> bool:
        """One lock-step iteration of a data-parallel engine: the DP ranks agree on whether
        anyone still has work and on the largest token count (the per-step CPU all-reduce of
        vllm_ascend/worker/model_runner_v1.py:669-707); ranks without work run a dummy batch
        so they still meet the others in the expert-parallel collectives
        (vllm_ascend/worker/worker.py:1048-1051).  Returns False when every rank is done."""
        import torch.distributed as dist
        t0 = time.perf_counter()
        busy = self.scheduler.has_unfinished()
        # a scheduler that talks to its peers inside schedule() (cross-replica load balancing) must be
        # called on every rank every step, and may have received work there
        collective = getattr(self.scheduler, "collective_schedule", False)
        so = self.scheduler.schedule() if (busy or collective) else None
        busy = busy or (collective and self.scheduler.has_unfinished())
        ntok = so.num_scheduled_tokens if so is not None else 0
        nrows = 0 if so is None else sum(1 for r, n in so.scheduled if r.num_computed_tokens + n >= r.num_tokens)
        sync = torch.tensor([int(busy), max(ntok, 1), nrows], dtype=torch.int32)
        dist.all_reduce(sync, op=dist.ReduceOp.MAX, group=self.dp.cpu_group)
        if int(sync[0]) == 0:
            return False
        if self.moe_runtime is not None:
            self.moe_runtime.max_tokens_across_dp = int(sync[1])
        from ..parallel.finegrained import get_fg
        fg = get_fg()
        if fg is not None:           # pad targets of the fine-grained TP collectives in this step
            fg.max_tokens, fg.max_rows = int(sync[1]), int(sync[2])
        t1 = time.perf_counter()
        if so is None or so.is_empty:
            self.runner.execute_dummy()
            if self.eplb is not None:
                self.eplb.step()
            self.host_times["execute"] += time.perf_counter() - t1
            return True
        if self.kv_connector is not None:
            self.kv_connector.start_load_kv(so)
        if self._model_proposer:
            self.runner.proposer.note_step_start(so)
        sampled = self.runner.execute(so)
        t2 = time.perf_counter()
        now = time.monotonic()
        for req, _ in so.scheduled:
            if req.first_token_time is None and req.request_id in sampled:
                req.first_token_time = now
        self.scheduler.update_from_output(so, sampled)
        self._propose(so, sampled)
        if self.kv_connector is not None:
            self.kv_connector.step_finished(so, self.scheduler)
        if self.eplb is not None:
            self.eplb.step()
        self.host_times["schedule"] += t1 - t0
        self.host_times["execute"] += t2 - t1
        self.host_times["update"] += time.perf_counter() - t2
        return True

    def check_health(self) -> None:
        self.worker.check_health()


class LLM:
    """vLLM-style offline interface.

    ``model`` is a preset name (random-init weights of that architecture), an HF
    checkpoint directory, or a ``ModelConfig``.
    """

    def __init__(self, model: Union[str, ModelConfig], tensor_parallel_size: int = 1,
                 pipeline_parallel_size: int = 1, enable_expert_parallel: bool = False,
                 dtype: Optional[str] = None, device: Optional[str] = None,
                 max_model_len: int = 4096, max_num_seqs: int = 1024,
                 max_num_batched_tokens: int = 8192, block_size: Optional[int] = None,
                 gpu_memory_utilization: float = 0.92, num_gpu_blocks_override: Optional[int] = None,
                 enable_prefix_caching: bool = False, enforce_eager: bool = False,
                 enable_chunked_prefill: bool = True, quantization: Optional[str] = None,
                 seed: int = 0, additional_config: Optional[dict] = None,
                 kv_transfer_config: Optional[dict] = None, ec_transfer_config: Optional[dict] = None,
                 speculative_config: Optional[dict] = None, enable_sleep_mode: bool = False,
                 cudagraph_capture_sizes: Optional[list] = None,
                 decode_context_parallel_size: int = 1, prefill_context_parallel_size: int = 1,
                 enable_lora: bool = False, max_loras: int = 4,
                 max_lora_rank: int = 64, async_scheduling: Optional[bool] = None, load_format: str = "auto",
                 model_loader_extra_config: Optional[dict] = None, **unused):
        mcfg = model if isinstance(model, ModelConfig) else get_model_config(model)
        if dtype:
            mcfg.dtype = dtype
        if quantization:
            mcfg.quantization = quantization
        mcfg.seed = seed
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        device_index = None
        if device.startswith("cuda:"):
            device, device_index = "cuda", int(device.split(":")[1])
        if block_size is None:
            block_size = 128 if device == "cuda" else 16
        cfg = EngineConfig(
            model=mcfg,
            cache=CacheConfig(block_size=block_size, gpu_memory_utilization=gpu_memory_utilization,
                              num_gpu_blocks=num_gpu_blocks_override,
                              enable_prefix_caching=enable_prefix_caching),
            scheduler=SchedulerConfig(max_num_seqs=max_num_seqs,
                                      max_num_batched_tokens=max(max_num_batched_tokens, 1),
                                      max_model_len=max_model_len,
                                      enable_chunked_prefill=enable_chunked_prefill),
            parallel=ParallelConfig(tensor_parallel_size=tensor_parallel_size,
                                    pipeline_parallel_size=pipeline_parallel_size,
                                    enable_expert_parallel=enable_expert_parallel,
                                    decode_context_parallel_size=decode_context_parallel_size,
                                    prefill_context_parallel_size=prefill_context_parallel_size),
            compilation=CompilationConfig(
                cudagraph_mode="NONE" if enforce_eager else "FULL_DECODE_ONLY",
                cudagraph_capture_sizes=cudagraph_capture_sizes),
            additional_config=additional_config or {}, device=device, device_index=device_index, seed=seed,
            kv_transfer_config=kv_transfer_config, ec_transfer_config=ec_transfer_config,
            speculative_config=speculative_config,
            enable_sleep_mode=enable_sleep_mode, enable_lora=enable_lora, max_loras=max_loras,
            max_lora_rank=max_lora_rank, async_scheduling=async_scheduling, load_format=load_format,
            model_loader_extra_config=model_loader_extra_config)
        if device == "cuda":
            cfg.scheduler.decode_batch_alignment = 256
        from ..platform_config import check_and_update_config
        check_and_update_config(cfg)
        self.cfg = cfg
        self.engine = LLMEngine(cfg)

    # ------------------------------------------------------------------
    def encode_multimodal(self, multi_modal_data: dict) -> list[dict]:
        """Encoder-instance entry point of a disaggregated deployment: runs the vision tower over
        the items, publishes every output through the EC connector and returns
        ``{"hash", "grid_thw"}`` descriptors a prefill / decode instance accepts in place of pixels."""
        eng = self.engine
        mm = eng.runner.mm
        if mm is None:
            raise ValueError("the model has no vision tower")
        from ..multimodal import build_mm_request
        mcfg = self.cfg.model
        out = []
        for modality, tok in (("image", mcfg.image_token_id), ("video", mcfg.video_token_id)):
            entries = multi_modal_data.get(modality) or []
            if not entries:
                continue
            _, items = build_mm_request([tok] * len(entries), {modality: entries}, mcfg)

            class _Req:
                request_id = f"_encode-{modality}"
            with torch.inference_mode():
                mm._run_encoder([(_Req, k, it) for k, it in enumerate(items)])
            for k, it in enumerate(items):
                emb = mm.encoder_cache.pop((_Req.request_id, k))
                if mm.ec_connector is not None and not mm.ec_connector.is_producer:
                    mm.ec_connector.save(it.hash, emb)
                out.append({"modality": modality, "hash": it.hash, "grid_thw": list(it.grid_thw)})
        return out

    def set_guided_vocabulary(self, tokens, eos_token_id: Optional[int] = None) -> None:
        self.engine.set_guided_vocabulary(tokens, eos_token_id)

    def beam_search(self, prompts, beam_width: int = 4, max_tokens: int = 16, length_penalty: float = 1.0,
                    ignore_eos: bool = False, temperature: float = 0.0) -> list[list[dict]]:
        """Beam search over the engine: every round extends all live beams of all prompts by one
        token in ONE batch (``logprobs = 2 * beam_width`` candidates each; automatic prefix caching
        makes a round cost one decode step per beam), keeps the ``beam_width`` best continuations
        per prompt by cumulative log-probability and retires beams that emit the end token.
        Returns, per prompt, the ``beam_width`` best sequences as dicts ``{"tokens",
        "cum_logprob", "score"}`` with score = cum_logprob / len ** length_penalty."""
        del temperature
        eos = self.engine.eos_token_id
        width = int(beam_width)
        plist = [list(p["prompt_token_ids"]) if isinstance(p, dict) else list(p) for p in prompts]
        live = [[(p, 0.0)] for p in plist]              # per prompt: (tokens, cum_logprob)
        done: list[list[tuple]] = [[] for _ in plist]
        sp = SamplingParams(temperature=0.0, max_tokens=1, logprobs=2 * width, ignore_eos=True)

        def score(tokens, cum, n_prompt):
            return cum / (max(len(tokens) - n_prompt, 1) ** length_penalty)
        for _ in range(max_tokens):
            flat = [(i, b) for i, beams in enumerate(live) for b in beams]
            if not flat:
                break
            outs = self.generate([b[0] for _, b in flat], sp)
            cands: list[list[tuple]] = [[] for _ in plist]
            for (i, (toks, cum)), o in zip(flat, outs):
                for tok, lp in o.outputs[0].logprobs[0].items():
                    cands[i].append((toks + [int(tok)], cum + float(lp)))
            for i, cs in enumerate(cands):
                cs.sort(key=lambda c: c[1], reverse=True)
                nxt = []
                for toks, cum in cs:
                    if not ignore_eos and eos is not None and toks[-1] == eos:
                        done[i].append((toks, cum))
                    else:
                        nxt.append((toks, cum))
                    if len(nxt) >= width:
                        break
                # a prompt stops once it holds `width` finished beams that beat every live one
                if len(done[i]) >= width:
                    n0 = len(plist[i])
                    worst_done = sorted((score(t, c, n0) for t, c in done[i]), reverse=True)[width - 1]
                    if not nxt or worst_done >= max(score(t, c, n0) for t, c in nxt):
                        nxt = []
                live[i] = nxt
        result = []
        for i, n0 in enumerate(len(p) for p in plist):
            allb = done[i] + live[i]
            allb.sort(key=lambda b: score(b[0], b[1], n0), reverse=True)
            result.append([{"tokens": t[n0:], "cum_logprob": c, "score": score(t, c, n0)} for t, c in allb[:width]])
        return result

    def embed(self, prompts, normalize: bool = True) -> list:
        """Sequence embeddings: the final hidden state of every prompt's last token (last-token
        pooling, the pooling of decoder-only embedding models), L2-normalised by default."""
        sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True, extra_args={"pooling": True})
        eng = self.engine
        rids = [eng.add_request(p["prompt_token_ids"] if isinstance(p, dict) else p, sp) for p in prompts]
        reqs = [eng.scheduler.requests[r] for r in rids]
        while eng.has_unfinished():
            eng.step()
        out = []
        for r in reqs:
            v = r.pooled
            out.append(torch.nn.functional.normalize(v, dim=-1) if normalize else v)
        return out

    @staticmethod
    def _child_params(sp: SamplingParams, j: int) -> SamplingParams:
        """Sampling parameters of the j-th of ``sp.n`` samples: independent random streams (seed + j
        when a seed is given), everything else shared."""
        if sp.n <= 1:
            return sp
        import copy
        c = copy.copy(sp)
        c.n = 1
        if sp.seed is not None:
            c.seed = sp.seed + j
        return c

    def generate(self, prompts, sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 use_tqdm: bool = False, lora_request=None,
                 max_concurrency: Optional[int] = None) -> list[RequestOutput]:
        """``prompts``: list of token-id lists (or dicts with ``prompt_token_ids`` and optionally
        ``request_id``, ``job_id`` (the batch-job scheduler groups requests by it), ``multi_modal_data``,
        ``prompt_embeds``, ``kv_transfer_params``).

        ``max_concurrency``: closed-loop admission.  At most that many requests are in flight (per
        data-parallel replica: its share of the total); the next prompt enters when one finishes.
        This is the fixed-concurrency serving workload of the reference's benchmark cases
        (benchmarks/tests/serving-tests.json, ``max_concurrency``); ``None`` submits everything at once.
        A request's ``arrival_time`` is the moment it is admitted."""
        if sampling_params is None:
            sampling_params = SamplingParams()
        eng = self.engine
        dp = eng.dp
        order: list[str] = []
        mine: list[int] = []
        reqs: dict[str, Request] = {}
        pending = [i for i in range(len(prompts))
                   if dp.world_size == 1 or i % dp.world_size == dp.rank_in_group]
        pending.reverse()             # data parallel: every DP rank serves its own slice
        limit = None
        if max_concurrency is not None:
            limit = max(1, int(max_concurrency) // max(dp.world_size, 1))

        def admit() -> None:
            while pending and (limit is None or eng.scheduler.num_unfinished < limit):
                i = pending.pop()
                p = prompts[i]
                ids = p.get("prompt_token_ids") if isinstance(p, dict) else p
                sp = sampling_params[i] if isinstance(sampling_params, (list, tuple)) else sampling_params
                ktp = p.get("kv_transfer_params") if isinstance(p, dict) else None
                lr = lora_request[i] if isinstance(lora_request, (list, tuple)) else lora_request
                mmd = p.get("multi_modal_data") if isinstance(p, dict) else None
                pe = p.get("prompt_embeds") if isinstance(p, dict) else None
                job = p.get("job_id") if isinstance(p, dict) else None       # batch-job scheduling
                given_id = p.get("request_id") if isinstance(p, dict) else None
                if pe is not None and ids is None:
                    ids = []
                rid = eng.add_request(ids, self._child_params(sp, 0), request_id=given_id, kv_transfer_params=ktp,
                                      job_id=job, lora_request=lr, multi_modal_data=mmd, prompt_embeds=pe)
                order.append(rid)
                mine.append(i)
                reqs[rid] = eng.scheduler.requests[rid]
                reqs[rid].client_index, reqs[rid].origin_rank = i, dp.rank_in_group
                reqs[rid].siblings = []
                for j in range(1, max(1, sp.n)):          # n > 1: sibling requests over the same prompt
                    sid = eng.add_request(ids, self._child_params(sp, j), kv_transfer_params=ktp, job_id=job,
                                          lora_request=lr, multi_modal_data=mmd, prompt_embeds=pe)
                    reqs[rid].siblings.append(eng.scheduler.requests[sid])

        admit()
        if dp.world_size > 1:
            while eng.step_dp():
                admit()
        else:
            while eng.has_unfinished() or pending:
                eng.step()
                admit()
        eng.check_health()
        if dp.world_size > 1:
            # requests may have moved between DP ranks (load balancing): report what finished here
            done = [r for r in eng.scheduler.requests.values()
                    if r.is_finished and getattr(r, "client_index", None) is not None]
            for r in done:
                if getattr(r, "siblings", None) and not all(s_.is_finished for s_ in r.siblings):
                    raise RuntimeError("n > 1 is not supported together with cross-replica request migration")
            mine = [r.client_index for r in done]
            order = [r.request_id for r in done]
            reqs = {r.request_id: r for r in done}
        outs = []
        for rid in order:
            r = reqs[rid]
            family = [r] + list(getattr(r, "siblings", None) or [])
            outs.append(RequestOutput(
                request_id=rid, prompt_token_ids=r.prompt_token_ids.tolist(),
                outputs=[CompletionOutput(j, list(c.output_token_ids or []),
                                          finish_reason=_FINISH_REASON.get(c.status), logprobs=c.logprobs,
                                          stop_reason=c.stop_reason)
                         for j, c in enumerate(family)],
                finished=True,
                metrics=RequestMetrics(r.arrival_time, r.first_token_time, r.finish_time),
                kv_transfer_params=r.kv_transfer_params, num_cached_tokens=r.num_cached_tokens,
                prompt_logprobs=r.prompt_logprobs))
            for c in family:
                eng.scheduler.requests.pop(c.request_id, None)
        if dp.world_size > 1:
            # every rank returns the complete, input-ordered list
            merged: list = [None] * len(prompts)
            for idxs, part in dp.all_gather_object((mine, outs)):
                for i, o in zip(idxs, part):
                    merged[i] = o
            outs = merged
        return outs

    # -- RL / lifecycle passthroughs (implemented by the worker-level mixins) ------
    def sleep(self, level: int = 1) -> None:
        from ..device_allocator.sleep import sleep as _sleep
        _sleep(self.engine, level)

    def wake_up(self, tags: Optional[list[str]] = None) -> None:
        from ..device_allocator.sleep import wake_up as _wake
        _wake(self.engine, tags)

    def shutdown(self) -> None:
        """Release device-side state in dependency order: captured graphs first (they may
        hold collectives), then connectors and peer mappings, then the process groups."""
        import torch.distributed as dist
        eng = self.engine
        if eng.device.type == "cuda":
            torch.cuda.synchronize()
        eng.runner.drop_graphs()
        if eng.kv_connector is not None:
            eng.kv_connector.close()
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
            if eng.device.type == "cuda":
                torch.cuda.synchronize()
            dist.destroy_process_group()

    def save_sharded_state(self, path: str, max_bytes: int = 5 << 30) -> list:
        """Every rank writes the tensors it holds; load them back with
        ``load_format="sharded_state", model_loader_extra_config={"path": path}``."""
        import os
        from ..model_loader.sharded_state import save_sharded_state
        return save_sharded_state(self.engine.runner.model, path, int(os.environ.get("RANK", "0")), max_bytes)

    def reload_weights(self, path: Optional[str] = None) -> int:
        """Re-read the weights in place (same tensors, same addresses: captured graphs and peer
        mappings stay valid) from ``path`` or from the directory the model was loaded from; the KV
        cache of earlier weights is dropped.  Returns the number of tensors loaded."""
        from ..models.transformer import iterate_safetensors
        src = path or self.cfg.model.model_path
        if not src:
            raise ValueError("reload_weights needs a checkpoint directory")
        if self.engine.has_unfinished():
            raise RuntimeError("reload_weights with requests in flight")
        model = self.engine.runner.model
        n = len(model.load_weights(iterate_safetensors(src)))
        if getattr(model, "norm_folded", False):        # the norm weights just came back: fold them again
            from ..models.folded import fold_norms
            fold_norms(model)
        self.cfg.model.model_path = src
        self.engine.scheduler.pool.reset_prefix_cache()
        return n

    def serve_weights(self, host: str = "127.0.0.1", port: int = 0):
        """Let starting instances pull this instance's weights (netloader / rfork seed)."""
        from ..model_loader.netloader import WeightSource
        tp = pstate.get_tp_group()
        self._weight_source = WeightSource(self.engine.runner.model, host, port, tp.rank_in_group, tp.world_size,
                                           self.cfg.model.name)
        return self._weight_source

    def reset_prefix_cache(self) -> bool:
        return self.engine.scheduler.pool.reset_prefix_cache()

    def get_metrics(self) -> dict:
        from ..observability.metrics import collect
        return collect(self.engine)
