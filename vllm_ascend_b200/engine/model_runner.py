"""Model runner: persistent input batch, input preparation, forward (eager or
CUDA-graph replay), logits and sampling.

Responsibilities mirror ``NPUModelRunner`` (vllm_ascend/worker/model_runner_v1.py):
``_prepare_inputs`` (:850-1285), attention metadata (:2813-3122), batch padding and
graph dispatch (:2714-2811), KV-cache allocation as separate K and V tensors per
layer (:3863-4069), ``capture_model`` (:4852-4862).  Device-side metadata lives in
persistent buffers so graph replay needs no host-side argument refresh.
"""
from __future__ import annotations

import math
import os
import time
from typing import Optional

import numpy as np
import torch

from .. import _native, envs, ops
from ..attention.metadata import (AttentionMetadata, AttentionState, build_tile_worklist,
                                  split_decodes_and_prefills)
from ..config import EngineConfig
from ..parallel import state as pstate
from ..sample.sampler import Sampler, SamplingMetadata
from .request import Request
from .scheduler import SchedulerOutput


def default_capture_sizes(max_size: int) -> list[int]:
    """1, 2, 4, 8, then multiples of 8 up to 64, of 16 up to 256, of 32 beyond."""
    sizes = [1, 2, 4]
    s = 8
    while s <= max_size:
        sizes.append(s)
        s += 8 if s < 64 else (16 if s < 256 else 32)
    if sizes[-1] != max_size and max_size > sizes[-1]:
        sizes.append(max_size)
    return [x for x in sizes if x <= max_size]


class _SpecRow:
    """One logits row of a speculative verification step seen as a request: the request itself with
    its first ``j`` draft tokens appended to the generated history."""
    __slots__ = ("_r", "_j", "output_token_ids", "num_output_tokens", "num_inflight", "guided")

    def __init__(self, req, j: int):
        self._r, self._j = req, j
        self.output_token_ids = list(req.output_token_ids or []) + [int(t) for t in req.spec_token_ids[:j]]
        self.num_output_tokens = req.num_output_tokens + j
        self.num_inflight = getattr(req, "num_inflight", 0)
        self.guided = None

    def __getattr__(self, name):
        return getattr(self._r, name)


class _StepHandle:
    """A step that was enqueued but whose sampled tokens have not been read yet."""
    __slots__ = ("tokens", "reqs", "host", "event", "kind", "t_start", "index", "logprobs", "ev_start", "num_tokens",
                 "h_sel")

    def __init__(self, tokens, reqs, host, event, kind, t_start):
        self.tokens, self.reqs, self.host, self.event, self.kind, self.t_start = tokens, reqs, host, event, kind, t_start
        self.index = {r.request_id: i for i, r in enumerate(reqs)}
        self.logprobs = None
        self.ev_start = None
        self.num_tokens = 0
        self.h_sel = None          # hidden rows awaiting a deferred sampling (finish_sampling)


class ModelRunner:
    def __init__(self, cfg: EngineConfig, device: torch.device):
        self._step_timing = device.type == "cuda" and os.environ.get("VLLM_B200_STEP_TIMING", "0") == "1"
        self._last_step_end = None
        self.cfg = cfg
        self.device = device
        self.mcfg = cfg.model
        self.block_size = cfg.cache.block_size
        self.max_seqs = cfg.scheduler.max_num_seqs
        self.max_tokens = cfg.scheduler.max_num_batched_tokens
        self.max_model_len = cfg.scheduler.max_model_len
        self.max_blocks_per_seq = (self.max_model_len + self.block_size - 1) // self.block_size
        self.model = None
        self.kv_caches: list = []
        self.num_blocks = 0
        self.sampler = Sampler()
        self.is_cuda = device.type == "cuda"
        # ---- persistent host state (one row per live request)
        self.token_ids_cpu = np.zeros((self.max_seqs, self.max_model_len), dtype=np.int32)
        self.block_table_cpu = np.zeros((self.max_seqs, self.max_blocks_per_seq), dtype=np.int32)
        self.row_owner: list[Optional[str]] = [None] * self.max_seqs
        self.row_num_blocks = np.zeros(self.max_seqs, dtype=np.int32)
        self.row_num_tokens = np.zeros(self.max_seqs, dtype=np.int32)
        # ---- persistent device inputs
        # room for one extra token per sequence: draft-model catch-up passes append the newly
        # sampled token of every request to a full step
        T, B = self.max_tokens + self.max_seqs, self.max_seqs
        from ..parallel import state as _ps0
        if _ps0.get_pcp_group().world_size > 1:
            B *= 2            # prefill context parallel: a request contributes up to two batch entries
        i64, i32 = torch.int64, torch.int32
        self.input_ids = torch.zeros(T, dtype=i64, device=device)
        self.positions = torch.zeros(T, dtype=i64, device=device)
        self.slot_mapping = torch.full((T,), -1, dtype=i64, device=device)
        self.query_start_loc = torch.zeros(B + 1, dtype=i32, device=device)
        self.seq_lens = torch.ones(B, dtype=i32, device=device)
        self.block_table = torch.zeros((B, self.max_blocks_per_seq), dtype=i32, device=device)
        max_tiles = T + B
        self.tile_seq = torch.zeros(max_tiles, dtype=i32, device=device)
        self.tile_qoff = torch.zeros(max_tiles, dtype=i32, device=device)
        pin = self.is_cuda
        self._h_ids = torch.zeros(T, dtype=i64, pin_memory=pin)
        self._h_pos = torch.zeros(T, dtype=i64, pin_memory=pin)
        self._h_slot = torch.zeros(T, dtype=i64, pin_memory=pin)
        self._h_req = torch.zeros(T, dtype=torch.int32, pin_memory=pin)
        self._req_rows = torch.zeros(T, dtype=torch.int32, device=device)
        self._h_qsl = torch.zeros(B + 1, dtype=i32, pin_memory=pin)
        self._h_sl = torch.zeros(B, dtype=i32, pin_memory=pin)
        self._h_bt = torch.zeros((B, self.max_blocks_per_seq), dtype=i32, pin_memory=pin)
        self._h_tile = torch.zeros((2, max_tiles), dtype=i32, pin_memory=pin)
        self._h_sampled = torch.zeros(B, dtype=i64, pin_memory=pin)
        self._h_state = torch.zeros((2, B), dtype=i32, pin_memory=pin)
        self.state_meta = torch.zeros((2, B), dtype=i32, device=device)     # [slot; has_initial_state]
        self._h_sampled2 = [torch.zeros(B, dtype=i64, pin_memory=pin) for _ in range(2)]   # async steps
        self._async_flip = 0
        # ---- CUDA graphs
        self.graphs: dict[tuple, object] = {}     # (capture size, has_lora) -> BatchDescriptor
        self.graph_wrapper = None
        self.lora_manager = None
        self.mm = None                   # MultimodalState for models with a vision tower
        self.sparse_offload = None       # per-layer host-resident KV stores (sparse attention offload)
        self.moe_runtime = None
        from ..parallel import state as _ps
        self.pp = _ps.get_pp_group()
        dcp = _ps.get_dcp_group()
        self.dcp_size, self.dcp_rank = dcp.world_size, dcp.rank_in_group
        self.dcp_interleave = int((cfg.additional_config or {}).get("cp_kv_cache_interleave_size", 1))
        if self.dcp_size > 1 and not cfg.model.use_mla:
            # the ranks of a DCP group shard one sequence of keys: they must hold the same KV heads
            tp_ = _ps.get_tp_group().world_size
            rep = max(1, tp_ // max(1, cfg.model.num_key_value_heads))
            if cfg.model.is_hybrid or cfg.model.sliding_window or rep % self.dcp_size:
                raise NotImplementedError(
                    "decode context parallelism for grouped-query attention needs KV heads replicated over the "
                    f"DCP ranks (tensor_parallel_size / num_key_value_heads = {rep} must be a multiple of "
                    f"{self.dcp_size}), no sliding window and no recurrent layers")
        self.pcp = _ps.get_pcp_group()
        if self.pcp.world_size > 1 and (cfg.model.use_mla or cfg.model.is_hybrid or cfg.model.is_multimodal):
            raise NotImplementedError("prefill context parallelism is implemented for GQA decoder models")
        self._pcp_bcast = False          # this step's tokens come from PCP rank 0
        self._prompt_lp_out: dict = {}
        self.plp_enabled = False     # set once a request asks for prompt log-probabilities
        self._plp_chunks: list = []
        self._logprobs_out: dict = {}
        self.proposer = None
        self.last_hidden = None      # final hidden states of the latest step, scheduling order
        self.rejection_sampler = None
        self.dynamic_spec = None         # spec_decode.dynamic.DynamicSpecController when configured
        self.spec_stats = {"draft_tokens": 0, "accepted_tokens": 0, "verify_steps": 0}
        self._sample_rows: list = []
        self.graph_pool = None
        self.capture_sizes: list[int] = []
        self.stats = {"graph_replays": 0, "eager_steps": 0, "h2d_bytes": 0, "d2h_bytes": 0,
                      "steps": 0, "graph_kernel_launches": 0, "t_prepare": 0.0, "t_launch": 0.0,
                      "t_wait": 0.0}
        self.sm_count = (torch.cuda.get_device_properties(device).multi_processor_count
                         if self.is_cuda else 1)

    # ------------------------------------------------------------------ model / memory
    def load_model(self, moe_runtime=None) -> None:
        from ..models import build_model
        t0 = time.time()
        self.moe_runtime = moe_runtime
        self.model = build_model(self.cfg, self.device, moe_runtime=moe_runtime)
        from ..model_loader import get_model_loader
        from ..parallel import state as pstate
        tp = pstate.get_tp_group()
        loader = get_model_loader(self.cfg.load_format, self.cfg.model_loader_extra_config, tp.rank_in_group,
                                  tp.world_size, self.mcfg.name)
        self.loaded_from_peer = bool(loader is not None and loader.load(self.model))
        if self.mcfg.model_path and not self.loaded_from_peer:
            from ..models.transformer import iterate_safetensors
            self.model.load_weights(iterate_safetensors(self.mcfg.model_path))
        self.load_time = time.time() - t0
        if self.mcfg.is_multimodal and self.model.is_first:
            from .mm_runner import MultimodalState
            self.mm = MultimodalState(self)
            # towers that split host index math from a capturable device part replay from graphs
            if self.is_cuda and self.cfg.compilation.cudagraph_mode != "NONE" \
                    and hasattr(self.model.visual, "host_inputs"):
                from ..compilation.encoder_graph import EncoderGraphManager
                self.mm.encoder_graphs = EncoderGraphManager(self.model.visual)

    def _attn_layer(self):
        """First layer with a paged KV cache (hybrid models start with recurrent layers)."""
        for L in self.model.layers:
            if not getattr(L.self_attn, "is_linear_attention", False):
                return L.self_attn
        raise RuntimeError("model has no attention layer with a KV cache")

    def _num_kv_layers(self) -> int:
        return sum(1 for L in self.model.layers if not getattr(L.self_attn, "is_linear_attention", False))

    def state_bytes(self) -> int:
        """Memory of the per-sequence recurrent / convolution states of linear-attention layers."""
        total = 0
        for L in self.model.layers:
            a = L.self_attn
            if getattr(a, "is_linear_attention", False):
                cs, ss = a.state_shapes(self.max_seqs + 1)
                n_c = 1
                for d in cs:
                    n_c *= d
                n_s = 1
                for d in ss:
                    n_s *= d
                total += n_c * 2 + n_s * 4
        return total

    def kv_bytes_per_block(self) -> int:
        m = self.model
        n_layers = self._num_kv_layers()
        itemsize = torch.tensor([], dtype=self.kv_dtype).element_size()
        per_tok = sum(self._cache_widths()) * itemsize
        return n_layers * self.block_size * per_tok

    @property
    def kv_dtype(self) -> torch.dtype:
        return self.mcfg.torch_dtype

    def _cache_widths(self) -> tuple[int, int]:
        c = self.mcfg
        if c.use_mla and c.use_sparse and self._offload_cfg().enabled:
            return (c.index_head_dim,)                    # only the index keys are paged on the device
        if c.use_mla:
            return (c.kv_lora_rank, c.qk_rope_head_dim) + ((c.index_head_dim,) if c.use_sparse else ())
        a = self._attn_layer()
        return (a.Hkv * a.D, a.Hkv * a.D)

    def activation_bytes_estimate(self) -> int:
        c = self.mcfg
        tp = self.cfg.parallel.tensor_parallel_size
        T = self.max_tokens
        inter = max(c.intermediate_size, c.moe_intermediate_size * max(1, c.num_experts_per_tok))
        per_tok = (6 * c.hidden_size + 3 * (c.num_attention_heads * c.q_head_dim) // tp
                   + 3 * inter // tp) * 2
        logits = self.max_seqs * c.vocab_size * 6
        return int(1.3 * (T * per_tok + logits)) + (1 << 30)

    def determine_num_blocks(self) -> int:
        cc = self.cfg.cache
        if cc.num_gpu_blocks:
            return cc.num_gpu_blocks
        if not self.is_cuda:
            return max(64, 4 * self.max_seqs)
        torch.cuda.synchronize()
        free, total = torch.cuda.mem_get_info(self.device)
        budget = total * cc.gpu_memory_utilization - (total - free) - self.activation_bytes_estimate() \
            - self.state_bytes()
        n = int(budget // self.kv_bytes_per_block())
        if n < 8:
            raise RuntimeError(f"not enough memory for the KV cache ({budget / 2**30:.1f} GiB left)")
        # a block beyond what max_num_seqs full-length sequences can use is wasted
        return min(n, self.max_seqs * self.max_blocks_per_seq + 1)

    def init_kv_cache(self, num_blocks: int) -> None:
        """Per layer two tensors (K, V) or (latent, rope), zero-filled so masked key
        positions never hold NaN bit patterns."""
        self.num_blocks = num_blocks
        c = self.mcfg
        self.kv_caches = []
        per_layer = []
        self._init_sparse_offload()
        for layer in self.model.layers:
            if getattr(layer.self_attn, "is_linear_attention", False):
                per_layer.append(None)              # recurrent state instead of a paged cache
                continue
            if c.use_mla:
                nb_main = 1 if self._offload_cfg().enabled else num_blocks      # host-resident: placeholders
                shapes = [(nb_main, self.block_size, 1, c.kv_lora_rank),
                          (nb_main, self.block_size, 1, c.qk_rope_head_dim)]
                if c.use_sparse:          # index keys of the lightning indexer
                    shapes.append((num_blocks, self.block_size, 1, c.index_head_dim))
            else:
                a = layer.self_attn
                shapes = [(num_blocks, self.block_size, a.Hkv, a.D)] * 2
            per_layer.append(shapes)
        layout = self.cfg.cache.kv_layout if self.is_cuda else "NHD"
        self.kv_arena = None
        if self.is_cuda and self.cfg.kv_transfer_config and not self.cfg.enable_sleep_mode:
            # one exportable allocation, so a decode engine in another process of this node
            # can map the whole cache through a single CUDA IPC handle
            from ..distributed.kv_transfer.nvlink_connector import KVArena
            torch.cuda.empty_cache()
            state_bytes = 0
            for layer, shapes in zip(self.model.layers, per_layer):
                if shapes is None:         # recurrent state caches travel with the KV (hybrid models)
                    cs, ss = layer.self_attn.state_shapes(self.max_seqs + 1)
                    state_bytes += KVArena.bytes_needed([cs], self.kv_dtype) + KVArena.bytes_needed([ss], torch.float32)
            self.kv_arena = KVArena(KVArena.bytes_needed([s for sh in per_layer if sh for s in sh],
                                                         self.kv_dtype) + state_bytes, self.device)
        for layer, shapes in zip(self.model.layers, per_layer):
            if shapes is None:
                # one state row per batch row, plus a scratch row for padded graph entries
                cs, ss = layer.self_attn.state_shapes(self.max_seqs + 1)
                if self.kv_arena is not None:
                    self.kv_caches.append((self.kv_arena.take(cs, self.kv_dtype), self.kv_arena.take(ss, torch.float32)))
                else:
                    self.kv_caches.append((torch.zeros(cs, dtype=self.kv_dtype, device=self.device),
                                           torch.zeros(ss, dtype=torch.float32, device=self.device)))
                continue
            self.kv_caches.append(tuple(
                ops.alloc_kv_cache(s[0], s[1], s[2], s[3], self.kv_dtype, self.device, layout,
                                   arena=self.kv_arena)
                for s in shapes))

    # ------------------------------------------------------------------ persistent batch
    def _offload_cfg(self):
        from ..platform_config import get_b200_config
        return get_b200_config().sparse_kv_offload_config

    def _init_sparse_offload(self) -> None:
        oc, c = self._offload_cfg(), self.mcfg
        if not (oc.enabled and c.use_sparse):
            return
        from ..attention.sparse_offload import SparseOffloadLayer
        slots = oc.device_slots_per_seq or 4 * c.index_topk
        slots = max(slots, c.index_topk)
        self.sparse_offload = []
        for layer in self.model.layers:
            so_ = SparseOffloadLayer(self.max_seqs, self.max_model_len, slots, c.kv_lora_rank, c.qk_rope_head_dim,
                                     self.kv_dtype, self.device, oc.num_threads)
            layer.self_attn.offload = so_
            self.sparse_offload.append(so_)

    def _sync_rows(self, so: SchedulerOutput) -> None:
        for req in so.new_block_rows:
            row = req.row
            if row < 0:
                continue
            if self.row_owner[row] != req.request_id and self.sparse_offload is not None:
                for so_ in self.sparse_offload:          # a new sequence starts with an empty resident set
                    so_.release(row)
            if self.row_owner[row] != req.request_id:
                self.row_owner[row] = req.request_id
                self.row_num_blocks[row] = 0
                n = req.num_prompt_tokens
                self.token_ids_cpu[row, :n] = req.prompt_token_ids
                if req.output_token_ids:
                    k = len(req.output_token_ids)
                    self.token_ids_cpu[row, n:n + k] = req.output_token_ids
                self.row_num_tokens[row] = req.num_tokens
            have = self.row_num_blocks[row]
            nb = len(req.block_ids)
            if nb > have:
                self.block_table_cpu[row, have:nb] = req.block_ids[have:nb]
                self.row_num_blocks[row] = nb
            elif nb < have:          # preempted and re-admitted with fewer blocks
                self.block_table_cpu[row, :nb] = req.block_ids
                self.row_num_blocks[row] = nb

    def _use_device_slots(self) -> bool:
        from .. import envs
        return envs.VLLM_B200_DEVICE_SLOT_MAPPING == "1" and self.device.type == "cuda"

    def _prepare_inputs(self, so: SchedulerOutput, pad_to: Optional[int] = None):
        from ..profiler import nvtx_range
        with nvtx_range("prepare_inputs"):
            return self._prepare_inputs_impl(so, pad_to)

    def _prepare_inputs_impl(self, so: SchedulerOutput, pad_to: Optional[int] = None):
        reqs = [r for r, _ in so.scheduled]
        B = len(reqs)
        q_lens = np.fromiter((n for _, n in so.scheduled), dtype=np.int32, count=B)
        rows = np.fromiter((r.row for r in reqs), dtype=np.int64, count=B)
        starts = np.fromiter((r.num_computed_tokens for r in reqs), dtype=np.int32, count=B)
        T = int(q_lens.sum())
        cu = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu[1:])
        req_idx = np.repeat(np.arange(B, dtype=np.int64), q_lens)
        pos = np.arange(T, dtype=np.int64) - np.repeat(cu[:-1].astype(np.int64), q_lens) \
            + np.repeat(starts.astype(np.int64), q_lens)
        tok_rows = rows[req_idx]
        for r in reqs:                      # draft tokens under verification follow the last token
            sp_ = getattr(r, "spec_token_ids", None)
            if sp_:
                self.token_ids_cpu[r.row, r.num_tokens:r.num_tokens + len(sp_)] = sp_
        ids = self.token_ids_cpu[tok_rows, pos]
        if self.dcp_size > 1:
            # sequence-sharded cache: a virtual block of block_size * dcp tokens keeps
            # block_size of them on this rank
            from ..attention.dcp import local_slot_mapping
            blk = self.block_table_cpu[tok_rows, pos // (self.block_size * self.dcp_size)]
            slots = local_slot_mapping(pos, blk, self.block_size, self.dcp_size, self.dcp_rank,
                                       self.dcp_interleave)
        else:
            blk = self.block_table_cpu[tok_rows, pos // self.block_size].astype(np.int64)
            slots = blk * self.block_size + pos % self.block_size
        pcp_meta = None
        self._pcp_bcast = False
        g_cu, g_starts, g_qlens = cu, starts, q_lens       # per request, global token order
        inv = None
        P = self.pcp.world_size
        if P > 1 and pad_to is None and B and int(q_lens.max()) >= 2 * P:
            # split prefill step: keep this rank's share of the tokens; the attention batch gets one
            # entry per (request, piece) and K / V of all ranks are gathered inside the layers
            from ..attention.pcp import PCPMeta, build_plan
            plan = build_plan(starts, q_lens, cu, P)
            me = self.pcp.rank_in_group
            loc = plan.local_idx[me]
            gslots = np.full(P * plan.t_max, -1, dtype=np.int64)
            for r_, idx_ in enumerate(plan.local_idx):
                gslots[r_ * plan.t_max:r_ * plan.t_max + len(idx_)] = slots[idx_]
            pcp_meta = PCPMeta(self.pcp, plan.t_max, torch.from_numpy(gslots).to(self.device))
            inv = np.full(T, -1, dtype=np.int64)
            inv[loc] = np.arange(len(loc))
            ids, pos, slots = ids[loc], pos[loc], slots[loc]
            ent = plan.entries[me]
            e_req = np.fromiter((e[0] for e in ent), dtype=np.int64, count=len(ent))
            starts = np.fromiter((e[1] for e in ent), dtype=np.int32, count=len(ent))
            q_lens = np.fromiter((e[2] - e[1] for e in ent), dtype=np.int32, count=len(ent))
            rows = rows[e_req]
            B, T = len(ent), len(loc)
            cu = np.zeros(B + 1, dtype=np.int32)
            np.cumsum(q_lens, out=cu[1:])
            self._pcp_bcast = True
        seq_lens = starts + q_lens
        Bp = pad_to or B
        Tp = T + (Bp - B)                       # padded rows carry one dummy token each
        h = self
        h._h_ids[:T] = torch.from_numpy(ids.astype(np.int64))
        h._h_pos[:T] = torch.from_numpy(pos)
        h._h_slot[:T] = torch.from_numpy(slots)
        h._h_qsl[:B + 1] = torch.from_numpy(cu)
        h._h_sl[:B] = torch.from_numpy(seq_lens)
        h._h_bt[:B] = torch.from_numpy(self.block_table_cpu[rows])
        if Bp > B:
            h._h_ids[T:Tp] = 0
            h._h_pos[T:Tp] = 0
            h._h_slot[T:Tp] = -1
            h._h_qsl[B + 1:Bp + 1] = torch.arange(T + 1, Tp + 1, dtype=torch.int32)
            h._h_sl[B:Bp] = 1
            h._h_bt[B:Bp] = 0
        nb = True
        self.input_ids[:Tp].copy_(h._h_ids[:Tp], non_blocking=nb)
        self.positions[:Tp].copy_(h._h_pos[:Tp], non_blocking=nb)
        self.query_start_loc[:Bp + 1].copy_(h._h_qsl[:Bp + 1], non_blocking=nb)
        self.seq_lens[:Bp].copy_(h._h_sl[:Bp], non_blocking=nb)
        self.block_table[:Bp].copy_(h._h_bt[:Bp], non_blocking=nb)
        if self._use_device_slots() and pcp_meta is None and self.dcp_size == 1:
            # slots from the block table on the device: the request row of every token travels
            # (4 bytes per token) instead of the slot (8 bytes), padding rows carry -1
            from ..ops.bookkeeping import slot_mapping as device_slot_mapping
            h._h_req[:T] = torch.from_numpy(req_idx.astype(np.int32))
            h._h_req[T:Tp] = -1
            self._req_rows[:Tp].copy_(h._h_req[:Tp], non_blocking=nb)
            device_slot_mapping(self.block_table[:Bp], self._req_rows[:Tp], self.positions[:Tp], self.block_size,
                                self.num_blocks, out=self.slot_mapping[:Tp])
        else:
            self.slot_mapping[:Tp].copy_(h._h_slot[:Tp], non_blocking=nb)
        self.stats["h2d_bytes"] += Tp * 24 + (Bp + 1) * 4 + Bp * 4 + Bp * self.max_blocks_per_seq * 4

        if self.lora_manager is not None:
            self._update_lora(reqs, q_lens, Tp)
        max_q = int(q_lens.max()) if B else 0
        max_s = int(seq_lens.max()) if B else 0
        nd, npf, ndt, _ = split_decodes_and_prefills(q_lens)
        if max_q == 1:
            state = AttentionState.DecodeOnly
        elif (starts == 0).all():
            state = AttentionState.PrefillNoCache
        else:
            state = AttentionState.ChunkedPrefill
        qsl_cpu = cu if Bp == B else np.concatenate([cu, np.arange(T + 1, Tp + 1, dtype=np.int32)])
        sl_cpu = seq_lens if Bp == B else np.concatenate([seq_lens, np.ones(Bp - B, dtype=np.int32)])
        meta = AttentionMetadata(
            num_reqs=Bp, num_actual_tokens=T, max_query_len=max_q, max_seq_len=max_s,
            query_start_loc=self.query_start_loc[:Bp + 1], seq_lens=self.seq_lens[:Bp],
            block_table=self.block_table[:Bp], slot_mapping=self.slot_mapping[:Tp],
            positions=self.positions[:Tp], query_start_loc_cpu=qsl_cpu, seq_lens_cpu=sl_cpu,
            attn_state=state, num_decodes=nd, num_decode_tokens=ndt, num_prefills=npf,
            num_input_tokens=Tp)
        meta.dcp_interleave = self.dcp_interleave
        if self.dcp_size > 1:
            from ..attention.dcp import local_seq_lens
            lsl = np.ones(Bp, dtype=np.int32)
            lsl[:B] = local_seq_lens(seq_lens, self.block_size, self.dcp_size, self.dcp_rank, self.dcp_interleave)
            if not hasattr(self, "_dcp_sl"):
                self._dcp_sl = torch.zeros(self.max_seqs + 8, dtype=torch.int32, device=self.device)
            self._dcp_sl[:Bp].copy_(torch.from_numpy(lsl), non_blocking=False)
            meta.dcp_seq_lens = self._dcp_sl[:Bp]
        meta.pcp = pcp_meta
        if self.sparse_offload is not None:
            tr = np.full(Tp, -1, dtype=np.int64)
            tr[:T] = rows[req_idx] if pcp_meta is None else -1
            pc_ = np.zeros(Tp, dtype=np.int64)
            pc_[:T] = pos
            meta.extra = dict(meta.extra or {}, tok_rows=tr, positions_cpu=pc_)
        if self.mm is not None:
            self.mm.prepare(reqs, starts, q_lens, cu, pos, req_idx, T, Tp, meta)
        if self.mcfg.is_hybrid:
            # recurrent layers index their state by the request's batch row; padded rows use the
            # scratch row
            hs = self._h_state
            hs[0, :B] = torch.from_numpy(rows.astype(np.int32))
            hs[1, :B] = torch.from_numpy((starts > 0).astype(np.int32))
            if Bp > B:
                hs[0, B:Bp] = self.max_seqs
                hs[1, B:Bp] = 0
            self.state_meta[:, :Bp].copy_(hs[:, :Bp], non_blocking=True)
            meta.state_slots = self.state_meta[0, :Bp]
            meta.has_initial_state = self.state_meta[1, :Bp]
        if self.is_cuda and not self.mcfg.use_mla:
            a = self._attn_layer()
            G = a.Hq // a.Hkv
            tok_per_tile = max(1, 128 // G)
            if max_q > 1:
                # decode sequences (leading, one token each) go to the decode kernel when it
                # supports the head layout; the work list then covers the rest
                skip = nd if (a.D == 128 and 16 % G == 0 and envs.VLLM_B200_DECODE_ATTN == "native") else 0
                ts, tq = build_tile_worklist(q_lens[skip:], tok_per_tile, seq_lens[skip:])
                ts = ts + np.int32(skip)
                if skip == 0:
                    meta.num_decodes = meta.num_decode_tokens = 0
                nt = len(ts)
                h._h_tile[0, :nt] = torch.from_numpy(ts)
                h._h_tile[1, :nt] = torch.from_numpy(tq)
                self.tile_seq[:nt].copy_(h._h_tile[0, :nt], non_blocking=True)
                self.tile_qoff[:nt].copy_(h._h_tile[1, :nt], non_blocking=True)
                meta.tile_seq, meta.tile_qoff, meta.num_tiles = self.tile_seq[:nt], self.tile_qoff[:nt], nt
                self.stats["h2d_bytes"] += nt * 8
            else:
                meta.num_splits = self._decode_splits(Bp, a.Hkv)
        logits_idx = None
        sample_reqs = []
        sel = []
        rows_per_req = []
        for i, r in enumerate(reqs):
            end = int(g_starts[i] + g_qlens[i])
            ntok = r.num_tokens + getattr(r, "num_inflight", 0)   # incl. a token still being sampled
            if end >= ntok:
                nrow = end - ntok + 1                  # 1 + draft tokens verified in this step
                base = int(g_cu[i + 1]) - nrow
                sel.extend(range(base, base + nrow))
                sample_reqs.append(r)
                rows_per_req.append(nrow)
        if inv is not None:
            # rows of this rank's hidden states; the last token of every chunk sits on PCP rank 0
            sel = [int(inv[g]) for g in sel]
            if self.pcp.rank_in_group != 0:
                sel = [-1] * len(sel)
        self._sample_rows = rows_per_req
        # chunk geometry of requests that asked for prompt log-probabilities
        self._plp_chunks = [(r, int(g_starts[i]), int(g_qlens[i]), int(g_cu[i])) for i, r in enumerate(reqs)
                            if getattr(getattr(r, "sampling_params", None), "prompt_logprobs", None) is not None
                            and int(g_starts[i]) < r.num_prompt_tokens - 1] if (inv is None and self.plp_enabled) else []
        return meta, T, Tp, sel, sample_reqs

    def _prompt_logprobs(self, hidden: torch.Tensor) -> None:
        """Log-probability of every prompt token given its prefix (plus the top-N alternatives) for
        the prompt chunks computed in this step: row p of a chunk predicts prompt token p + 1."""
        for r, s, n, cu in self._plp_chunks:
            P = r.num_prompt_tokens
            hi = min(s + n, P - 1)                     # positions s .. hi-1 predict tokens s+1 .. hi
            if hi <= s:
                continue
            k = int(r.sampling_params.prompt_logprobs)
            targets = torch.from_numpy(np.asarray(r.prompt_token_ids[s + 1:hi + 1], dtype=np.int64)).to(self.device)
            for a in range(0, hi - s, 1024):           # bounded logits footprint
                b = min(a + 1024, hi - s)
                lp = torch.log_softmax(self.model.compute_logits(hidden[cu + a:cu + b]).float(), dim=-1)
                tgt = targets[a:b]
                tok_lp = lp.gather(1, tgt.unsqueeze(1)).squeeze(1).cpu()
                if k > 0:
                    vals, ids = lp.topk(min(k, lp.shape[-1]), dim=-1)
                    vals, ids = vals.cpu(), ids.cpu()
                out = self._prompt_lp_out.setdefault(r.request_id, [])
                for j in range(b - a):
                    entry = {int(ids[j, q]): float(vals[j, q]) for q in range(ids.shape[1])} if k > 0 else {}
                    entry[int(tgt[j])] = float(tok_lp[j])
                    out.append((s + a + j + 1, entry))
        self._plp_chunks = []

    def take_prompt_logprobs(self) -> dict:
        out, self._prompt_lp_out = self._prompt_lp_out, {}
        return out

    def init_lora(self) -> None:
        from ..lora.manager import LoRAManager
        self.lora_manager = LoRAManager(self.model, self.cfg.max_loras, self.cfg.max_lora_rank,
                                        self.max_tokens + self.max_seqs, self.max_seqs, self.device,
                                        next(iter(self.model.named_parameters()))[1].dtype)

    def _update_lora(self, reqs, q_lens, padded_tokens: int) -> None:
        mgr = self.lora_manager
        in_use = {r.lora_request.lora_int_id for r in reqs if getattr(r, "lora_request", None) is not None}
        slots = []
        for r in reqs:
            lr = getattr(r, "lora_request", None)
            if lr is None:
                slots.append(-1)
                continue
            if not mgr.add(lr, in_use):
                raise RuntimeError(f"no adapter slot for LoRA {lr.lora_int_id}: raise max_loras")
            slots.append(mgr.slot_of(lr.lora_int_id))
        mgr.punica.update_metadata(slots, q_lens, padded_tokens)

    def _decode_splits(self, batch: int, Hkv: int) -> int:
        """Split factor depends only on the (padded) batch size so that it is a
        compile-time constant of the captured graph."""
        return ops.choose_num_splits(batch, Hkv, self.max_model_len, self.sm_count)

    # ------------------------------------------------------------------ execution
    def _forward(self, T: int, meta: AttentionMetadata) -> torch.Tensor:
        from ..profiler import nvtx_range
        with nvtx_range(f"forward[{T}]"):
            return self._forward_impl(T, meta)

    def _forward_impl(self, T: int, meta: AttentionMetadata) -> torch.Tensor:
        pp = self.pp
        emb = self.mm.inputs_embeds(self.input_ids[:T]) if self.mm is not None else None
        if emb is not None:
            meta.deepstack = self.mm.deepstack
        if pp.world_size == 1:
            if emb is not None:
                return self.model.forward(self.input_ids[:T], meta, self.kv_caches, inputs_embeds=emb)
            return self.model.forward(self.input_ids[:T], meta, self.kv_caches)
        # Pipeline stage: activations (hidden, residual) arrive from the previous stage and
        # leave for the next one; only the last stage returns final hidden states
        # (vllm_ascend/worker/worker.py:634-673 does the same with irecv/isend of a tensor dict).
        inter = None
        H, dt = self.mcfg.hidden_size, self.model.dtype
        if not self.model.is_first:
            h = torch.empty((T, H), dtype=dt, device=self.device)
            res = torch.empty((T, H), dtype=dt, device=self.device)
            pp.recv(h, pp.rank_in_group - 1)
            pp.recv(res, pp.rank_in_group - 1)
            inter = (h, res)
        out = self.model.forward(self.input_ids[:T], meta, self.kv_caches, inter, inputs_embeds=emb)
        if self.model.is_last:
            return out
        h, res = out
        pp.send(h.contiguous(), pp.rank_in_group + 1)
        pp.send((res if res is not None else h).contiguous(), pp.rank_in_group + 1)
        return h

    def _lora_step_needs_eager(self, so: SchedulerOutput) -> bool:
        lm = self.lora_manager
        return lm is not None and not lm.graph_safe and any(r.lora_request is not None for r, _ in so.scheduled)

    def _graph_size_for(self, B: int) -> Optional[int]:
        if not self.capture_sizes or B > self.capture_sizes[-1]:
            return None
        if self.moe_runtime is not None and not self.moe_runtime.graph_safe(B):
            return None          # some DP rank has too many tokens for the fused MoE path this step
        for s in self.capture_sizes:
            if s >= B:
                return s
        return None

    @torch.inference_mode()
    def execute(self, so: SchedulerOutput) -> dict:
        """Runs one step; returns {request_id: [sampled token ids]}."""
        if so.is_empty:
            return {}
        t_start = time.perf_counter()
        self.stats["steps"] += 1
        self._sync_rows(so)
        if self.pp.world_size > 1:
            return self._execute_pipeline(so)
        B = len(so.scheduled)
        decode_only = all(n == 1 for _, n in so.scheduled)
        gsize = self._graph_size_for(B) if decode_only else None
        if gsize is not None and self._lora_step_needs_eager(so):
            gsize = None
        meta, T, Tp, sel, sample_reqs = self._prepare_inputs(so, pad_to=gsize)
        t_prep = time.perf_counter()
        if gsize is not None:
            desc = self.graphs[(gsize, self.lora_manager is not None and self.lora_manager.punica.any_active)]
            hidden_out = self.graph_wrapper.replay(desc)
            self.stats["graph_replays"] += 1
            self.stats["graph_kernel_launches"] += self.graph_wrapper.entries[desc].num_launches
            self.last_hidden = hidden_out
            self._capture_pooled(hidden_out[:B], sample_reqs)
            logits = None if self._reduce_sample(sample_reqs) else self.model.compute_logits(hidden_out[:B])
        else:
            hidden = self._forward(Tp, meta)
            self.last_hidden = hidden
            self.stats["eager_steps"] += 1
            if self._plp_chunks:
                self._prompt_logprobs(hidden)
            if not sel:
                self._meet_lm_head(hidden)
                return {}
            if self._pcp_bcast:
                return self._sample_pcp(hidden, sel, sample_reqs)
            if len(sel) == T:
                h_sel = hidden[:T]
            else:
                h_sel = hidden[torch.tensor(sel, dtype=torch.int64, device=self.device)]
            self._capture_pooled(h_sel, sample_reqs)
            logits = None if self._reduce_sample(sample_reqs) else self.model.compute_logits(h_sel)
        if logits is None:
            tokens = self.model.lm_head.greedy_tokens(h_sel if gsize is None else hidden_out[:B])
        if logits is not None and any(k > 1 for k in self._sample_rows):
            out = self._sample_speculative(logits, sample_reqs, self._sample_rows)
            t_sync = time.perf_counter()
            self.stats["t_spec"] = self.stats.get("t_spec", 0.0) + (t_sync - t_start)
            self.stats["n_spec"] = self.stats.get("n_spec", 0) + 1
            return out
        if logits is not None:
            md = SamplingMetadata.build(sample_reqs, self.device, self.mcfg.vocab_size, self.cfg.seed)
            if not md.all_greedy and not self.is_cuda:
                md.generator = self._cpu_generator()
            tokens = self.sampler(logits, md)
        dev_lp = self._device_logprobs(logits, tokens, sample_reqs)
        n = tokens.shape[0]
        t_launch = time.perf_counter()
        if self.is_cuda:
            self._h_sampled[:n].copy_(tokens, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            toks = self._h_sampled[:n].numpy()
        else:
            toks = tokens.numpy()
        self._store_logprobs(dev_lp, sample_reqs, toks)
        self.stats["d2h_bytes"] += n * 8
        t_sync = time.perf_counter()
        key = "decode" if gsize is not None else ("decode_eager" if decode_only else "mixed")
        self.stats["t_" + key] = self.stats.get("t_" + key, 0.0) + (t_sync - t_start)
        self.stats["n_" + key] = self.stats.get("n_" + key, 0) + 1
        self.stats["t_prepare"] += t_prep - t_start
        self.stats["t_launch"] += t_launch - t_prep
        self.stats["t_wait"] += t_sync - t_launch
        out = {}
        for r, t in zip(sample_reqs, toks):
            t = int(t)
            row = r.row
            self.token_ids_cpu[row, r.num_tokens] = t
            out[r.request_id] = [t]
        return out

    def _sample_pcp(self, hidden: torch.Tensor, sel: list, sample_reqs: list) -> dict:
        """Split prefill step: PCP rank 0 holds the last token of every chunk, samples, and sends
        the token ids to the other ranks of the group."""
        n = len(sel)
        if self.pcp.rank_in_group == 0:
            h_sel = hidden[torch.tensor(sel, dtype=torch.int64, device=self.device)]
            logits = self.model.compute_logits(h_sel)
            md = SamplingMetadata.build(sample_reqs, self.device, self.mcfg.vocab_size, self.cfg.seed)
            if not md.all_greedy and not self.is_cuda:
                md.generator = self._cpu_generator()
            tokens = self.sampler(logits, md).to(torch.int64)
            dev_lp = self._device_logprobs(logits, tokens, sample_reqs)
        else:
            tokens = torch.zeros(n, dtype=torch.int64, device=self.device)
            dev_lp = None
        tokens = self.pcp.broadcast(tokens.contiguous(), src=0)
        toks = tokens.cpu().numpy()
        if any(r.sampling_params.logprobs is not None for r in sample_reqs):
            # every rank of the group reports the same log-probabilities
            host_lp = None if dev_lp is None else tuple(t.cpu() for t in dev_lp)
            host_lp = self.pcp.broadcast_object(host_lp, src=0)
            self._store_logprobs(host_lp, sample_reqs, toks)
        out = {}
        for r, t in zip(sample_reqs, toks):
            self.token_ids_cpu[r.row, r.num_tokens] = int(t)
            out[r.request_id] = [int(t)]
        return out

    # ------------------------------------------------------------------ asynchronous stepping
    @torch.inference_mode()
    def execute_async(self, so: SchedulerOutput, prev=None, defer_sampling: bool = False):
        """Enqueue one step without waiting for its result.  Tokens that the previous step
        (``prev``, still running) is sampling are not known on the host: they are copied on the
        device from its output into this step's input ids.  Returns a handle for ``collect``.

        ``defer_sampling``: stop after the forward pass and keep the hidden rows of the sampling
        positions in the handle; ``finish_sampling`` computes the logits and samples later, when a
        caller-side constraint on the logits (a host engine's grammar bitmask for this very step)
        has arrived."""
        if so.is_empty:
            return None
        t_start = time.perf_counter()
        self.stats["steps"] += 1
        self._sync_rows(so)
        B = len(so.scheduled)
        decode_only = all(n == 1 for _, n in so.scheduled)
        gsize = self._graph_size_for(B) if decode_only else None
        if gsize is not None and self._lora_step_needs_eager(so):
            gsize = None
        ev_start = None
        if self._step_timing:
            # device-side account of the step: time between the first and the last GPU operation of
            # the step, and the idle gap since the previous step's last one
            ev_start = torch.cuda.Event(enable_timing=True)
            ev_start.record()
        meta, T, Tp, sel, sample_reqs = self._prepare_inputs(so, pad_to=gsize)
        if prev is not None:
            src, dst = [], []
            off = 0
            for req, n in so.scheduled:
                off += n
                if req.num_inflight > 0:
                    j = prev.index.get(req.request_id)
                    if j is not None:
                        src.append(j)
                        dst.append(off - 1)          # the pending token is the last one scheduled
            if src:
                idx = self._to_dev(torch.tensor([src, dst], dtype=torch.int64))
                self.input_ids.index_copy_(0, idx[1], prev.tokens.index_select(0, idx[0]))
        t_prep = time.perf_counter()
        if gsize is not None:
            desc = self.graphs[(gsize, self.lora_manager is not None and self.lora_manager.punica.any_active)]
            hidden_out = self.graph_wrapper.replay(desc)
            self.stats["graph_replays"] += 1
            self.stats["graph_kernel_launches"] += self.graph_wrapper.entries[desc].num_launches
            self.last_hidden = hidden_out
            h_sel = hidden_out[:B]
        else:
            hidden = self._forward(Tp, meta)
            self.last_hidden = hidden
            self.stats["eager_steps"] += 1
            if self._plp_chunks:
                self._prompt_logprobs(hidden)
            if not sel:
                return _StepHandle(None, [], None, None, "mixed", t_start)
            h_sel = hidden[:T] if len(sel) == T else hidden[self._to_dev(torch.tensor(sel, dtype=torch.int64))]
        self._capture_pooled(h_sel, sample_reqs)
        kind = "decode" if gsize is not None else ("decode_eager" if decode_only else "mixed")
        handle = _StepHandle(None, sample_reqs, None, None, kind, t_start)
        handle.ev_start = ev_start
        handle.num_tokens = T
        self.stats["t_prepare"] += t_prep - t_start
        if defer_sampling:
            handle.h_sel = h_sel
            self.stats["t_launch"] += time.perf_counter() - t_prep
            return handle
        self._sample_into(handle, h_sel, None)
        self.stats["t_launch"] += time.perf_counter() - t_prep
        return handle

    def finish_sampling(self, handle, allowed: Optional[dict] = None):
        """Second half of a step enqueued with ``defer_sampling``.  ``allowed``: request id -> bool
        tensor [vocab] (True = token may be sampled) for the requests whose logits are constrained."""
        if handle is None or handle.h_sel is None:
            return handle
        h_sel, handle.h_sel = handle.h_sel, None
        self._sample_into(handle, h_sel, allowed)
        return handle

    def _sample_into(self, handle, h_sel: torch.Tensor, allowed: Optional[dict]) -> None:
        sample_reqs = handle.reqs
        dev_lp = None
        if not allowed and self._reduce_sample(sample_reqs):
            tokens = self.model.lm_head.greedy_tokens(h_sel)
        else:
            logits = self.model.compute_logits(h_sel)
            if allowed:
                rows = [i for i, r in enumerate(sample_reqs) if r.request_id in allowed]
                if rows:
                    mask = torch.stack([allowed[sample_reqs[i].request_id] for i in rows]).to(logits.device)
                    idx = torch.tensor(rows, dtype=torch.int64, device=logits.device)
                    sub = logits.index_select(0, idx)
                    logits.index_copy_(0, idx, sub.masked_fill(~mask[:, :sub.shape[1]], float("-inf")))
            md = SamplingMetadata.build(sample_reqs, self.device, self.mcfg.vocab_size, self.cfg.seed)
            if not md.all_greedy and not self.is_cuda:
                md.generator = self._cpu_generator()
            tokens = self.sampler(logits, md)
            dev_lp = self._device_logprobs(logits, tokens, sample_reqs)
        n = tokens.shape[0]
        buf = self._h_sampled2[self._async_flip]
        self._async_flip ^= 1
        buf[:n].copy_(tokens, non_blocking=True)
        ev = None
        if self.is_cuda:
            ev = torch.cuda.Event(enable_timing=self._step_timing)
            ev.record()
        self.stats["d2h_bytes"] += n * 8
        handle.tokens, handle.host, handle.event = tokens, buf, ev
        handle.logprobs = dev_lp

    def _reduce_sample(self, sample_reqs: list) -> bool:
        """Greedy batches on a vocabulary-sharded LM head pick their tokens from per-rank
        (max, index) pairs instead of gathering [B, vocab] logits on every rank."""
        head = self.model.lm_head
        if head.comm.size <= 1 or any(k > 1 for k in self._sample_rows):
            return False
        return all(r.sampling_params.greedy and not r.sampling_params.has_penalties
                   and not r.sampling_params.has_processors and r.sampling_params.logprobs is None
                   for r in sample_reqs)

    def _device_logprobs(self, logits, tokens, sample_reqs):
        """(token logprob, top ids, top values) on the device when a request of the step asked for
        log-probabilities, else None."""
        ks = [r.sampling_params.logprobs for r in sample_reqs]
        if logits is None or all(k is None for k in ks):
            return None
        from ..sample.sampler import compute_logprobs
        return compute_logprobs(logits, tokens, max(int(k or 0) for k in ks))

    def _store_logprobs(self, dev_lp, sample_reqs, toks) -> None:
        if dev_lp is None:
            return
        tok_lp, ids, vals = (t.cpu() for t in dev_lp)
        for i, r in enumerate(sample_reqs):
            k = r.sampling_params.logprobs
            if k is None:
                continue
            entry = {int(ids[i, j]): float(vals[i, j]) for j in range(min(int(k), ids.shape[1]))}
            entry[int(toks[i])] = float(tok_lp[i])
            self._logprobs_out.setdefault(r.request_id, []).append(entry)

    def _capture_pooled(self, h_sel: torch.Tensor, sample_reqs: list) -> None:
        """Embedding requests keep the final hidden state of their last prompt token."""
        if len(self._sample_rows) != len(sample_reqs) or any(k != 1 for k in self._sample_rows):
            return
        for i, r in enumerate(sample_reqs):
            ea = r.sampling_params.extra_args
            if ea and ea.get("pooling") and r.num_output_tokens == 0:
                r.pooled = h_sel[i].float().cpu()

    def take_logprobs(self) -> dict:
        out, self._logprobs_out = self._logprobs_out, {}
        return out

    def _to_dev(self, t: torch.Tensor) -> torch.Tensor:
        """Host index tensor to the device without blocking the host on the stream."""
        return t.pin_memory().to(self.device, non_blocking=True) if self.is_cuda else t

    def collect(self, handle) -> dict:
        """Wait for a step enqueued by ``execute_async`` and return its sampled tokens."""
        if handle is None or handle.tokens is None:
            return {}
        t0 = time.perf_counter()
        if handle.event is not None:
            handle.event.synchronize()
            if getattr(handle, "ev_start", None) is not None:
                st = self.stats
                st["gpu_ms_" + handle.kind] = st.get("gpu_ms_" + handle.kind, 0.0) + handle.ev_start.elapsed_time(handle.event)
                if self._last_step_end is not None:
                    st["gpu_idle_ms"] = st.get("gpu_idle_ms", 0.0) + max(0.0, self._last_step_end.elapsed_time(handle.ev_start))
                self._last_step_end = handle.event
        toks = handle.host[:len(handle.reqs)].numpy()
        self._store_logprobs(handle.logprobs, handle.reqs, toks)
        out = {}
        for r, t in zip(handle.reqs, toks):
            t = int(t)
            if r.row >= 0 and self.row_owner[r.row] == r.request_id:
                self.token_ids_cpu[r.row, r.num_tokens] = t
            out[r.request_id] = [t]
        now = time.perf_counter()
        self.stats["t_wait"] += now - t0
        self.stats["t_" + handle.kind] = self.stats.get("t_" + handle.kind, 0.0) + (now - handle.t_start)
        self.stats["n_" + handle.kind] = self.stats.get("n_" + handle.kind, 0) + 1
        return out

    def _execute_pipeline(self, so: SchedulerOutput) -> dict:
        """One step of a pipeline-parallel engine: every stage runs its layers, the last stage
        samples and the sampled tokens go back to all stages, whose schedulers advance together."""
        meta, T, Tp, sel, sample_reqs = self._prepare_inputs(so)
        hidden = self._forward(Tp, meta)
        self.stats["eager_steps"] += 1
        pp = self.pp
        toks = None
        if self.model.is_last and sel:
            h_sel = hidden[:T] if len(sel) == T else hidden[torch.tensor(sel, dtype=torch.int64, device=self.device)]
            logits = self.model.compute_logits(h_sel)
            md = SamplingMetadata.build(sample_reqs, self.device, self.mcfg.vocab_size, self.cfg.seed)
            if not md.all_greedy and not self.is_cuda:
                md.generator = self._cpu_generator()
            tokens = self.sampler(logits, md)
            dev_lp = self._device_logprobs(logits, tokens, sample_reqs)
            toks = (tokens.cpu().tolist(), None if dev_lp is None else tuple(t.cpu() for t in dev_lp))
        toks = pp.broadcast_object(toks, src=pp.world_size - 1)
        if toks is not None:
            toks, host_lp = toks
            self._store_logprobs(host_lp, sample_reqs, toks)
        out = {}
        for r, t in zip(sample_reqs, toks or []):
            self.token_ids_cpu[r.row, r.num_tokens] = int(t)
            out[r.request_id] = [int(t)]
        return out

    def _sample_speculative(self, logits: torch.Tensor, sample_reqs: list, rows: list) -> dict:
        """Verification step: ``rows[i]`` logits rows belong to request i (its last accepted
        token followed by rows[i]-1 draft tokens).  Every row is sampled with the request's own
        parameters (the last row gives the bonus token), then the rejection sampler decides how
        many draft tokens stand."""
        from ..sample.rejection_sampler import RejectionSampler
        if self.rejection_sampler is None:
            from ..platform_config import get_b200_config
            rc = get_b200_config().rejection_sampler_config
            method = "block_verify" if rc.enable_block_verify else (
                "entropy_verify" if rc.enable_entropy_verify else "standard")
            self.rejection_sampler = RejectionSampler(method, rc.posterior_alpha, rc.posterior_threshold)
        dev = self.device
        # row j of a request sees the request's history extended by its first j draft tokens: logit
        # processors, penalties and the position in the random stream are those of a step that
        # had really generated them
        expanded = [_SpecRow(r, j) for r, k in zip(sample_reqs, rows) for j in range(k)]
        md = SamplingMetadata.build(expanded, dev, self.mcfg.vocab_size, self.cfg.seed)
        if not md.all_greedy and not self.is_cuda:
            md.generator = self._cpu_generator()
        processed = self.sampler.apply_processors(logits.float(), md)
        cu_rows = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
        last_rows = torch.from_numpy(cu_rows[1:] - 1).to(dev)
        draft_rows = torch.from_numpy(np.concatenate([np.arange(cu_rows[i], cu_rows[i + 1] - 1)
                                                      for i in range(len(rows))]).astype(np.int64)).to(dev)
        target_logits = processed[draft_rows]
        target_probs = None
        if not md.all_greedy and draft_rows.numel():
            target_probs = self.sampler.filtered_probs(target_logits, md, draft_rows)
        tokens_all = self.sampler.sample_processed(processed.clone() if not md.all_greedy else processed,
                                                   md).to(torch.int32)
        draft = np.concatenate([np.asarray(r.spec_token_ids[:k - 1], dtype=np.int32)
                                for r, k in zip(sample_reqs, rows)]) if draft_rows.numel() else np.zeros(0, np.int32)
        cu_draft = torch.from_numpy((cu_rows - np.arange(len(rows) + 1)).astype(np.int32)).to(dev)
        is_greedy = torch.tensor([r.sampling_params.greedy for r in sample_reqs], dtype=torch.bool, device=dev)
        temp = torch.tensor([max(r.sampling_params.temperature, 1e-5) for r in sample_reqs], dtype=torch.float32,
                            device=dev)
        max_spec = max(rows) - 1
        first_rows = torch.from_numpy(cu_rows[:-1]).to(dev)
        out, num = self.rejection_sampler(
            torch.from_numpy(draft).to(dev), cu_draft, target_logits, tokens_all[last_rows].contiguous(),
            is_greedy, temp, max_spec, target_probs=target_probs,
            seeds=None if md.seeds is None else md.seeds[first_rows],
            offsets=None if md.offsets is None else md.offsets[first_rows])
        out_h, num_h = out.cpu().numpy(), num.cpu().numpy()
        self.stats["d2h_bytes"] += out_h.nbytes + num_h.nbytes
        res = {}
        for i, r in enumerate(sample_reqs):
            toks = [int(t) for t in out_h[i, :num_h[i]]]
            self.token_ids_cpu[r.row, r.num_tokens:r.num_tokens + len(toks)] = toks
            res[r.request_id] = toks
            if self.dynamic_spec is not None:
                self.dynamic_spec.update(r.request_id, rows[i] - 1, max(int(num_h[i]) - 1, 0))
        self.spec_stats["draft_tokens"] += int(draft.size)
        self.spec_stats["accepted_tokens"] += int(np.maximum(num_h - 1, 0).sum())
        self.spec_stats["verify_steps"] += 1
        return res

    def propose_draft_tokens(self, reqs: list) -> None:
        """Fill ``req.spec_token_ids`` for running decode requests (after their tokens of this
        step were appended)."""
        if self.proposer is None or not reqs:
            return
        rows = np.fromiter((r.row for r in reqs), dtype=np.int64, count=len(reqs))
        lens = np.fromiter((r.num_tokens for r in reqs), dtype=np.int64, count=len(reqs))
        props = self.proposer.propose(self.token_ids_cpu, lens, rows)
        budgets = None
        if self.dynamic_spec is not None:
            # confidences of this step's draft tokens, when the proposer has them ([B, k], padded with 0)
            budgets = self.dynamic_spec.budgets([r.request_id for r in reqs],
                                                getattr(self.proposer, "last_token_probs", None))
        for i, (r, p) in enumerate(zip(reqs, props)):
            left = r.sampling_params.max_tokens - r.num_output_tokens - 1
            if budgets is not None:
                left = min(left, budgets[i])
            r.spec_token_ids = [int(t) for t in p[:max(left, 0)]]

    @torch.inference_mode()
    def execute_dummy(self) -> None:
        """Forward of one padding token that writes nothing to the KV cache; used by idle
        data-parallel ranks so collectives inside the model still match up."""
        meta, T, Tp, _, _ = self._dummy_meta(1, 1)
        meta.slot_mapping.fill_(-1)
        hidden = self._forward(Tp, meta)
        self._meet_lm_head(hidden)

    @torch.inference_mode()
    def profile_prefill_latency(self, num_tokens: int) -> float:
        """Seconds of one prefill-shaped forward of ``num_tokens`` tokens of a single sequence that
        writes nothing to the KV cache (the start-up profiling of the chunk-size predictor,
        vllm_ascend/worker/worker.py profile_prefill_latency)."""
        import time
        n = int(max(1, min(num_tokens, self.max_tokens, self.max_model_len - 1)))
        meta, T, Tp, _, _ = self._dummy_meta(1, n)
        meta.slot_mapping.fill_(-1)
        if self.is_cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        self._forward(Tp, meta)
        if self.is_cuda:
            torch.cuda.synchronize()
        return time.perf_counter() - t0

    def _meet_lm_head(self, hidden: torch.Tensor) -> None:
        """A rank with nothing to sample still joins the LM head's collectives when the head is
        sharded over a fine-grained TP group."""
        from ..parallel.finegrained import get_fg
        fg = get_fg()
        if fg is not None and fg.lmtp is not None and self.model.is_last:
            self.model.compute_logits(hidden[:0])

    def total_launches(self) -> int:
        """Launches of this package's own kernels so far (eager + inside replayed graphs)."""
        return ops.launch_counter[0] + self.stats["graph_kernel_launches"]

    def _cpu_generator(self) -> torch.Generator:
        g = getattr(self, "_gen", None)
        if g is None:
            g = torch.Generator()
            g.manual_seed(self.cfg.seed)
            self._gen = g
        return g

    # ------------------------------------------------------------------ warm-up / capture
    def _dummy_meta(self, B: int, q_len: int, pad_to: Optional[int] = None):
        """Synthetic batch of B sequences of q_len tokens over block 0."""
        class _R:  # minimal request stand-in
            pass
        sched = []
        for i in range(B):
            r = _R()
            r.row, r.num_computed_tokens, r.num_tokens = i, 0, q_len + 1
            r.request_id = f"_dummy{i}"
            sched.append((r, q_len))
        so = SchedulerOutput(scheduled=sched)
        saved = self.block_table_cpu[:B].copy()
        self.block_table_cpu[:B] = 0
        try:
            return self._prepare_inputs(so, pad_to=pad_to)
        finally:
            self.block_table_cpu[:B] = saved

    @torch.inference_mode()
    def warmup(self) -> None:
        """One prefill-shaped and one decode-shaped eager pass (kernel attribute setup,
        allocator warm-up) before any capture."""
        B = min(self.max_seqs, 8)
        q = max(1, min(self.max_tokens // B, self.max_model_len - 1, 256))
        meta, T, Tp, _, _ = self._dummy_meta(B, q)
        from ..parallel.finegrained import get_fg
        if get_fg() is not None:            # every rank warms up with the same shapes
            get_fg().max_tokens, get_fg().max_rows = Tp, B
        meta.slot_mapping.fill_(-1)
        h = self._forward(Tp, meta)
        self.model.compute_logits(h[:B])
        meta, T, Tp, _, _ = self._dummy_meta(B, 1)
        meta.slot_mapping.fill_(-1)
        self._forward(Tp, meta)
        if self.is_cuda:
            torch.cuda.synchronize()

    def drop_graphs(self) -> None:
        """Forget every captured graph; decode steps run eagerly until the next capture."""
        self.graphs.clear()
        self.capture_sizes = []
        if self.graph_wrapper is not None:
            self.graph_wrapper.clear()
        if self.mm is not None and self.mm.encoder_graphs is not None:
            self.mm.encoder_graphs.buckets.clear()

    @torch.inference_mode()
    def capture_graphs(self) -> None:
        cc = self.cfg.compilation
        if not self.is_cuda or cc.cudagraph_mode == "NONE" or not envs.VLLM_B200_CUDA_GRAPH:
            return
        if self.dcp_size > 1:
            return          # context-parallel steps read per-step host metadata: not captured
        max_size = cc.max_cudagraph_capture_size or min(self.max_seqs, 1024)
        sizes = cc.cudagraph_capture_sizes or default_capture_sizes(max_size)
        self.capture_sizes = sorted(set(int(s) for s in sizes if s <= self.max_seqs))
        if self.moe_runtime is not None:
            # expert-parallel steps are only capturable on the fused dispatch/combine path
            self.moe_runtime.max_tokens_across_dp = 0
            self.capture_sizes = [s for s in self.capture_sizes if self.moe_runtime.graph_safe(s)]
            if not self.capture_sizes:
                return
        # scratch for split-KV partials must exist before capture
        if not self.mcfg.use_mla:
            a = self._attn_layer()
            worst = 0
            for s in self.capture_sizes:
                ns = self._decode_splits(s, a.Hkv)
                if ns > 1:
                    worst = max(worst, s * a.Hq * ns * (a.D + 1) * 4)
            if worst:
                ops.reserve_attention_scratch(self.device, worst)
        from ..compilation.cuda_graph import BatchDescriptor, CUDAGraphWrapper, global_graph_pool
        self.graph_pool = global_graph_pool()

        def warm(Tp, meta):
            self.model.compute_logits(self._forward(Tp, meta))
        self.graph_wrapper = CUDAGraphWrapper(self._forward, cc.cudagraph_mode, self.graph_pool,
                                              launch_counter=ops.launch_counter)
        # with adapters enabled every size is captured twice: the LoRA kernels are part of the
        # graph only when some request of the step uses an adapter
        variants = [False, True] if (self.lora_manager is not None and self.lora_manager.graph_safe) else [False]
        for size in sorted(self.capture_sizes, reverse=True):
            for has_lora in variants:
                meta, T, Tp, _, _ = self._dummy_meta(size, 1)
                meta.slot_mapping.fill_(-1)
                if self.lora_manager is not None:
                    self.lora_manager.punica.any_active = has_lora
                desc = BatchDescriptor(num_tokens=size, has_lora=has_lora)
                self.graph_wrapper.capture(desc, Tp, meta, warmup=warm)
                self.graphs[(size, has_lora)] = desc
        if self.lora_manager is not None:
            self.lora_manager.punica.any_active = False
        torch.cuda.synchronize()
