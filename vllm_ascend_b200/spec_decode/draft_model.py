"""Model-based proposers: a separate small draft model, or an EAGLE/MTP-style head that is
conditioned on the target model's hidden states and shares its embeddings and LM head.

Both keep their own paged KV cache but reuse the target's block tables, so a draft position
lives in the same (block, offset) as the target position.  Each engine step the proposer
first catches up on the positions the target has just made final, then runs K-1 further
single-token steps on its own predictions (vllm_ascend/spec_decode/llm_base_proposer.py:
sharing of embeddings/LM head 354-495, K draft steps 718-1340, input preparation 1795-2025).
Draft tokens are argmax picks, i.e. deterministic proposals for the rejection sampler.
"""
from __future__ import annotations

import copy
import os
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..config import get_model_config
from ..engine.scheduler import SchedulerOutput
from ..models.layers import ParamFactory, RMSNorm, TPComm
from ..parallel import state as pstate


class _Standin:
    """What ``ModelRunner._prepare_inputs`` reads from a request."""
    spec_token_ids: list = []
    lora_request = None

    def __init__(self, row: int, start: int, end: int, rid: str):
        self.row, self.num_computed_tokens, self.num_tokens, self.request_id = row, start, end, rid


class EagleHead:
    """h_0 = fc([embed(token_{i+1}); hidden_i]) -> one decoder layer -> norm -> shared LM head."""

    def __init__(self, target, cfg, device, max_model_len: int, seed_name: str = "eagle"):
        from ..models.transformer import DecoderLayer
        dtype = target.embed_tokens.weight.dtype
        dcfg = copy.copy(cfg)
        dcfg.num_experts = 0
        pf = ParamFactory(dcfg, device, dtype)
        comm = TPComm(pstate.get_tp_group())
        self.embed_tokens = target.embed_tokens
        self.lm_head = target.lm_head
        H = cfg.hidden_size
        self.fc_weight = pf.normal(f"{seed_name}.fc", (H, 2 * H))
        self.layers = [DecoderLayer(pf, dcfg, 10_000, comm, max_model_len)]
        self.norm = RMSNorm(pf, H, cfg.rms_norm_eps)

    def forward(self, input_ids, prev_hidden, meta, kv_caches):
        x = torch.cat([self.embed_tokens(input_ids), prev_hidden.to(self.fc_weight.dtype)], dim=-1)
        h = ops.linear(x, self.fc_weight, None, None)
        residual = None
        for layer, cache in zip(self.layers, kv_caches):
            h, residual = layer(h, residual, meta, cache)
        out, _ = self.norm(h, residual)
        return out

    def compute_logits(self, hidden):
        return self.lm_head(hidden)


class MTPHead:
    """Multi-token-prediction module of DeepSeek-V3 style checkpoints: layer N = num_hidden_layers.
    h_0 = eh_proj([enorm(embed(token_{i+1})); hnorm(hidden_i)]) -> one full decoder layer of the
    target's own kind (MLA / MoE included) -> shared_head.norm -> LM head shared with the target.
    Weight names: ``model.layers.N.{enorm,hnorm,eh_proj,shared_head.norm,shared_head.head}`` next to
    the layer's ordinary ``self_attn`` / ``mlp`` tensors.  Role of the MTP proposer the reference
    runs through its base proposer (vllm_ascend/spec_decode/llm_base_proposer.py, models/deepseek_mtp)."""

    def __init__(self, target, cfg, device, max_model_len: int, ep_group=None, moe_runtime=None):
        from ..models.transformer import DecoderLayer
        dtype = target.embed_tokens.weight.dtype
        pf = ParamFactory(cfg, device, dtype)
        comm = TPComm(pstate.get_tp_group())
        self.cfg = cfg
        self.comm = comm
        H, N = cfg.hidden_size, cfg.num_hidden_layers
        self.idx = N
        self.embed_tokens = target.embed_tokens
        self.lm_head = target.lm_head
        self.enorm = RMSNorm(pf, H, cfg.rms_norm_eps)
        self.hnorm = RMSNorm(pf, H, cfg.rms_norm_eps)
        self.eh_proj_weight = pf.normal(f"model.layers.{N}.eh_proj", (H, 2 * H))
        self.layers = [DecoderLayer(pf, cfg, N, comm, max_model_len, ep_group, moe_runtime)]
        self.norm = RMSNorm(pf, H, cfg.rms_norm_eps)

    def forward(self, input_ids, prev_hidden, meta, kv_caches):
        e, _ = self.enorm(self.embed_tokens(input_ids))
        h, _ = self.hnorm(prev_hidden.to(e.dtype).contiguous())
        x = ops.linear(torch.cat([e, h], dim=-1), self.eh_proj_weight, None, None)
        h, residual = self.layers[0](x, None, meta, kv_caches[0])
        out, _ = self.norm(h, residual)
        return out

    def compute_logits(self, hidden):
        return self.lm_head(hidden)

    def load_weights(self, weights) -> set:
        """Picks the tensors of layer N out of a full checkpoint stream (the target skips them)."""
        from ..models.transformer import CausalLM
        N = self.idx
        pre = f"model.layers.{N}."
        own = {f"{pre}enorm.weight": self.enorm.weight, f"{pre}hnorm.weight": self.hnorm.weight,
               f"{pre}eh_proj.weight": self.eh_proj_weight, f"{pre}shared_head.norm.weight": self.norm.weight}
        loaded, rest = set(), []
        for name, w in weights:
            if not name.startswith(pre):
                continue
            if name in own:
                own[name].copy_(w.to(own[name].dtype))
                loaded.add(name)
            elif "shared_head.head" in name or "embed_tokens" in name:
                loaded.add(name)                       # tied to the target's embedding / LM head
            else:
                rest.append((name, w))
        # the decoder layer itself loads through the target's loader (same sharding rules)
        shell = CausalLM.__new__(CausalLM)
        shell.cfg, shell.comm, shell.layers = self.cfg, self.comm, self.layers
        shell.named_parameters = lambda: ((n, t) for n, t in CausalLM.named_parameters(shell)
                                          if n.startswith(pre))
        shell.embed_tokens, shell.norm, shell.lm_head = self.embed_tokens, self.norm, self.lm_head
        loaded |= CausalLM.load_weights(shell, rest)
        return loaded


class Eagle3Head:
    """EAGLE-3 draft head.  Conditioning is the target's residual stream at three depths (low, middle,
    high), concatenated and projected by ``fc``; the single decoder layer attends over
    [norm(embed(token_{i+1})); norm(h_i)] (a 2H-wide qkv input) and its pre-norm output is the
    conditioning of the next draft step.  The head may predict over a reduced draft vocabulary;
    ``d2t`` maps a draft index to its target token id (index + offset).  Architecture of the
    eagle3 proposer the reference drives (vllm_ascend/spec_decode/llm_base_proposer.py:354-495 with
    upstream llama_eagle3)."""

    def __init__(self, target, cfg, device, max_model_len: int, seed_name: str = "eagle3",
                 draft_vocab_size: Optional[int] = None):
        from ..models.layers import ColumnParallelLinear, ParallelLMHead, VocabParallelEmbedding
        from ..models.transformer import DecoderLayer
        dtype = target.embed_tokens.weight.dtype
        dcfg = copy.copy(cfg)
        dcfg.num_experts = 0
        dcfg.full_attention_interval = 0
        pf = ParamFactory(dcfg, device, dtype)
        comm = TPComm(pstate.get_tp_group())
        H = cfg.hidden_size
        self.H = H
        self.embed_tokens = target.embed_tokens
        self.fc_weight = pf.normal(f"{seed_name}.fc", (H, 3 * H))
        layer = DecoderLayer(pf, dcfg, 10_000, comm, max_model_len)
        a = layer.self_attn
        kv_out = a.total_kv * a.D if a.total_kv >= comm.size else comm.size * a.D
        a.qkv_proj = ColumnParallelLinear(pf, f"{seed_name}.midlayer.self_attn.qkv_proj", 2 * H,
                                          [cfg.num_attention_heads * a.D, kv_out, kv_out], comm,
                                          bias=cfg.attention_bias)
        self.layers = [layer]
        self.hidden_norm = RMSNorm(pf, H, cfg.rms_norm_eps)
        self.norm = RMSNorm(pf, H, cfg.rms_norm_eps)
        self.d2t = None
        if draft_vocab_size and draft_vocab_size < cfg.vocab_size:
            head = VocabParallelEmbedding(pf, f"{seed_name}.lm_head", draft_vocab_size, H, comm)
            self.lm_head = ParallelLMHead(head)
            self.d2t = torch.zeros(draft_vocab_size, dtype=torch.int64, device=device)
        else:
            self.lm_head = target.lm_head

    def forward(self, input_ids, prev_hidden, meta, kv_caches):
        """prev_hidden: [T, 3H] target residual streams (first pass) or [T, H] own pre-norm output."""
        layer = self.layers[0]
        hs = prev_hidden.to(self.fc_weight.dtype)
        if hs.shape[-1] == 3 * self.H:
            hs = ops.linear(hs, self.fc_weight, None, None)
        emb, _ = layer.input_layernorm(self.embed_tokens(input_ids))
        hn, _ = self.hidden_norm(hs)
        attn = layer.self_attn(torch.cat([emb, hn], dim=-1), meta, kv_caches[0])
        x, residual = layer.post_attention_layernorm(attn, hs.contiguous())
        return layer.mlp(x) + residual                       # pre-norm: conditions the next draft step

    def compute_logits(self, hidden):
        out, _ = self.norm(hidden)
        return self.lm_head(out)

    def draft_tokens(self, hidden) -> torch.Tensor:
        idx = self.compute_logits(hidden).argmax(-1)
        return idx if self.d2t is None else idx + self.d2t[idx]

    def named_parameters(self):
        L = self.layers[0]
        yield "fc.weight", self.fc_weight
        yield "midlayer.input_layernorm.weight", L.input_layernorm.weight
        yield "midlayer.hidden_norm.weight", self.hidden_norm.weight
        yield "midlayer.post_attention_layernorm.weight", L.post_attention_layernorm.weight
        for attr in ("qkv_proj", "o_proj"):
            for n, t in getattr(L.self_attn, attr).named_tensors():
                yield f"midlayer.self_attn.{attr}.{n}", t
        for attr in ("gate_up_proj", "down_proj"):
            for n, t in getattr(L.mlp, attr).named_tensors():
                yield f"midlayer.mlp.{attr}.{n}", t
        yield "norm.weight", self.norm.weight
        if self.d2t is not None:
            yield "lm_head.weight", self.lm_head.weight
            yield "d2t", self.d2t

    def load_weights(self, weights) -> set:
        """HF EAGLE-3 checkpoint names (``fc``, ``midlayer.*`` / ``layers.0.*``, ``norm``, ``lm_head``,
        ``d2t``); q/k/v and gate/up are merged.  Single-rank layout (draft heads are small: every TP
        rank would load its slice the same way the target does)."""
        params = dict(self.named_parameters())
        L = self.layers[0].self_attn
        nq, nkv = L.Hq * L.D, L.Hkv * L.D
        loaded = set()
        for name, w in weights:
            n = name.replace("model.", "", 1) if name.startswith("model.") else name
            n = n.replace("layers.0.", "midlayer.")
            tgt, rows = n, None
            for hf, (lo, hi) in (("q_proj", (0, nq)), ("k_proj", (nq, nq + nkv)), ("v_proj", (nq + nkv, nq + 2 * nkv))):
                if f".{hf}." in n:
                    tgt, rows = n.replace(hf, "qkv_proj"), (lo, hi)
            for hf, half in (("gate_proj", 0), ("up_proj", 1)):
                if f".{hf}." in n:
                    tgt = n.replace(hf, "gate_up_proj")
                    I = params[tgt].shape[0] // 2
                    rows = (half * I, half * I + I)
            if tgt not in params:
                continue
            dst = params[tgt] if rows is None else params[tgt][rows[0]:rows[1]]
            dst.copy_(w.to(dst.dtype).to(dst.device))
            loaded.add(name)
        return loaded


class DraftModelProposer:
    name = "draft_model"

    def __init__(self, method: str, num_speculative_tokens: int, spec_cfg: dict, runner):
        self.method, self.k, self.runner = method, num_speculative_tokens, runner
        self.needs_hidden_states = method in ("eagle", "eagle3", "mtp")
        dev = runner.device
        if method == "eagle3":
            self.model = Eagle3Head(runner.model, runner.mcfg, dev, runner.max_model_len,
                                    draft_vocab_size=spec_cfg.get("draft_vocab_size"))
            N = runner.mcfg.num_hidden_layers
            runner.model.aux_layers = (min(2, N - 1), N // 2, max(N - 3, 0))
            path = spec_cfg.get("model")
            if isinstance(path, str) and os.path.isdir(path):
                from ..models.transformer import iterate_safetensors
                self.model.load_weights(iterate_safetensors(path))
        elif method == "mtp":
            from ..parallel import state as _ps
            st = _ps.get_state()
            ep = st.ep if (runner.cfg.parallel.enable_expert_parallel and st.ep is not None
                           and st.ep.world_size > 1) else None
            self.model = MTPHead(runner.model, runner.mcfg, dev, runner.max_model_len, ep, runner.moe_runtime)
            if runner.mcfg.model_path:
                from ..models.transformer import iterate_safetensors
                self.model.load_weights(iterate_safetensors(runner.mcfg.model_path))
        elif self.needs_hidden_states:
            self.model = EagleHead(runner.model, runner.mcfg, dev, runner.max_model_len, seed_name=method)
        else:
            from ..models import build_model
            dm = spec_cfg.get("model")
            dcfg = dm if not isinstance(dm, str) else get_model_config(dm)
            if dcfg.vocab_size != runner.mcfg.vocab_size:
                raise ValueError("draft and target models must share a vocabulary")
            ecfg = copy.copy(runner.cfg)
            ecfg.model = dcfg
            self.model = build_model(ecfg, dev)
            if dcfg.model_path:
                from ..models.transformer import iterate_safetensors
                self.model.load_weights(iterate_safetensors(dcfg.model_path))
        self.kv_caches: Optional[list] = None
        self.computed: dict[str, int] = {}        # request id -> draft positions with valid KV
        self.stats = {"draft_forwards": 0}

    def _ensure_cache(self) -> None:
        if self.kv_caches is not None:
            return
        r = self.runner
        layout = r.cfg.cache.kv_layout if r.is_cuda else "NHD"
        self.kv_caches = []
        for layer in self.model.layers:
            a = layer.self_attn
            if hasattr(a, "dc"):                  # MLA draft layer: latent, rope key (and index keys)
                widths = [a.dc, a.dr] + ([a.idx_dim] if getattr(a, "index_topk", 0) else [])
                self.kv_caches.append(tuple(ops.alloc_kv_cache(r.num_blocks, r.block_size, 1, w, r.kv_dtype,
                                                               r.device, "NHD") for w in widths))
                continue
            self.kv_caches.append(tuple(ops.alloc_kv_cache(r.num_blocks, r.block_size, a.Hkv, a.D, r.kv_dtype,
                                                           r.device, layout) for _ in range(2)))

    # ------------------------------------------------------------------
    def _forward(self, items: list, shift: int, hidden_rows: Optional[torch.Tensor]):
        """items: (request, start, end) position ranges.  Returns (hidden of every processed
        position [T, H], index of each item's last row)."""
        r = self.runner
        so = SchedulerOutput(scheduled=[(_Standin(q.row, s, e, q.request_id), e - s) for q, s, e in items])
        meta, T, Tp, sel, _ = r._prepare_inputs(so)
        ids = r.input_ids[:T]
        if shift:
            rows = np.repeat([q.row for q, _, _ in items], [e - s for _, s, e in items])
            pos = np.concatenate([np.arange(s, e) for _, s, e in items]) + shift
            ids = torch.from_numpy(r.token_ids_cpu[rows, pos].astype(np.int64)).to(r.device)
        self.stats["draft_forwards"] += 1
        if self.needs_hidden_states:
            h = self.model.forward(ids, hidden_rows, meta, self.kv_caches)
        else:
            h = self.model.forward(ids, meta, self.kv_caches)
        return h, torch.tensor(sel, dtype=torch.int64, device=r.device)

    @torch.inference_mode()
    def propose_step(self, so, sampled: dict, hidden: Optional[torch.Tensor], scheduler) -> None:
        """Called once per engine step after the scheduler consumed the sampled tokens.
        ``hidden`` holds the target's final hidden state of every token of the step, in
        scheduling order (needed by the hidden-state-conditioned heads)."""
        self._ensure_cache()
        r = self.runner
        shift = 1 if self.needs_hidden_states else 0
        items, hid_idx, proposers = [], [], []
        off = 0
        for req, n in so.scheduled:
            off_req, off = off, off + n
            if req.is_finished or req.row < 0:
                self.computed.pop(req.request_id, None)
                continue
            # positions of this step that stay in the sequence: up to the new computed count
            end = req.num_computed_tokens                    # already advanced by the scheduler
            d = min(self.computed.get(req.request_id, 0), req.num_tokens - 1)
            if self.needs_hidden_states:
                # usable target hidden rows: positions [step_start, end); the head must not skip any
                step_start = self._step_start.get(req.request_id, 0)
                if d < step_start:
                    d = step_start                          # first seen mid-sequence (e.g. after preemption)
                last = min(end, req.num_tokens - 1)         # token_{i+1} must exist
                if last <= d:
                    continue
                items.append((req, d, last))
                hid_idx.append(np.arange(off_req + (d - step_start), off_req + (last - step_start)))
            else:
                last = req.num_tokens if req.request_id in sampled else min(end, req.num_tokens)
                if last <= d:
                    continue
                items.append((req, d, last))
            if req.request_id in sampled and req.status.name == "RUNNING":
                proposers.append(len(items) - 1)
        if not items:
            return
        hrows = None
        if self.needs_hidden_states:
            hrows = hidden[torch.from_numpy(np.concatenate(hid_idx)).to(hidden.device)]
        h, last_rows = self._forward(items, shift, hrows)
        for q, s, e in items:
            self.computed[q.request_id] = e
        if not proposers:
            return
        # first draft token of every request that sampled this step
        live = [items[i][0] for i in proposers]
        h_last = h[last_rows[torch.tensor(proposers, device=h.device)]]
        drafts = [[] for _ in live]
        budget = []
        for q in live:
            room = min(self.k, r.max_model_len - q.num_tokens - 1,
                       q.sampling_params.max_tokens - q.num_output_tokens - 1)
            if r.dynamic_spec is not None:
                room = min(room, r.dynamic_spec.budget(q.request_id))
            if room > 0 and not scheduler.try_extend(q, q.num_tokens + room):
                room = 0
            budget.append(max(room, 0))
        r._sync_rows(SchedulerOutput(scheduled=[], new_block_rows=live))
        for j in range(self.k):
            act = [i for i, b in enumerate(budget) if b > j]
            if not act:
                break
            idx = torch.tensor(act, device=h_last.device)
            if hasattr(self.model, "draft_tokens"):
                tok = self.model.draft_tokens(h_last[idx]).cpu().numpy()
            else:
                tok = self.model.compute_logits(h_last[idx]).argmax(-1).cpu().numpy()
            for i, t in zip(act, tok):
                q = live[i]
                drafts[i].append(int(t))
                r.token_ids_cpu[q.row, q.num_tokens + j] = int(t)
            if j == self.k - 1 or not any(b > j + 1 for b in budget):
                break
            nxt = [i for i in act if budget[i] > j + 1]
            pos0 = [live[i].num_tokens + j - shift for i in nxt]          # position of the next input
            step_items = [(live[i], p, p + 1) for i, p in zip(nxt, pos0)]
            hr = None
            if self.needs_hidden_states:
                keep = torch.tensor([act.index(i) for i in nxt], device=h_last.device)
                hr = h_last[idx][keep]
            hn, lr = self._forward(step_items, shift, hr)
            h_new = torch.zeros_like(h_last)
            h_new[torch.tensor(nxt, device=h_last.device)] = hn[lr]
            h_last = h_new
        for q, dts in zip(live, drafts):
            q.spec_token_ids = dts

    def note_step_start(self, so) -> None:
        """Records the first position each request processes in the coming step (the hidden
        rows of the step are indexed relative to it)."""
        self._step_start = {req.request_id: req.num_computed_tokens for req, _ in so.scheduled}

    _step_start: dict = {}
