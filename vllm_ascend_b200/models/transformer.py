"""Decoder-only transformer covering the model families the benchmarks name:
Llama / Qwen2 / Qwen3 (dense, GQA), Qwen3-MoE (routed experts) and
DeepSeek-V2/V3 (MLA attention + shared/routed experts, leading dense layers).

The reference takes model definitions from upstream vLLM and overrides layers
through its OOT op table (vllm_ascend/utils.py:703-732); here the definitions
live in the framework and call the op entry points directly.  Checkpoints use the
HF parameter names (``load_weights``), so the same safetensors files load.
"""
from __future__ import annotations

import re
from typing import Iterable, Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..ops import fused_moe, reference as ref
from ..parallel import state as pstate
from .layers import (ColumnParallelLinear, GQAAttention, Linear, ParallelLMHead, ParamFactory,
                     RMSNorm, RowParallelLinear, SwiGLUMLP, TPComm, VocabParallelEmbedding,
                     get_cos_sin_cache)


# ---------------------------------------------------------------- MoE block
class SparseMoeBlock:
    """Router + routed experts (+ shared experts).  Experts are sharded over the EP
    group when expert parallelism is on, else over TP along the intermediate dim."""

    def __init__(self, pf: ParamFactory, cfg: ModelConfig, layer_idx: int, comm: TPComm,
                 ep_group: Optional[pstate.GroupCoordinator], moe_runtime=None):
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.comm = comm
        prefix = f"model.layers.{layer_idx}.mlp"
        E, H, I = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        self.gate_weight = pf.normal(f"{prefix}.gate", (E, H), dtype=torch.float32)
        self.e_bias = pf.zeros((E,), dtype=torch.float32) if cfg.e_score_correction_bias else None
        self.ep = ep_group if (ep_group is not None and ep_group.world_size > 1) else None
        self.runtime = moe_runtime
        if self.ep is not None:
            ep, r = self.ep.world_size, self.ep.rank_in_group
            assert E % ep == 0
            self.E_local = E // ep
            self.expert_start = r * self.E_local
            g = pf.normal(f"{prefix}.experts.w1", (E, I, H), 0, r, ep)
            u = pf.normal(f"{prefix}.experts.w3", (E, I, H), 0, r, ep)
            self.w13 = torch.cat([g, u], dim=1).contiguous()
            self.w2 = pf.normal(f"{prefix}.experts.w2", (E, H, I), 0, r, ep)
            emap = torch.full((E,), -1, dtype=torch.int32)
            emap[self.expert_start:self.expert_start + self.E_local] = torch.arange(self.E_local, dtype=torch.int32)
            self.expert_map = emap.to(pf.device)
        else:
            tp, r = comm.size, comm.rank
            self.E_local = E
            self.expert_start = 0
            g = pf.normal(f"{prefix}.experts.w1", (E, I, H), 1, r, tp)
            u = pf.normal(f"{prefix}.experts.w3", (E, I, H), 1, r, tp)
            self.w13 = torch.cat([g, u], dim=1).contiguous()
            self.w2 = pf.normal(f"{prefix}.experts.w2", (E, H, I), 2, r, tp)
            self.expert_map = None
        self.quant = None
        self.shared = None
        self.shared_gate_weight = None
        shared_inter = cfg.shared_expert_intermediate_size or I * cfg.n_shared_experts
        self.shared_exec = None
        if shared_inter > 0:
            from ..ops.shared_experts import SharedExperts
            from ..platform_config import get_b200_config
            # replicated shared-expert weights: every rank holds the whole MLP and runs part of the rows
            self.shared_replicated = bool(get_b200_config().enable_shared_expert_dp) and comm.size > 1
            s_comm = TPComm(pstate.single_rank_group()) if self.shared_replicated else comm
            self.shared = SwiGLUMLP(pf, f"{prefix}.shared_experts", H, shared_inter, s_comm, reduce_results=False)
            if cfg.shared_expert_gate:           # Qwen2-MoE / Qwen3-Next: sigmoid(x . w) scales the shared expert
                self.shared_gate_weight = pf.normal(f"{prefix}.shared_expert_gate", (1, H))
            self.shared_exec = SharedExperts(self.shared, comm, self.shared_replicated, self.shared_gate_weight)
        # logical -> physical redirect for redundant experts (EPLB); identity by default
        self._gate_bf16: Optional[torch.Tensor] = None
        self.log2phy: Optional[torch.Tensor] = None          # [E, max_replicas] physical slot ids
        self.log2phy_count: Optional[torch.Tensor] = None    # [E] replicas per expert
        self.expert_load: Optional[torch.Tensor] = None      # per-physical-expert hit counter

    def _shared_out(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's shared-expert result for the rows of ``x``: a partial sum when the weights are
        TP shards, the complete result of the given rows when they are replicated."""
        self.shared_exec.gate_weight = self.shared_gate_weight      # may have been reloaded
        return self.shared_exec.local(x)

    def route(self, x: torch.Tensor):
        cfg = self.cfg
        if x.is_cuda and x.dtype == torch.bfloat16 and cfg.scoring_func == "softmax" and not cfg.use_mla:
            # softmax routers of bf16 checkpoints run their gate in the model dtype (as the
            # original implementation does): one tensor-core GEMM instead of an fp32 SIMT one
            if self._gate_bf16 is None:
                self._gate_bf16 = self.gate_weight.to(torch.bfloat16)
            logits = ops.linear(x, self._gate_bf16).float()
        else:
            logits = torch.nn.functional.linear(x.float(), self.gate_weight)
        w, ids = fused_moe.gating_topk(logits, cfg.num_experts_per_tok, cfg.scoring_func,
                                       cfg.norm_topk_prob, cfg.n_group, cfg.topk_group,
                                       self.e_bias, cfg.routed_scaling_factor)
        if self.expert_load is not None:          # per logical expert, before any redirect
            self.expert_load.scatter_add_(0, ids.flatten().long(),
                                          torch.ones(ids.numel(), dtype=self.expert_load.dtype,
                                                     device=ids.device))
        if self.log2phy is not None:
            # logical -> physical slot; tokens spread over an expert's replicas round-robin
            lid = ids.long()
            n = self.log2phy_count[lid]
            pick = torch.arange(ids.shape[0], device=ids.device).unsqueeze(1) % n
            ids = self.log2phy[lid, pick].to(torch.int32)
        return w, ids

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        w, ids = self.route(x)
        overlap = None
        if self.shared is not None and self.ep is not None and x.is_cuda and self._overlap_shared() \
                and not torch.cuda.is_current_stream_capturing():
            # shared experts run on a side stream while the routed tokens travel: the stream
            # forks after routing and joins before the sum (the reference gates the same overlap
            # on dispatch / combine events, ops/fused_moe/shared_experts.py:49-349)
            from ..utils import side_stream
            side = side_stream("shared_expert", x.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                overlap = self._shared_out(x)
                x.record_stream(side)
        moe_lora = getattr(self, "lora", None)
        if self.runtime is not None and self.ep is not None:
            y = self.runtime.forward(self, x, w, ids)          # EP dispatch/combine paths
        elif moe_lora is not None and moe_lora.punica.any_active and self.quant is None:
            from ..lora.moe import fused_experts_lora
            y = fused_experts_lora(x, self.w13, self.w2, w, ids, self.expert_map, moe_lora)
        else:
            y = fused_moe.fused_experts(x, self.w13, self.w2, w, ids, self.expert_map, self.quant)
        replicated = self.shared is not None and self.shared_replicated
        if self.ep is None:
            # TP-sharded experts (and shared experts) hold partial sums: one reduction
            if self.shared is not None and not replicated:
                y = y + self._shared_out(x)
            if self.comm.size > 1:
                y = self.comm.all_reduce(y)
            if replicated:
                # whole shared expert on every rank: each runs its part of the rows, rows gathered
                self.shared_exec.gate_weight = self.shared_gate_weight
                y = y + self.shared_exec.forward(x)
            return y
        if self.shared is not None:
            if overlap is not None:
                torch.cuda.current_stream().wait_stream(side)
                s = overlap
                if self.comm.size > 1 and not replicated:
                    s = self.comm.all_reduce(s)
            else:
                self.shared_exec.gate_weight = self.shared_gate_weight
                s = self.shared_exec.forward(x)
            y = y + s
        return y

    @staticmethod
    def _overlap_shared() -> bool:
        from ..platform_config import get_b200_config
        return get_b200_config().multistream_overlap_shared_expert


# ---------------------------------------------------------------- MLA attention
_HEAD_OFFSETS: dict = {}       # (device, heads, tokens) -> int32 group offsets of the per-head grouped GEMM


class MLAAttention:
    """Multi-head latent attention with absorbed weights.

    Cache contract (vllm_ascend/attention/mla_v1.py:1296-1326): per token one
    normalised latent vector (kv_lora_rank) and one RoPE'd key slice
    (qk_rope_head_dim), in two paged tensors.  Scores are
    q_nope·W_UK·latent + q_pe·k_pe; the value path is latent·W_UV — i.e. MQA over a
    576-wide key with the up-projections folded into q and the output
    (``W_UK_T`` / ``W_UV`` of mla_v1.py:907-971).
    """

    def __init__(self, pf: ParamFactory, cfg: ModelConfig, layer_idx: int, comm: TPComm,
                 max_pos: int):
        self.cfg = cfg
        tp = comm.size
        self.H = cfg.num_attention_heads // tp
        self.dn, self.dr, self.dv, self.dc = (cfg.qk_nope_head_dim, cfg.qk_rope_head_dim,
                                              cfg.v_head_dim, cfg.kv_lora_rank)
        hid = cfg.hidden_size
        p = f"model.layers.{layer_idx}.self_attn"
        rep = TPComm(pstate.GroupCoordinator("single", [0], 0))   # replicated (not sharded)
        qd = cfg.num_attention_heads * (self.dn + self.dr)
        if cfg.q_lora_rank:
            self.q_a_proj = ColumnParallelLinear(pf, f"{p}.q_a_proj", hid, [cfg.q_lora_rank], rep)
            self.q_a_norm = RMSNorm(pf, cfg.q_lora_rank, cfg.rms_norm_eps)
            self.q_b_proj = ColumnParallelLinear(pf, f"{p}.q_b_proj", cfg.q_lora_rank, [qd], comm)
            self.q_proj = None
        else:
            self.q_proj = ColumnParallelLinear(pf, f"{p}.q_proj", hid, [qd], comm)
        self.kv_a_proj = ColumnParallelLinear(pf, f"{p}.kv_a_proj_with_mqa", hid,
                                              [self.dc + self.dr], rep)
        self.kv_a_norm = RMSNorm(pf, self.dc, cfg.rms_norm_eps)
        # kv_b_proj [H*(dn+dv), dc] kept for checkpoint parity, used through the absorbed views
        self.kv_b_proj = ColumnParallelLinear(pf, f"{p}.kv_b_proj", self.dc,
                                              [cfg.num_attention_heads * (self.dn + self.dv)], comm)
        self.o_proj = RowParallelLinear(pf, f"{p}.o_proj", cfg.num_attention_heads * self.dv, hid,
                                        comm)
        self.scale = (self.dn + self.dr) ** -0.5
        sc = cfg.rope_scaling
        if sc and sc.get("mscale_all_dim"):
            import math
            m = 0.1 * sc["mscale_all_dim"] * math.log(sc.get("factor", 1.0)) + 1.0
            self.scale *= m * m
        self.cos_sin = get_cos_sin_cache(self.dr, max_pos, cfg.rope_theta,
                                         dict(sc, rope_type="deepseek_yarn") if sc else None,
                                         pf.device)
        # lightning indexer (sparse attention): a few small heads score every cached key per query and
        # attention runs over the index_topk best; weights are replicated over TP (every rank needs
        # the full selection).  Names follow the published checkpoints (self_attn.indexer.*).
        self.index_topk = cfg.index_topk if cfg.use_sparse else 0
        self.offload = None            # attention.sparse_offload.SparseOffloadLayer when the KV is host-resident
        if self.index_topk:
            if not cfg.q_lora_rank:
                raise ValueError("the indexer reads the compressed query (q_lora_rank must be set)")
            Hn, Dh = cfg.index_n_heads, cfg.index_head_dim
            self.idx_heads, self.idx_dim = Hn, Dh
            self.idx_wq_b = ColumnParallelLinear(pf, f"{p}.indexer.wq_b", cfg.q_lora_rank, [Hn * Dh], rep)
            self.idx_wk = ColumnParallelLinear(pf, f"{p}.indexer.wk", hid, [Dh], rep)
            self.idx_k_norm_w = pf.ones((Dh,))
            self.idx_k_norm_b = pf.zeros((Dh,))
            self.idx_weights_proj = ColumnParallelLinear(pf, f"{p}.indexer.weights_proj", hid, [Hn], rep)
            self.idx_scale = Hn ** -0.5 * Dh ** -0.5
        self.process_weights_after_loading()

    def process_weights_after_loading(self) -> None:
        w = self.kv_b_proj.weight.view(self.H, self.dn + self.dv, self.dc)
        self.W_UK = w[:, :self.dn, :].contiguous()                        # [H, dn, dc]
        self.W_UV = w[:, self.dn:, :].transpose(1, 2).contiguous()        # [H, dc, dv]
        # the same matrices as [out, in] per head: operands of the grouped (one group per head) GEMM
        self.W_UK_nk = self.W_UK.transpose(1, 2).contiguous()             # [H, dc, dn]
        self.W_UV_nk = w[:, self.dn:, :].contiguous()                     # [H, dv, dc]

    def __call__(self, x: torch.Tensor, meta, kv_cache) -> torch.Tensor:
        T = x.shape[0]
        if self.q_proj is None:
            qr = self.q_a_norm(self.q_a_proj(x))[0]
            q = self.q_b_proj(qr)
        else:
            q = self.q_proj(x)
            qr = None
        q = q.view(T, self.H, self.dn + self.dr)
        kv = self.kv_a_proj(x)
        lat_cache, pe_cache = kv_cache[0], kv_cache[1]
        from ..attention import mla as mla_ops
        if self.offload is None and not self.kv_a_norm.gemma:
            # one pass: latent RMSNorm + rope of the shared key -> their cache slots, rope of every
            # query head in place
            ops.mla_preprocess(q, kv, self.kv_a_norm.weight, self.kv_a_norm.eps, meta.positions, self.cos_sin,
                               meta.slot_mapping, lat_cache, pe_cache, self.dn, self.dr)
            q_pe = q[..., self.dn:]
        else:
            latent = self.kv_a_norm(kv[:, :self.dc].contiguous())[0]
            k_pe = kv[:, self.dc:].reshape(T, 1, self.dr)
            q_pe = ref.apply_rope_interleaved(q[..., self.dn:], meta.positions, self.cos_sin, self.dr)
            k_pe = ref.apply_rope_interleaved(k_pe, meta.positions, self.cos_sin, self.dr)
            if self.offload is None:
                mla_ops.write_latent_cache(latent, k_pe.view(T, self.dr), lat_cache, pe_cache, meta.slot_mapping)
            else:   # host-resident KV: the rows of this step's tokens go to the sequence's host store
                self.offload.append(meta.extra["tok_rows"], meta.extra["positions_cpu"], latent,
                                    k_pe.view(T, self.dr))
        # absorb W_UK into q: [T,H,dn] x [H,dn,dc] -> [T,H,dc]
        q_lat = self._per_head_matmul(q[..., :self.dn], self.W_UK, self.W_UK_nk)
        dcp = pstate.get_dcp_group()
        if self.index_topk:
            o_lat = self._sparse_attention(x, qr, q_lat.contiguous(), q_pe.contiguous(), lat_cache, pe_cache,
                                           kv_cache[2], meta)
        elif dcp.world_size > 1:
            from ..attention.dcp import mla_attention_dcp
            o_lat = mla_attention_dcp(q_lat, q_pe, lat_cache, pe_cache, meta, self.scale, dcp,
                                      getattr(meta, "dcp_interleave", 1))
        else:
            o_lat = mla_ops.mla_paged_attention(q_lat, q_pe, lat_cache, pe_cache, meta, self.scale)
        o = self._per_head_matmul(o_lat, self.W_UV, self.W_UV_nk)
        return self.o_proj(o.reshape(T, self.H * self.dv))

    def _per_head_matmul(self, x: torch.Tensor, w_kn: torch.Tensor, w_nk: torch.Tensor) -> torch.Tensor:
        """x [T, H, K] times one [K, N] matrix per head -> [T, H, N] (the two weight absorptions of MLA:
        W_UK into the query, W_UV out of the latent result).  On the GPU the heads are the groups of the
        grouped tcgen05 GEMM: rows are laid out head-major, every head's T rows meet that head's matrix
        (the reference has a dedicated op for this product, csrc/batch_matmul_transpose/)."""
        T, H, K = x.shape
        N = w_nk.shape[1]
        from ..ops import moe_native
        if not (x.is_cuda and x.dtype == torch.bfloat16 and w_nk.dtype == torch.bfloat16 and moe_native.available()
                and K % 8 == 0 and N % 8 == 0 and H <= 256 and T > 0):
            return torch.einsum("thk,hkn->thn", x, w_kn.to(x.dtype))
        # group offsets per token count, kept for the life of the process: a captured graph keeps
        # reading the tensor it was recorded with
        key = (x.device, H, T)
        off = _HEAD_OFFSETS.get(key)
        if off is None:
            off = torch.arange(0, H + 1, dtype=torch.int32, device=x.device) * T
            _HEAD_OFFSETS[key] = off
        rows = x.transpose(0, 1).contiguous().view(H * T, K)             # head-major rows
        out = moe_native.grouped_gemm(rows, w_nk, off, False)            # [H * T, N]
        return out.view(H, T, N).transpose(0, 1)

    def _sparse_attention(self, x, qr, q_lat, q_pe, lat_cache, pe_cache, idx_cache, meta):
        """Indexer scores -> top-k key positions per query -> MLA attention over those keys.
        The rotary part of the indexer's q / k is the leading qk_rope_head_dim slice, rotated in the
        half-split (neox) pairing; the orthogonal Hadamard rotation the published model applies to
        both q and k before low-precision scoring leaves the dot products unchanged and is omitted."""
        from ..attention import sfa
        T = x.shape[0]
        Hn, Dh, dr = self.idx_heads, self.idx_dim, self.dr
        q_idx = self.idx_wq_b(qr).view(T, Hn, Dh)
        k_idx = torch.nn.functional.layer_norm(self.idx_wk(x).float(), (Dh,), self.idx_k_norm_w.float(),
                                               self.idx_k_norm_b.float(), 1e-6).to(x.dtype).view(T, 1, Dh)
        q_idx = ref.apply_rope_neox(q_idx, meta.positions, self.cos_sin, dr)
        k_idx = ref.apply_rope_neox(k_idx, meta.positions, self.cos_sin, dr)
        w = self.idx_weights_proj(x).float() * self.idx_scale                       # [T, Hn]
        # index keys live in their own paged cache, addressed like the latent cache
        valid = (meta.slot_mapping >= 0).unsqueeze(-1)
        slot = meta.slot_mapping.clamp(min=0)
        flat = idx_cache.view(-1, Dh)
        flat.index_copy_(0, slot, torch.where(valid, k_idx.view(T, Dh).to(flat.dtype), flat[slot]))
        indices = sfa.lightning_indexer(q_idx.contiguous(), w, idx_cache, meta, self.index_topk)
        if self.offload is not None:
            return self.offload.attend(q_lat, q_pe, meta.extra["tok_rows"], indices, self.scale)
        return sfa.sparse_mla_attention(q_lat, q_pe, lat_cache, pe_cache, meta, indices, self.scale)


# ---------------------------------------------------------------- decoder layer / model
class DecoderLayer:
    def __init__(self, pf: ParamFactory, cfg: ModelConfig, idx: int, comm: TPComm, max_pos: int,
                 ep_group=None, moe_runtime=None):
        p = f"model.layers.{idx}"
        self.idx = idx
        self.input_layernorm = RMSNorm(pf, cfg.hidden_size, cfg.rms_norm_eps, gemma=cfg.gemma_norm)
        self.post_attention_layernorm = RMSNorm(pf, cfg.hidden_size, cfg.rms_norm_eps, gemma=cfg.gemma_norm)
        # sandwich norms (GLM-4): each sub-layer's output is normalised before it joins the residual stream
        self.post_self_attn_layernorm = self.post_mlp_layernorm = None
        if cfg.sandwich_norm:
            self.post_self_attn_layernorm = RMSNorm(pf, cfg.hidden_size, cfg.rms_norm_eps, gemma=cfg.gemma_norm)
            self.post_mlp_layernorm = RMSNorm(pf, cfg.hidden_size, cfg.rms_norm_eps, gemma=cfg.gemma_norm)
        self.residual_multiplier = float(cfg.residual_multiplier)
        self.pre_norm = bool(cfg.pre_norm)
        self.hc_attn = self.hc_ffn = None
        if cfg.hc_mult > 1:
            from ..ops.hyper_connection import HyperConnection
            self.hc_attn = HyperConnection(pf, f"{p}.hc_attn", cfg.hidden_size, cfg.hc_mult, cfg.hc_sinkhorn_iters,
                                           cfg.rms_norm_eps)
            self.hc_ffn = HyperConnection(pf, f"{p}.hc_ffn", cfg.hidden_size, cfg.hc_mult, cfg.hc_sinkhorn_iters,
                                          cfg.rms_norm_eps)
        self.deepnorm = None
        if cfg.deepnorm_factors:
            f = cfg.deepnorm_factors
            self.deepnorm = (tuple(f["linear" if cfg.is_linear_layer(idx) else "full"]), tuple(f["mlp"]))
        if cfg.is_linear_layer(idx) and cfg.linear_attn_kind == "lightning":
            from .lightning import LightningAttention
            self.self_attn = LightningAttention(pf, cfg, idx, comm)
        elif cfg.is_linear_layer(idx) and cfg.linear_attn_kind == "mamba2":
            from .mamba2 import Mamba2Mixer
            self.self_attn = Mamba2Mixer(pf, cfg, idx, comm)
        elif cfg.is_linear_layer(idx):
            from .gdn import GatedDeltaNet
            self.self_attn = GatedDeltaNet(pf, cfg, idx, comm)
        else:
            self.self_attn = (MLAAttention if cfg.use_mla else GQAAttention)(pf, cfg, idx, comm, max_pos)
        from ..parallel import finegrained as fgm
        fg = fgm.get_fg()
        if cfg.is_moe_layer(idx):
            self.mlp = SparseMoeBlock(pf, cfg, idx, comm, ep_group, moe_runtime)
        elif fg is not None and fg.mlp_tp is not None:
            inner = SwiGLUMLP(pf, f"{p}.mlp", cfg.hidden_size, cfg.intermediate_size, TPComm(fg.mlp_tp),
                              reduce_results=False)
            self.mlp = fgm.FGMLP(inner, fg.mlp_tp)
        else:
            if cfg.mlp_gated:
                self.mlp = SwiGLUMLP(pf, f"{p}.mlp", cfg.hidden_size, cfg.intermediate_size, comm, act=cfg.hidden_act)
            else:
                from .layers import PlainMLP
                self.mlp = PlainMLP(pf, f"{p}.mlp", cfg.hidden_size, cfg.intermediate_size, comm, act=cfg.hidden_act)
        if fg is not None and fg.otp is not None and isinstance(self.self_attn, GQAAttention):
            a = self.self_attn
            inner = RowParallelLinear(pf, f"{p}.self_attn.o_proj", cfg.num_attention_heads * a.D, cfg.hidden_size,
                                      TPComm(fg.otp), reduce_results=False)
            a.o_proj = fgm.FGOProj(inner, fg.otp)

    def __call__(self, h, residual, meta, kv_cache):
        if not self.pre_norm:
            # sub-layers read the stream as it is; their outputs are normalised before they join it
            s = h if residual is None else h + residual
            a, _ = self.post_self_attn_layernorm(self.self_attn(s, meta, kv_cache))
            s = s + a
            f, _ = self.post_mlp_layernorm(self.mlp(s))
            return s + f, None
        if self.hc_attn is not None:
            # h: the widened residual streams [T, m, H]; each sub-layer reads a mixture and writes back
            from ..ops.hyper_connection import hc_post
            streams = h
            x, post, comb = self.hc_attn.pre(streams)
            x, _ = self.input_layernorm(x)
            streams = hc_post(self.self_attn(x, meta, kv_cache), streams, post, comb)
            x, post, comb = self.hc_ffn.pre(streams)
            x, _ = self.post_attention_layernorm(x)
            return hc_post(self.mlp(x), streams, post, comb), None
        if self.deepnorm is not None:
            # the stream continues from the normalised value: s = norm(s); s = alpha s + beta f(s)
            (aa, ab), (ma, mb) = self.deepnorm
            x, _ = self.input_layernorm(h if residual is None else h + residual)
            s = x * aa + self.self_attn(x, meta, kv_cache) * ab
            y, _ = self.post_attention_layernorm(s)
            return y * ma + self.mlp(y) * mb, None
        # a norm whose only consumer is an fp8 GEMM emits fp8 + scales directly
        qa = self._attn_in_fp8
        if residual is None:
            residual = h
            x, _ = self.input_layernorm(h, quant_out=qa)
        else:
            x, residual = self.input_layernorm(h, residual, quant_out=qa)
        h = self.self_attn(x, meta, kv_cache)
        if self.residual_multiplier != 1.0:
            h = h * self.residual_multiplier
        if self.post_self_attn_layernorm is not None:
            h, _ = self.post_self_attn_layernorm(h)
        x, residual = self.post_attention_layernorm(h, residual, quant_out=self._mlp_in_fp8)
        h = self.mlp(x)
        if self.residual_multiplier != 1.0:
            h = h * self.residual_multiplier
        if self.post_mlp_layernorm is not None:
            h, _ = self.post_mlp_layernorm(h)
        return h, residual

    @property
    def _attn_in_fp8(self) -> bool:
        from .layers import wants_quant_act
        a = self.self_attn
        return hasattr(a, "qkv_proj") and wants_quant_act(a.qkv_proj)

    @property
    def _mlp_in_fp8(self) -> bool:
        from .layers import SwiGLUMLP, wants_quant_act
        m = self.mlp
        return isinstance(m, SwiGLUMLP) and wants_quant_act(m.gate_up_proj)


class CausalLM:
    """Model object the runner drives: ``forward`` -> hidden states, ``compute_logits``."""

    def __init__(self, cfg: ModelConfig, device, max_model_len: int = 4096,
                 tp_group: Optional[pstate.GroupCoordinator] = None,
                 ep_group: Optional[pstate.GroupCoordinator] = None, moe_runtime=None,
                 layer_range: Optional[tuple[int, int]] = None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = cfg.torch_dtype
        pf = ParamFactory(cfg, self.device, self.dtype)
        self.comm = TPComm(tp_group or pstate.get_tp_group())
        self.sp_ctx = None             # set by parallel.fused_linear.attach()
        self.sp_prefill = self.sp_decode = True     # which step classes use it (auto mode calibrates)
        self.sp_decode_max_tokens = 2048            # steps up to this many tokens count as decode-like
        self.layer_hook = None         # callable(local layer index), run after each layer
        self.aux_layers = None         # layer indices whose residual-stream output EAGLE-3 heads read
        self.aux_hidden = None         # [T, len(aux_layers) * H] of the latest eager forward
        self.full_embedding = None
        max_pos = max(max_model_len, 16)
        lo, hi = layer_range or (0, cfg.num_hidden_layers)
        self.layer_range = (lo, hi)
        self.is_first = lo == 0
        self.is_last = hi == cfg.num_hidden_layers
        from ..parallel import finegrained as fgm
        fg = fgm.get_fg()
        if fg is not None and cfg.tie_word_embeddings and (fg.lmtp is not None or fg.embed_tp is not None) \
                and getattr(fg.lmtp, "ranks", None) != getattr(fg.embed_tp, "ranks", None):
            raise ValueError("tied embeddings need the same group for lmhead and embedding tensor parallelism")
        self.embed_tokens = VocabParallelEmbedding(pf, "model.embed_tokens", cfg.vocab_size, cfg.hidden_size,
                                                   TPComm(fg.embed_tp) if fg and fg.embed_tp else self.comm)
        self.layers = [DecoderLayer(pf, cfg, i, self.comm, max_pos, ep_group, moe_runtime)
                       for i in range(lo, hi)]
        self.norm = RMSNorm(pf, cfg.hidden_size, cfg.rms_norm_eps, gemma=cfg.gemma_norm)
        self.hc_head = None
        if cfg.hc_mult > 1:
            if not (self.is_first and self.is_last):
                raise ValueError("hyper-connections: the widened residual streams are not carried between pipeline stages")
            m = cfg.hc_mult
            self.hc_head = (pf.normal("model.hc_head_fn", (m, m * cfg.hidden_size), std=1.0 / (m * cfg.hidden_size) ** 0.5,
                                      dtype=torch.float32),
                            pf.ones((1,), dtype=torch.float32), pf.zeros((m,), dtype=torch.float32))
        if cfg.tie_word_embeddings:
            self.lm_head = ParallelLMHead(self.embed_tokens)
        else:
            head = VocabParallelEmbedding(pf, "lm_head", cfg.vocab_size, cfg.hidden_size,
                                          TPComm(fg.lmtp) if fg and fg.lmtp else self.comm)
            self.lm_head = ParallelLMHead(head)
        if fg is not None and fg.lmtp is not None:
            self.lm_head = fgm.FGLMHead(self.lm_head, fg.lmtp)
        if fg is not None and fg.embed_tp is not None:
            self.embed_tokens = fgm.FGEmbedding(self.embed_tokens, fg.embed_tp)
        if cfg.quantization:
            from ..quantization import apply_quantization
            apply_quantization(self, cfg)

    # -- forward ---------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, meta, kv_caches: list,
                intermediate: Optional[tuple] = None, inputs_embeds: Optional[torch.Tensor] = None):
        if self.sp_ctx is not None and input_ids.is_cuda and inputs_embeds is None \
                and (self.sp_prefill if input_ids.shape[0] > self.sp_decode_max_tokens else self.sp_decode):
            from ..parallel.fused_linear import forward_sp
            return forward_sp(self, self.sp_ctx, input_ids, meta, kv_caches)
        if getattr(self, "norm_folded", False) and input_ids.is_cuda and inputs_embeds is None \
                and intermediate is None and not self.aux_layers and getattr(meta, "deepstack", None) is None:
            from . import folded
            if input_ids.shape[0] >= folded.min_rows() and \
                    not any(getattr(L, "offloaded_call", None) is not None for L in self.layers):
                return folded.forward_folded(self, input_ids, meta, kv_caches)
        if self.is_first:
            # multimodal steps pass embeddings with the encoder outputs already merged in
            h = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
            if self.cfg.embed_scale != 1.0 and inputs_embeds is None:
                h = h * torch.tensor(self.cfg.embed_scale, dtype=h.dtype)      # rounded to the model dtype first
            if self.hc_head is not None:
                h = h.unsqueeze(1).repeat(1, self.cfg.hc_mult, 1)              # [T, H] -> [T, m, H]
            residual = None
        else:
            h, residual = intermediate
        aux = [] if self.aux_layers else None
        deepstack = getattr(meta, "deepstack", None)
        from .. import envs
        per_layer_nvtx = envs.VLLM_B200_NVTX >= 2 and h.is_cuda
        for layer, cache in zip(self.layers, kv_caches):
            call = getattr(layer, "offloaded_call", None)      # set by the weight offloader
            if per_layer_nvtx:
                torch.cuda.nvtx.range_push(f"layer{layer.idx}")
            h, residual = call(h, residual, meta, cache) if call is not None else layer(h, residual, meta, cache)
            if per_layer_nvtx:
                torch.cuda.nvtx.range_pop()
            if deepstack is not None and layer.idx < deepstack[1].shape[0]:
                # visual features join the residual stream (h + residual) at the image-token rows
                h.index_add_(0, deepstack[0], deepstack[1][layer.idx].to(h.dtype))
            if aux is not None:
                for _ in range(self.aux_layers.count(layer.idx)):
                    aux.append(h if residual is None else h + residual)
            if self.layer_hook is not None:
                self.layer_hook(layer.idx - self.layer_range[0])   # e.g. layer-wise KV push
        if aux:
            self.aux_hidden = torch.cat(aux, dim=-1)
        if not self.is_last:
            return h, residual
        if self.hc_head is not None:
            from ..ops.hyper_connection import hc_head
            h = hc_head(h, self.hc_head[0], self.hc_head[1], self.hc_head[2], self.cfg.rms_norm_eps)
        h, _ = self.norm(h, residual)
        return h

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        logits = self.lm_head(hidden)
        if self.cfg.logits_scaling != 1.0:
            logits = logits / self.cfg.logits_scaling
        return logits

    def embed_input_ids(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.embed_tokens(input_ids)

    __call__ = forward

    # -- parameters --------------------------------------------------------
    def named_parameters(self):
        yield "model.embed_tokens.weight", self.embed_tokens.weight
        for L in self.layers:
            p = f"model.layers.{L.idx}"
            yield f"{p}.input_layernorm.weight", L.input_layernorm.weight
            yield f"{p}.post_attention_layernorm.weight", L.post_attention_layernorm.weight
            if L.hc_attn is not None:
                yield from L.hc_attn.named_tensors(f"{p}.hc_attn")
                yield from L.hc_ffn.named_tensors(f"{p}.hc_ffn")
            if L.post_self_attn_layernorm is not None:
                yield f"{p}.post_self_attn_layernorm.weight", L.post_self_attn_layernorm.weight
                yield f"{p}.post_mlp_layernorm.weight", L.post_mlp_layernorm.weight
            a = L.self_attn
            if getattr(a, "kind", "") == "lightning":
                for n, t in a.named_tensors():
                    yield f"{p}.self_attn.{n}", t
            elif getattr(a, "kind", "") == "mamba2":
                for n, t in a.named_tensors():
                    yield f"{p}.mamba.{n}", t
            elif getattr(a, "is_linear_attention", False):
                for attr in ("in_proj_qkvz", "in_proj_ba", "out_proj"):
                    for n, t in getattr(a, attr).named_tensors():
                        yield f"{p}.linear_attn.{attr}.{n}", t
                for n, t in a.named_tensors():
                    yield f"{p}.linear_attn.{n}", t
            for attr in ("qkv_proj", "o_proj", "q_a_proj", "q_b_proj", "q_proj", "kv_a_proj",
                         "kv_b_proj"):
                if getattr(a, "kind", "") in ("lightning", "mamba2"):       # yielded above under their own names
                    break
                lin = getattr(a, attr, None)
                lin = getattr(lin, "inner", lin)            # fine-grained TP wrapper
                if isinstance(lin, Linear):
                    for n, t in lin.named_tensors():
                        yield f"{p}.self_attn.{attr}.{n}", t
            for attr in ("q_norm", "k_norm"):
                t = getattr(a, attr, None)
                if isinstance(t, torch.Tensor):
                    yield f"{p}.self_attn.{attr}.weight", t
            for attr in ("q_a_norm", "kv_a_norm"):
                n = getattr(a, attr, None)
                if n is not None:
                    yield f"{p}.self_attn.{attr}.weight", n.weight
            if getattr(a, "index_topk", 0):
                yield f"{p}.self_attn.indexer.wq_b.weight", a.idx_wq_b.weight
                yield f"{p}.self_attn.indexer.wk.weight", a.idx_wk.weight
                yield f"{p}.self_attn.indexer.k_norm.weight", a.idx_k_norm_w
                yield f"{p}.self_attn.indexer.k_norm.bias", a.idx_k_norm_b
                yield f"{p}.self_attn.indexer.weights_proj.weight", a.idx_weights_proj.weight
            m = L.mlp
            if isinstance(m, SparseMoeBlock):
                yield f"{p}.mlp.gate.weight", m.gate_weight
                if m.e_bias is not None:
                    yield f"{p}.mlp.gate.e_score_correction_bias", m.e_bias
                yield f"{p}.mlp.experts.w13", m.w13
                yield f"{p}.mlp.experts.w2", m.w2
                if m.shared_gate_weight is not None:
                    yield f"{p}.mlp.shared_expert_gate.weight", m.shared_gate_weight
                if m.shared is not None:
                    for n, t in m.shared.gate_up_proj.named_tensors():
                        yield f"{p}.mlp.shared_experts.gate_up_proj.{n}", t
                    for n, t in m.shared.down_proj.named_tensors():
                        yield f"{p}.mlp.shared_experts.down_proj.{n}", t
            elif hasattr(m, "up_proj"):            # ungated MLP
                for n, t in m.up_proj.named_tensors():
                    yield f"{p}.mlp.up_proj.{n}", t
                for n, t in m.down_proj.named_tensors():
                    yield f"{p}.mlp.down_proj.{n}", t
            else:
                for n, t in m.gate_up_proj.named_tensors():
                    yield f"{p}.mlp.gate_up_proj.{n}", t
                for n, t in m.down_proj.named_tensors():
                    yield f"{p}.mlp.down_proj.{n}", t
        yield "model.norm.weight", self.norm.weight
        if getattr(self, "hc_head", None) is not None:
            yield "model.hc_head_fn", self.hc_head[0]
            yield "model.hc_head_scale", self.hc_head[1]
            yield "model.hc_head_base", self.hc_head[2]
        if not self.cfg.tie_word_embeddings:
            yield "lm_head.weight", self.lm_head.weight

    def num_parameters(self) -> int:
        return sum(t.numel() for _, t in self.named_parameters())

    # -- checkpoint loading ------------------------------------------------
    _STACKED = {"q_proj": ("qkv_proj", 0), "k_proj": ("qkv_proj", 1), "v_proj": ("qkv_proj", 2),
                "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1)}

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        """Loads HF-named tensors, slicing each to this rank's TP/EP shard."""
        loaded: set[str] = set()
        params = dict(self.named_parameters())
        layers = {L.idx: L for L in self.layers}
        tp, r = self.comm.size, self.comm.rank
        arch_internlm2 = self.cfg.architecture.startswith("InternLM2")
        cfg = self.cfg
        for name, w in weights:
            if name.endswith("rotary_emb.inv_freq"):
                continue
            orig_name = name
            if not cfg.pre_norm:            # OLMo-2 names its two output norms like other models' pre-norms
                name = name.replace(".post_attention_layernorm.", ".post_self_attn_layernorm.") \
                           .replace(".post_feedforward_layernorm.", ".post_mlp_layernorm.")
            if ".shared_mlp." in name and not self.cfg.is_moe:
                # Granite 4 dense hybrids: the gated MLP under its own names, gate and up rows in one tensor
                name = name.replace(".shared_mlp.input_linear.", ".mlp.gate_up_proj.") \
                           .replace(".shared_mlp.output_linear.", ".mlp.down_proj.")
            if cfg.rope_interleaved and re.search(r"self_attn\.(q|k)_proj\.(weight|bias)$", name):
                # checkpoints whose rotary pairs are (2i, 2i + 1): move every head's rotated rows into
                # the half-split order the kernels rotate; q.k is unchanged by a common permutation
                D = cfg.head_dim
                rot = int(D * cfg.partial_rotary_factor) // 2 * 2
                idx = torch.cat([torch.arange(0, rot, 2), torch.arange(1, rot, 2), torch.arange(rot, D)])
                w = w.view(-1, D, *w.shape[1:])[:, idx].reshape(w.shape)
            if name.endswith(".mlp.gate_up_proj.weight") and ".experts." not in name and cfg.split_fused_gate_up:
                # [gate rows; up rows] stored as one tensor: place the halves like separate projections
                tgt = name
                if tgt in params:
                    half = w.shape[0] // 2
                    tp_t, r_t = self._shard_of(tgt, tp, r)
                    self._copy_shard(tgt, params[tgt], w[:half], 0, tp_t, r_t)
                    self._copy_shard(tgt, params[tgt], w[half:], 1, tp_t, r_t)
                    loaded.add(orig_name)
                continue
            if arch_internlm2:
                name = _internlm2_name(name)
                if name.endswith("attention.wqkv.weight"):
                    # rows grouped per KV head: [q heads of the group..., k, v] x head_dim
                    D, Hkv = self.cfg.head_dim, self.cfg.num_key_value_heads
                    G = self.cfg.num_attention_heads // Hkv
                    w5 = w.view(Hkv, G + 2, D, -1)
                    base = name.replace("attention.wqkv", "self_attn.qkv_proj")
                    if base in params:
                        for sid, part in ((0, w5[:, :G].reshape(Hkv * G * D, -1)), (1, w5[:, G].reshape(Hkv * D, -1)),
                                          (2, w5[:, G + 1].reshape(Hkv * D, -1))):
                            self._copy_shard(base, params[base], part, sid, tp, r)
                        loaded.add(orig_name)
                    continue
            if name.endswith(".mlp.gate.moe_statics.e_score_correction_bias"):      # Ernie 4.5 MoE: [1, E]
                name = name.replace(".moe_statics.", ".")
                w = w.reshape(-1)
            if name.endswith(".mlp.e_score_correction_bias"):       # MiniMax-M2 keeps the bias beside the gate
                name = name.replace(".mlp.e_score_correction_bias", ".mlp.gate.e_score_correction_bias")
            if self.cfg.qk_norm_full and name.endswith("self_attn.k_norm.weight") and name in params:
                # [all KV heads x D]; ranks that replicate a KV head take the same slice
                Hkv, n = self.cfg.num_key_value_heads, params[name].shape[0]
                kv_rank = r if Hkv >= tp else r // (tp // Hkv)
                params[name].copy_(w[kv_rank * n:(kv_rank + 1) * n])
                loaded.add(orig_name)
                continue
            if "block_sparse_moe" in name:             # Mixtral's original tensor names
                name = name.replace("block_sparse_moe", "mlp").replace(".w1.", ".gate_proj.") \
                           .replace(".w3.", ".up_proj.").replace(".w2.", ".down_proj.")
            mf = re.match(r"model\.layers\.(\d+)\.mlp\.experts\.(gate_up_proj|down_proj)$", name)
            if mf and int(mf.group(1)) in layers and hasattr(layers[int(mf.group(1))].mlp, "w13"):
                # all experts of a layer in one tensor: [E, 2I, H] (gate rows, then up rows) / [E, H, I]
                L = layers[int(mf.group(1))].mlp
                I = self.cfg.moe_intermediate_size
                if L.ep is not None:
                    w = w[L.expert_start:L.expert_start + L.E_local]
                    if mf.group(2) == "gate_up_proj":
                        L.w13.copy_(w)
                    else:
                        L.w2.copy_(w)
                else:
                    Il = I // tp
                    if mf.group(2) == "gate_up_proj":
                        L.w13[:, :Il].copy_(w[:, r * Il:(r + 1) * Il])
                        L.w13[:, Il:].copy_(w[:, I + r * Il:I + (r + 1) * Il])
                    else:
                        L.w2.copy_(w[:, :, r * Il:(r + 1) * Il])
                loaded.add(orig_name)
                continue
            m = re.match(r"model\.layers\.(\d+)\.(.*)", name)
            if m and int(m.group(1)) not in layers:
                continue
            # routed experts
            me = re.match(r"model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight", name)
            if me:
                L = layers[int(me.group(1))].mlp
                e = int(me.group(2))
                I = self.cfg.moe_intermediate_size
                if L.ep is not None:
                    le = e - L.expert_start
                    if not (0 <= le < L.E_local):
                        continue
                    if me.group(3) == "gate_proj":
                        L.w13[le, :I].copy_(w)
                    elif me.group(3) == "up_proj":
                        L.w13[le, I:].copy_(w)
                    else:
                        L.w2[le].copy_(w)
                else:
                    Il = I // tp
                    if me.group(3) == "gate_proj":
                        L.w13[e, :Il].copy_(w[r * Il:(r + 1) * Il])
                    elif me.group(3) == "up_proj":
                        L.w13[e, Il:].copy_(w[r * Il:(r + 1) * Il])
                    else:
                        L.w2[e].copy_(w[:, r * Il:(r + 1) * Il])
                loaded.add(orig_name)
                continue
            if ".feed_forward." in name or ".pre_ff_layernorm." in name or name.startswith("model.final_layernorm"):
                # Bamba's names for the MLP, the norm in front of it and the last norm
                name = name.replace(".feed_forward.", ".mlp.").replace(".pre_ff_layernorm.", ".post_attention_layernorm.") \
                           .replace("model.final_layernorm", "model.norm")
            ml = re.match(r"model\.layers\.(\d+)\.(?:linear_attn|mamba)\.(.*)", name)
            if ml:
                a = layers[int(ml.group(1))].self_attn
                if getattr(a, "is_linear_attention", False) and a.load_hf(ml.group(2), w, tp, r):
                    loaded.add(orig_name)
                continue
            name = name.replace(".mlp.shared_expert.", ".mlp.shared_experts.")
            if self.cfg.attn_output_gate and name.endswith("self_attn.q_proj.weight"):
                # rows per head: [q (D) | gate (D)] -> q rows into slice 0, gate rows into slice 3 of the merged projection
                D = self.cfg.head_dim
                w4 = w.view(self.cfg.num_attention_heads, 2, D, -1)
                tgt = name.replace("q_proj", "qkv_proj")
                if tgt in params:
                    self._copy_shard(tgt, params[tgt], w4[:, 0].reshape(-1, w.shape[-1]), 0, tp, r)
                    self._copy_shard(tgt, params[tgt], w4[:, 1].reshape(-1, w.shape[-1]), 3, tp, r)
                    loaded.add(orig_name)
                continue
            target, shard_id = name, None
            for hf, (merged, sid) in self._STACKED.items():
                if f".{hf}." in name:
                    target, shard_id = name.replace(hf, merged), sid
                    break
            target = target.replace("kv_a_proj_with_mqa", "kv_a_proj") \
                           .replace("q_a_layernorm", "q_a_norm").replace("kv_a_layernorm", "kv_a_norm")
            if target not in params and name in params:
                target, shard_id = name, None          # e.g. the un-merged q_proj of MLA layers without q_lora
            if target not in params:
                continue
            dst = params[target]
            tp_t, r_t = self._shard_of(target, tp, r)
            self._copy_shard(target, dst, w, shard_id, tp_t, r_t)
            if self.cfg.gemma_norm and (target.endswith("self_attn.q_norm.weight") or target.endswith("self_attn.k_norm.weight")):
                dst.add_(1.0)          # stored as the effective scale (1 + weight) the fused kernel multiplies by
            loaded.add(orig_name)
        for L in self.layers:
            if isinstance(L.self_attn, MLAAttention):
                L.self_attn.process_weights_after_loading()
        for L in self.layers:                  # derived copies follow the new values
            if hasattr(L.mlp, "_gate_bf16"):
                L.mlp._gate_bf16 = None
        return loaded

    def _shard_of(self, target: str, tp: int, r: int) -> tuple[int, int]:
        """(group size, rank) a parameter is sharded over: the TP group unless fine-grained TP
        gives the module a group of its own."""
        from ..parallel import finegrained as fgm
        if "shared_experts" in target and tp > 1:
            from ..platform_config import get_b200_config
            if get_b200_config().enable_shared_expert_dp:
                return 1, 0                     # replicated: every rank loads the whole tensor
        fg = fgm.get_fg()
        if fg is None:
            return tp, r
        g = None
        if ".mlp." in target and ".experts." not in target and "shared_experts" not in target:
            g = fg.mlp_tp
        elif ".self_attn.o_proj." in target:
            g = fg.otp
        elif target.startswith("lm_head"):
            g = fg.lmtp
        elif "embed_tokens" in target:
            g = fg.embed_tp
        return (g.world_size, g.rank_in_group) if g is not None else (tp, r)

    def _copy_shard(self, target: str, dst: torch.Tensor, w: torch.Tensor, shard_id, tp: int, r: int):
        cfg = self.cfg
        if shard_id is not None and "qkv_proj" in target:
            D = cfg.head_dim
            Hq_l = cfg.num_attention_heads // tp
            Hkv = cfg.num_key_value_heads
            Hkv_l = max(1, Hkv // tp)
            if shard_id == 0:
                rows = slice(0, Hq_l * D)
                src = w[r * Hq_l * D:(r + 1) * Hq_l * D]
            elif shard_id == 3:        # output gate rows follow q, k, v
                base = (Hq_l + 2 * Hkv_l) * D
                rows = slice(base, base + Hq_l * D)
                src = w[r * Hq_l * D:(r + 1) * Hq_l * D]
            else:
                kv_rank = r if Hkv >= tp else r // (tp // Hkv)
                base = Hq_l * D + (shard_id - 1) * Hkv_l * D
                rows = slice(base, base + Hkv_l * D)
                src = w[kv_rank * Hkv_l * D:(kv_rank + 1) * Hkv_l * D]
            dst[rows].copy_(src)
            return
        if shard_id is not None:       # gate_up
            n = dst.shape[0] // 2
            dst[shard_id * n:(shard_id + 1) * n].copy_(w[r * n:(r + 1) * n])
            return
        if tuple(dst.shape) == tuple(w.shape):
            dst.copy_(w)
            return
        # TP-sharded single matrices: find the dim that differs
        for d in range(w.dim()):
            if dst.shape[d] != w.shape[d]:
                if d == 0 and ("embed_tokens" in target or "lm_head" in target):
                    n = dst.shape[0]
                    rows = min(max(w.shape[0] - r * n, 0), n)
                    dst[:rows].copy_(w[r * n:r * n + rows])
                else:
                    n = dst.shape[d]
                    dst.copy_(w.narrow(d, r * n, n))
                return
        raise ValueError(f"cannot place {target}: {tuple(w.shape)} -> {tuple(dst.shape)}")


def _internlm2_name(name: str) -> str:
    """InternLM2 tensor names -> the Llama-style names the loader works with."""
    return (name.replace("model.tok_embeddings.", "model.embed_tokens.").replace("output.weight", "lm_head.weight")
            .replace(".attention.wo.", ".self_attn.o_proj.").replace(".attention_norm.", ".input_layernorm.")
            .replace(".ffn_norm.", ".post_attention_layernorm.").replace(".feed_forward.w1.", ".mlp.gate_proj.")
            .replace(".feed_forward.w3.", ".mlp.up_proj.").replace(".feed_forward.w2.", ".mlp.down_proj."))


def iterate_safetensors(path: str):
    """Yields (name, tensor) from every *.safetensors file of an HF checkpoint dir."""
    import glob
    import os
    from safetensors import safe_open
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no safetensors files under {path}")
    for f in files:
        with safe_open(f, framework="pt", device="cpu") as sf:
            for k in sf.keys():
                yield k, sf.get_tensor(k)


def export_hf_state_dict(model: CausalLM) -> dict[str, torch.Tensor]:
    """Inverse of ``load_weights`` for single-rank models (tests, save_sharded_state)."""
    cfg = model.cfg
    out: dict[str, torch.Tensor] = {}
    D = cfg.head_dim
    for name, t in model.named_parameters():
        t = t.detach().cpu()
        if name.endswith("qkv_proj.weight") or name.endswith("qkv_proj.bias"):
            nq, nkv = cfg.num_attention_heads * D, cfg.num_key_value_heads * D
            suffix = name.rsplit(".", 1)[1]
            base = name[: -len("qkv_proj." + suffix)]
            out[f"{base}q_proj.{suffix}"] = t[:nq].clone()
            out[f"{base}k_proj.{suffix}"] = t[nq:nq + nkv].clone()
            out[f"{base}v_proj.{suffix}"] = t[nq + nkv:].clone()
        elif name.endswith("gate_up_proj.weight"):
            n = t.shape[0] // 2
            base = name[: -len("gate_up_proj.weight")]
            out[f"{base}gate_proj.weight"] = t[:n].clone()
            out[f"{base}up_proj.weight"] = t[n:].clone()
        elif name.endswith("experts.w13"):
            base = name[: -len("w13")]
            I = cfg.moe_intermediate_size
            for e in range(t.shape[0]):
                out[f"{base}{e}.gate_proj.weight"] = t[e, :I].clone()
                out[f"{base}{e}.up_proj.weight"] = t[e, I:].clone()
        elif name.endswith("experts.w2"):
            base = name[: -len("w2")]
            for e in range(t.shape[0]):
                out[f"{base}{e}.down_proj.weight"] = t[e].clone()
        else:
            name = name.replace("kv_a_proj.", "kv_a_proj_with_mqa.") \
                       .replace("q_a_norm", "q_a_layernorm").replace("kv_a_norm", "kv_a_layernorm")
            out[name] = t.clone()
    return out
