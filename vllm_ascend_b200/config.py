"""Engine configuration objects and the model presets named by the benchmarks.

``ModelConfig`` is an HF-``config.json``-shaped description of a decoder; it can
be built from a checkpoint directory (``from_pretrained``) or from a preset
(random-init weights).  ``EngineConfig`` groups the cache / scheduler /
parallel knobs, mirroring the fields of upstream ``VllmConfig`` that the
reference reads in ``vllm_ascend/platform.py:343-395``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Optional

import torch


@dataclass
class ModelConfig:
    architecture: str = "Qwen3ForCausalLM"
    vocab_size: int = 1024
    hidden_size: int = 256
    intermediate_size: int = 512
    num_hidden_layers: int = 2
    num_attention_heads: int = 4
    num_key_value_heads: int = 2
    head_dim: int = 64
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_scaling: Optional[dict] = None
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    qk_norm: bool = False            # Qwen3 per-head q/k RMSNorm
    qk_norm_full: bool = False       # MiniMax-M2: RMSNorm over the whole projected q (and k) vector, all heads together
    attention_bias: bool = False     # Qwen2 style qkv bias
    sliding_window: Optional[int] = None
    hidden_act: str = "silu"
    # ---- MoE ----
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    n_shared_experts: int = 0
    norm_topk_prob: bool = True
    scoring_func: str = "softmax"    # "softmax" | "sigmoid"
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    first_k_dense_replace: int = 0   # leading dense layers (DeepSeek)
    moe_layer_end_index: int = -1            # last MoE layer (-1: the last layer); Ernie 4.5 MoE
    moe_layer_interval: int = 1              # every n-th layer inside [first_k_dense_replace, end] is MoE
    e_score_correction_bias: bool = False
    # ---- linear attention (Gated DeltaNet hybrids: every `full_attention_interval`-th layer is
    # softmax attention, the others keep a recurrent state instead of a KV cache) ----
    full_attention_interval: int = 0
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    layer_types: Optional[list] = None       # per layer "linear_attention" | "full_attention" (overrides the interval)
    # Qwen3-Next attention / norm variants
    gemma_norm: bool = False                 # RMSNorm scales by (1 + weight)
    embed_scale: float = 1.0                 # token embeddings are multiplied by this (Gemma: sqrt(hidden))
    partial_rotary_factor: float = 1.0       # fraction of head_dim that is rotated
    no_rope_layers: Optional[list] = None    # per layer: 0 = this layer's attention uses no rotary embedding (SmolLM3)
    rope_interleaved: bool = False           # checkpoint rotates pairs (2i, 2i+1); q / k rows are re-ordered at load
    sandwich_norm: bool = False              # extra RMSNorm on every sub-layer output (GLM-4)
    mlp_gated: bool = True                   # False (Arcee): act(x W_up) W_down without a gate projection
    pre_norm: bool = True                    # False (OLMo-2): sub-layers read the raw stream, only their outputs are normalised
    # Granite: fixed multipliers on the embeddings (embed_scale), the attention scores, every sub-layer output
    # before it joins the residual stream, and the logits (divided by logits_scaling)
    attention_multiplier: Optional[float] = None
    residual_multiplier: float = 1.0
    logits_scaling: float = 1.0
    # MiniMax-Text-01: a sub-layer reads the *normalised* stream and the stream continues from it,
    # x = norm(s); s' = alpha * x + beta * f(x); (attention alpha, beta of full layers, of linear layers, MLP)
    deepnorm_factors: Optional[dict] = None
    # hyper-connections: the residual stream is hc_mult parallel streams mixed by learned weights (0 / 1 = plain residual)
    hc_mult: int = 0
    hc_sinkhorn_iters: int = 20
    linear_attn_kind: str = "gdn"            # "gdn" (Gated DeltaNet) | "lightning" (fixed decay per head) | "mamba2"
    mamba_config: Optional[dict] = None      # Mamba-2 mixer: n_heads, d_head, n_groups, d_state, d_conv, biases, dt limits
    lightning_block_size: int = 0
    split_fused_gate_up: bool = False        # checkpoint stores mlp.gate_up_proj as one [gate; up] tensor
    attn_output_gate: bool = False           # q_proj also produces a per-head sigmoid gate of the attention output
    shared_expert_gate: bool = False         # shared expert output scaled by sigmoid(x . w)
    shared_expert_intermediate_size: int = 0
    # sparse attention (DeepSeek-V3.2 style lightning indexer over MLA): keys kept per query, indexer heads
    index_topk: int = 0
    index_n_heads: int = 0
    index_head_dim: int = 128
    # multimodal (Qwen2-VL family): rotary sections over (temporal, height, width) positions,
    # vision-tower config (HF ``vision_config`` dict) and the placeholder token ids
    mrope_section: Optional[list] = None
    mrope_interleaved: bool = False
    vision_config: Optional[dict] = None
    audio_config: Optional[dict] = None     # HF ``audio_config`` of audio-language models
    audio_token_id: int = -1
    image_token_id: int = -1
    video_token_id: int = -1
    tokens_per_second: float = 2.0
    # ---- MLA ----
    use_mla: bool = False
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # ---- numerics / quantization ----
    dtype: str = "bfloat16"
    quantization: Optional[str] = None   # None | "fp8" (128x128 block) | "w8a8_dynamic"
    quantization_config: Optional[dict] = None   # the checkpoint's own description (compressed-tensors, ModelOpt)
    weight_block_size: tuple = (128, 128)
    init_std: float = 0.02
    seed: int = 0
    name: str = "tiny-qwen"
    model_path: Optional[str] = None

    @property
    def torch_dtype(self) -> torch.dtype:
        return {"bfloat16": torch.bfloat16, "float16": torch.float16,
                "float32": torch.float32}[self.dtype]

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def use_sparse(self) -> bool:
        return self.use_mla and self.index_topk > 0

    @property
    def is_multimodal(self) -> bool:
        return self.vision_config is not None or self.audio_config is not None

    @property
    def is_hybrid(self) -> bool:
        return self.full_attention_interval > 0

    def is_linear_layer(self, layer_idx: int) -> bool:
        if self.layer_types and layer_idx < len(self.layer_types):
            return self.layer_types[layer_idx] == "linear_attention"
        return self.is_hybrid and (layer_idx + 1) % self.full_attention_interval != 0

    def is_moe_layer(self, layer_idx: int) -> bool:
        if not self.is_moe or layer_idx < self.first_k_dense_replace:
            return False
        if self.moe_layer_end_index >= 0 and layer_idx > self.moe_layer_end_index:
            return False
        return (layer_idx + 1) % max(self.moe_layer_interval, 1) == 0

    @property
    def q_head_dim(self) -> int:
        return (self.qk_nope_head_dim + self.qk_rope_head_dim) if self.use_mla else self.head_dim

    @property
    def kv_cache_entry_dims(self) -> tuple[int, int]:
        """Per-token per-layer widths of the two cache tensors.

        GQA: (kv_heads*head_dim, kv_heads*head_dim); MLA: (kv_lora_rank, rope_dim)
        — the layout contract of vllm_ascend/worker/model_runner_v1.py:3994-4069.
        """
        if self.use_mla:
            return (self.kv_lora_rank, self.qk_rope_head_dim)
        w = self.num_key_value_heads * self.head_dim
        return (w, w)

    # ------------------------------------------------------------------
    @classmethod
    def from_hf_dict(cls, d: dict, **over) -> "ModelConfig":
        arch = (d.get("architectures") or ["LlamaForCausalLM"])[0]
        top = d
        if "text_config" in d and "hidden_size" not in d:      # nested multimodal layout
            d = {**d["text_config"], "architectures": [arch]}
            for k in ("vision_config", "image_token_id", "video_token_id", "quantization_config",
                      "tie_word_embeddings", "audio_config", "audio_token_id", "audio_token_index"):
                if k in top and (k not in d or k != "tie_word_embeddings"):
                    d[k] = top[k]
        hs = d["hidden_size"]
        nh = d["num_attention_heads"]
        rp_ = d.get("rope_parameters") or {}
        if not d.get("rope_scaling") and (rp_.get("rope_type") or rp_.get("type")) not in (None, "default", "mrope"):
            d = dict(d, rope_scaling={k: v for k, v in rp_.items() if k != "rope_theta"})   # newer config layout
        if "rope_theta" not in d and rp_.get("rope_theta"):
            d = dict(d, rope_theta=rp_["rope_theta"])
        kw: dict[str, Any] = dict(
            architecture=arch,
            vocab_size=d["vocab_size"], hidden_size=hs,
            intermediate_size=d.get("intermediate_size", 4 * hs),
            num_hidden_layers=d["num_hidden_layers"], num_attention_heads=nh,
            num_key_value_heads=d.get("num_key_value_heads", nh),
            head_dim=d.get("head_dim") or hs // nh,
            rms_norm_eps=d.get("rms_norm_eps", 1e-6),
            rope_theta=d.get("rope_theta", 10000.0),
            rope_scaling=d.get("rope_scaling"),
            max_position_embeddings=d.get("max_position_embeddings", 32768),
            tie_word_embeddings=d.get("tie_word_embeddings", False),
            qk_norm=arch.startswith("Qwen3"),
            attention_bias=d.get("attention_bias", arch.startswith("Qwen2")),
            # Qwen2 gates its window with use_sliding_window; Mistral-style configs apply it whenever it is set
            sliding_window=(d.get("sliding_window") if d.get("use_sliding_window", not arch.startswith("Qwen"))
                            else None),
            hidden_act=d.get("hidden_activation") or d.get("hidden_act", "silu"),
            dtype=str(d.get("torch_dtype") or d.get("dtype") or "bfloat16").replace("torch.", ""),
        )
        if d.get("shared_expert_intermediate_size"):       # Qwen2-MoE / Qwen3-Next: one gated shared expert
            kw.update(shared_expert_intermediate_size=int(d["shared_expert_intermediate_size"]), shared_expert_gate=True)
        if arch.startswith("Glm4Moe"):
            # GLM-4.5 / 4.6: Llama-style attention with optional per-head q / k norms, half of every head
            # rotated (rotate-half pairing), DeepSeek-V3 style router (sigmoid, selection bias, expert groups)
            kw.update(qk_norm=bool(d.get("use_qk_norm", False)), attention_bias=bool(d.get("attention_bias", False)),
                      partial_rotary_factor=float(rp_.get("partial_rotary_factor", d.get("partial_rotary_factor", 0.5))))
            d = dict(d, scoring_func="sigmoid", topk_method="noaux_tc")
        elif arch.startswith("Glm"):
            kw.update(rope_interleaved=True, split_fused_gate_up=True, sandwich_norm=arch.startswith("Glm4"),
                      partial_rotary_factor=float(d.get("partial_rotary_factor",
                                                        (d.get("rope_parameters") or {}).get("partial_rotary_factor", 0.5))),
                      attention_bias=bool(d.get("attention_bias", True)))
        if arch.startswith("Ernie4_5"):
            kw.update(rope_interleaved=True, attention_bias=bool(d.get("use_bias", False)),
                      tie_word_embeddings=d.get("tie_word_embeddings", True))
        if arch.startswith("GraniteMoeHybrid"):
            # Granite 4 hybrids: Mamba-2 / attention layers by layer_types, attention without rotary
            # ("nope"), a gated MLP stored as one fused input projection (dense form: no routed experts)
            if d.get("num_local_experts"):
                raise ValueError("GraniteMoeHybrid with routed experts is not supported (dense shared MLP only)")
            lt = [("full_attention" if t == "attention" else "linear_attention") for t in d["layer_types"]]
            kw.update(linear_attn_kind="mamba2", full_attention_interval=2, layer_types=lt, split_fused_gate_up=True,
                      intermediate_size=int(d.get("shared_intermediate_size", kw["intermediate_size"])),
                      partial_rotary_factor=0.0 if d.get("position_embedding_type", "rope") == "nope" else 1.0,
                      mamba_config={"n_heads": d["mamba_n_heads"], "d_head": d["mamba_d_head"],
                                    "n_groups": d.get("mamba_n_groups", 1), "d_state": d.get("mamba_d_state", 256),
                                    "d_conv": d.get("mamba_d_conv", 4), "conv_bias": d.get("mamba_conv_bias", True),
                                    "proj_bias": d.get("mamba_proj_bias", False),
                                    "chunk_size": d.get("mamba_chunk_size", 256),
                                    "time_step_limit": [float(x) for x in d.get("time_step_limit", (0.0, float("inf")))]})
            d = dict(d, num_local_experts=0)
        if arch.startswith("Bamba"):
            attn_idx = set(d.get("attn_layer_indices") or [])
            kw.update(linear_attn_kind="mamba2", full_attention_interval=2,
                      layer_types=["full_attention" if i in attn_idx else "linear_attention"
                                   for i in range(d["num_hidden_layers"])],
                      partial_rotary_factor=float(rp_.get("partial_rotary_factor", d.get("partial_rotary_factor", 0.5))),
                      mamba_config={"n_heads": d["mamba_n_heads"], "d_head": d["mamba_d_head"],
                                    "n_groups": d.get("mamba_n_groups", 1), "d_state": d.get("mamba_d_state", 256),
                                    "d_conv": d.get("mamba_d_conv", 4), "conv_bias": d.get("mamba_conv_bias", True),
                                    "proj_bias": d.get("mamba_proj_bias", False),
                                    "chunk_size": d.get("mamba_chunk_size", 256),
                                    "time_step_limit": [float(x) for x in d.get("time_step_limit", (0.0, float("inf")))]})
        if arch == "MiniMaxForCausalLM" or arch.startswith("MiniMaxText01"):
            lt = d.get("layer_types") or ["full_attention" if (i + 1) % 2 else "linear_attention"
                                          for i in range(d["num_hidden_layers"])]
            kw.update(linear_attn_kind="lightning", layer_types=list(lt), full_attention_interval=2,
                      lightning_block_size=min(int(d.get("block_size", 256)), 64),
                      deepnorm_factors={"full": (float(d.get("full_attn_alpha_factor", 1)), float(d.get("full_attn_beta_factor", 1))),
                                        "linear": (float(d.get("linear_attn_alpha_factor", 1)), float(d.get("linear_attn_beta_factor", 1))),
                                        "mlp": (float(d.get("mlp_alpha_factor", 1)), float(d.get("mlp_beta_factor", 1)))})
        if d.get("hc_mult"):
            kw.update(hc_mult=int(d["hc_mult"]), hc_sinkhorn_iters=int(d.get("hc_sinkhorn_iters", 20)))
        if d.get("no_rope_layers"):
            kw.update(no_rope_layers=[int(x) for x in d["no_rope_layers"]])
        if arch.startswith("Dots1"):
            # dots.llm1: Qwen3-style per-head q / k norms on a DeepSeek-V3 style MoE (sigmoid router, selection bias)
            kw.update(qk_norm=True)
            d = dict(d, scoring_func="sigmoid", topk_method="noaux_tc")
        if arch.startswith("Helium"):
            kw.update(rope_interleaved=True)
        if arch.startswith("Granite"):
            kw.update(embed_scale=float(d.get("embedding_multiplier", 1.0)),
                      attention_multiplier=float(d["attention_multiplier"]) if d.get("attention_multiplier") else None,
                      residual_multiplier=float(d.get("residual_multiplier", 1.0)),
                      logits_scaling=float(d.get("logits_scaling", 1.0)),
                      tie_word_embeddings=d.get("tie_word_embeddings", True))
        if arch.startswith("Arcee"):
            kw.update(mlp_gated=False)
        if arch.startswith("Olmo2"):
            # OLMo-2: no norm in front of a sub-layer, RMSNorm on its output; q / k normalised over all heads
            kw.update(pre_norm=False, sandwich_norm=True, qk_norm_full=True)
        if arch.startswith("Olmoe"):
            # OLMoE: q / k normalised over all heads at once, softmax router without renormalisation by default
            kw.update(qk_norm_full=True)
            d = dict(d, norm_topk_prob=bool(d.get("norm_topk_prob", False)))
        if arch.startswith("MiniMaxM2"):
            # sigmoid router with a selection bias and renormalised weights, rotary on the first rotary_dim
            # channels of a head, q / k normalised over all heads at once
            prf = rp_.get("partial_rotary_factor", d.get("partial_rotary_factor"))
            if prf is None:                     # the published config names the rotated width instead
                prf = float(d.get("rotary_dim", kw["head_dim"])) / kw["head_dim"]
            kw.update(qk_norm_full=True, partial_rotary_factor=float(prf))
            d = dict(d, scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True)
        if arch.startswith("Gemma"):
            kw.update(gemma_norm=True, embed_scale=float(hs) ** 0.5,
                      tie_word_embeddings=d.get("tie_word_embeddings", True))
        if arch.startswith("Ernie4_5_Moe"):
            # softmax router whose selection (not the weights) is shifted by a learned bias; MoE layers from
            # moe_layer_start_index to moe_layer_end_index, every moe_layer_interval-th
            start = d.get("moe_layer_start_index", 0)
            end = d.get("moe_layer_end_index", -1)
            d = dict(d, num_experts=d.get("moe_num_experts", 0), num_experts_per_tok=d.get("moe_k", 2),
                     n_shared_experts=d.get("moe_num_shared_experts", 0), scoring_func="softmax",
                     topk_method="noaux_tc", norm_topk_prob=True,
                     first_k_dense_replace=int(start if isinstance(start, int) else min(start)))
            kw.update(moe_layer_end_index=int(end if isinstance(end, int) else max(end)),
                      moe_layer_interval=int(d.get("moe_layer_interval", 1)))
        n_exp = d.get("num_experts") or d.get("n_routed_experts") or d.get("num_local_experts") or 0
        if n_exp:
            kw.update(
                num_experts=n_exp,
                num_experts_per_tok=d.get("num_experts_per_tok", 0),
                # Mixtral-style configs size their experts with intermediate_size
                moe_intermediate_size=d.get("moe_intermediate_size") or d.get("intermediate_size", 0),
                n_shared_experts=d.get("n_shared_experts", 0) or 0,
                norm_topk_prob=d.get("norm_topk_prob", True),
                # DeepSeek-V3 family routers are sigmoid + bias-corrected top-k even when the config omits it
                scoring_func=d.get("scoring_func", "sigmoid" if arch.startswith("DeepseekV3") else "softmax"),
                n_group=d.get("n_group", 1) or 1, topk_group=d.get("topk_group", 1) or 1,
                routed_scaling_factor=d.get("routed_scaling_factor", 1.0),
                first_k_dense_replace=d.get("first_k_dense_replace", 0),
                e_score_correction_bias=d.get("topk_method", "noaux_tc" if arch.startswith("DeepseekV3") else "")
                == "noaux_tc",
            )
        if d.get("index_topk"):
            kw.update(index_topk=int(d["index_topk"]), index_n_heads=int(d.get("index_n_heads", 64)),
                      index_head_dim=int(d.get("index_head_dim", 128)))
        if "kv_lora_rank" in d:
            kw.update(use_mla=True, q_lora_rank=d.get("q_lora_rank"),
                      kv_lora_rank=d["kv_lora_rank"],
                      qk_nope_head_dim=d["qk_nope_head_dim"],
                      qk_rope_head_dim=d["qk_rope_head_dim"], v_head_dim=d["v_head_dim"])
        if d.get("full_attention_interval") or "linear_num_value_heads" in d:
            rp = d.get("rope_parameters") or {}
            lt = d.get("layer_types")
            interval = d.get("full_attention_interval") or ((lt.index("full_attention") + 1) if lt and "full_attention" in lt else 4)
            kw.update(full_attention_interval=int(interval), layer_types=list(lt) if lt else None,
                      linear_num_key_heads=d["linear_num_key_heads"], linear_num_value_heads=d["linear_num_value_heads"],
                      linear_key_head_dim=d["linear_key_head_dim"], linear_value_head_dim=d["linear_value_head_dim"],
                      linear_conv_kernel_dim=d.get("linear_conv_kernel_dim", 4),
                      gemma_norm=True, attn_output_gate=True, qk_norm=True,
                      partial_rotary_factor=float(d.get("partial_rotary_factor", rp.get("partial_rotary_factor", 1.0))),
                      shared_expert_intermediate_size=int(d.get("shared_expert_intermediate_size", 0) or 0),
                      shared_expert_gate=bool(d.get("shared_expert_intermediate_size")))
            if rp.get("rope_theta") and "rope_theta" not in d:
                kw["rope_theta"] = rp["rope_theta"]
        rs = d.get("rope_scaling") or d.get("rope_parameters") or {}
        if rs.get("mrope_section"):
            kw.update(mrope_section=list(rs["mrope_section"]),
                      mrope_interleaved=bool(rs.get("mrope_interleaved", False)))
            if rs.get("rope_theta") and "rope_theta" not in d:
                kw["rope_theta"] = rs["rope_theta"]
            if (rs.get("rope_type") or rs.get("type")) in ("mrope", "default", None):
                kw["rope_scaling"] = None
        if d.get("vision_config"):
            vc = dict(d["vision_config"])
            kw.update(vision_config=vc, image_token_id=d.get("image_token_id", -1),
                      video_token_id=d.get("video_token_id", -1),
                      tokens_per_second=float(vc.get("tokens_per_second", 2.0)))
        if d.get("audio_config"):
            kw.update(audio_config=dict(d["audio_config"]),
                      audio_token_id=int(d.get("audio_token_id", d.get("audio_token_index", -1))))
        qc = d.get("quantization_config")
        if qc:
            method = qc.get("quant_method", "")
            if method == "fp8" and qc.get("weight_block_size"):
                kw.update(quantization="fp8", weight_block_size=tuple(qc["weight_block_size"]))
            elif method == "compressed-tensors":
                kw.update(quantization="compressed-tensors", quantization_config=dict(qc))
            elif method:
                kw.update(quantization=method, quantization_config=dict(qc))
        kw.update(over)
        return cls(**kw)

    @classmethod
    def from_pretrained(cls, path: str, **over) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            d = json.load(f)
        mo = os.path.join(path, "hf_quant_config.json")       # ModelOpt exports keep their description here
        if "quantization_config" not in d and os.path.exists(mo):
            with open(mo) as f:
                d = dict(d, quantization_config=dict(json.load(f), quant_method="modelopt"))
        cfg = cls.from_hf_dict(d, **over)
        cfg.model_path = path
        cfg.name = os.path.basename(os.path.normpath(path))
        return cfg

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["torch_dtype"] = self.dtype
        if self.is_moe:
            d["n_routed_experts"] = self.num_experts
        return d


def _preset(**kw) -> ModelConfig:
    return ModelConfig(**kw)


#: Architectures named by the benchmark configs (random-init, synthetic prompts).
PRESETS: dict[str, Any] = {
    "tiny-qwen": lambda: _preset(
        name="tiny-qwen", architecture="Qwen3ForCausalLM", vocab_size=1024, hidden_size=256,
        intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=64, rope_theta=1e6, qk_norm=True, dtype="float32"),
    "qwen3-8b": lambda: _preset(
        name="qwen3-8b", architecture="Qwen3ForCausalLM", vocab_size=151936, hidden_size=4096,
        intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
        num_key_value_heads=8, head_dim=128, rope_theta=1e6, qk_norm=True,
        max_position_embeddings=40960),
    "llama-3.1-70b": lambda: _preset(
        name="llama-3.1-70b", architecture="LlamaForCausalLM", vocab_size=128256,
        hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
        num_attention_heads=64, num_key_value_heads=8, head_dim=128, rope_theta=5e5,
        rms_norm_eps=1e-5, max_position_embeddings=131072),
    "qwen3-30b-a3b": lambda: _preset(
        name="qwen3-30b-a3b", architecture="Qwen3MoeForCausalLM", vocab_size=151936,
        hidden_size=2048, intermediate_size=6144, num_hidden_layers=48,
        num_attention_heads=32, num_key_value_heads=4, head_dim=128, rope_theta=1e6,
        qk_norm=True, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
        norm_topk_prob=True, max_position_embeddings=40960),
    "deepseek-v3": lambda: _preset(
        name="deepseek-v3", architecture="DeepseekV3ForCausalLM", vocab_size=129280,
        hidden_size=7168, intermediate_size=18432, num_hidden_layers=61,
        num_attention_heads=128, num_key_value_heads=128, head_dim=192, rope_theta=1e4,
        num_experts=256, num_experts_per_tok=8, moe_intermediate_size=2048,
        n_shared_experts=1, scoring_func="sigmoid", n_group=8, topk_group=4,
        routed_scaling_factor=2.5, first_k_dense_replace=3, e_score_correction_bias=True,
        use_mla=True, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
        qk_rope_head_dim=64, v_head_dim=128, quantization="fp8",
        max_position_embeddings=163840),
    # small shapes of each family for tests
    "tiny-llama": lambda: _preset(
        name="tiny-llama", architecture="LlamaForCausalLM", vocab_size=512, hidden_size=128,
        intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, rope_theta=1e4, dtype="float32"),
    "tiny-mqa": lambda: _preset(          # one KV head: replicated over TP ranks (decode context parallelism)
        name="tiny-mqa", architecture="Qwen3ForCausalLM", vocab_size=512, hidden_size=128,
        intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=1, head_dim=32, rope_theta=1e6, qk_norm=True, dtype="float32"),
    "tiny-moe": lambda: _preset(
        name="tiny-moe", architecture="Qwen3MoeForCausalLM", vocab_size=512, hidden_size=128,
        intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, rope_theta=1e6, qk_norm=True, num_experts=8,
        num_experts_per_tok=2, moe_intermediate_size=64, dtype="float32"),
    "tiny-deepseek-sparse": lambda: _preset(
        name="tiny-deepseek-sparse", architecture="DeepseekV32ForCausalLM", vocab_size=512,
        hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
        num_key_value_heads=4, head_dim=48, rope_theta=1e4, num_experts=8,
        num_experts_per_tok=2, moe_intermediate_size=64, n_shared_experts=1,
        scoring_func="sigmoid", n_group=4, topk_group=2, routed_scaling_factor=2.5,
        first_k_dense_replace=1, e_score_correction_bias=True, use_mla=True, q_lora_rank=64,
        kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, dtype="float32",
        index_topk=16, index_n_heads=4, index_head_dim=32),
    "tiny-vl": lambda: _preset(
        name="tiny-vl", architecture="Qwen2_5_VLForConditionalGeneration", vocab_size=512, hidden_size=128,
        intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        head_dim=32, rope_theta=1e6, attention_bias=True, dtype="float32", mrope_section=[4, 6, 6],
        image_token_id=500, video_token_id=501,
        vision_config=dict(depth=2, hidden_size=64, num_heads=4, intermediate_size=96, out_hidden_size=128,
                           patch_size=14, window_size=56, fullatt_block_indexes=[1])),
    "tiny-gdn": lambda: _preset(
        name="tiny-gdn", architecture="Qwen3NextForCausalLM", vocab_size=512, hidden_size=128,
        intermediate_size=256, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
        head_dim=32, rope_theta=1e6, qk_norm=True, dtype="float32", full_attention_interval=2,
        linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32,
        linear_value_head_dim=32, linear_conv_kernel_dim=4),
    "tiny-deepseek": lambda: _preset(
        name="tiny-deepseek", architecture="DeepseekV3ForCausalLM", vocab_size=512,
        hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
        num_key_value_heads=4, head_dim=48, rope_theta=1e4, num_experts=8,
        num_experts_per_tok=2, moe_intermediate_size=64, n_shared_experts=1,
        scoring_func="sigmoid", n_group=4, topk_group=2, routed_scaling_factor=2.5,
        first_k_dense_replace=1, e_score_correction_bias=True, use_mla=True, q_lora_rank=64,
        kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
        dtype="float32"),
}


def get_model_config(name_or_path: str, **over) -> ModelConfig:
    if name_or_path in PRESETS:
        cfg = PRESETS[name_or_path]()
        for k, v in over.items():
            setattr(cfg, k, v)
        return cfg
    if os.path.isdir(name_or_path):
        return ModelConfig.from_pretrained(name_or_path, **over)
    raise ValueError(f"unknown model {name_or_path!r}: not a preset {sorted(PRESETS)} nor a directory")


@dataclass
class CacheConfig:
    block_size: int = 128              # reference default (vllm_ascend/utils.py:1162-1212)
    gpu_memory_utilization: float = 0.92
    num_gpu_blocks: Optional[int] = None   # override; else profiled
    enable_prefix_caching: bool = False
    kv_cache_dtype: str = "auto"
    kv_layout: str = "HND"             # physical order inside a block: HND (per-head pages) | NHD


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 1024
    max_num_batched_tokens: int = 8192
    max_model_len: int = 4096
    enable_chunked_prefill: bool = True
    policy: str = "fcfs"               # fcfs | short_request_first | batch_job | recompute
    async_scheduling: bool = False
    reserve_full_sequence: bool = True   # admit only what can finish without preemption
    decode_batch_alignment: int = 1      # rows per decode GEMM tile (256 on GPU, see Scheduler)


@dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    enable_expert_parallel: bool = False
    decode_context_parallel_size: int = 1
    prefill_context_parallel_size: int = 1
    enable_sequence_parallel: bool = False
    rank: int = 0
    local_rank: int = 0
    world_size: int = 1
    backend: str = "nccl"


@dataclass
class CompilationConfig:
    """CUDA-graph settings (modes of vllm_ascend/platform.py:937-1008)."""
    cudagraph_mode: str = "FULL_DECODE_ONLY"   # NONE|PIECEWISE|FULL|FULL_DECODE_ONLY|FULL_AND_PIECEWISE
    cudagraph_capture_sizes: Optional[list] = None
    max_cudagraph_capture_size: Optional[int] = None


@dataclass
class EngineConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    cache: CacheConfig = field(default_factory=CacheConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    compilation: CompilationConfig = field(default_factory=CompilationConfig)
    additional_config: dict = field(default_factory=dict)
    device: str = "cuda"
    device_index: Optional[int] = None      # single-process engines only
    seed: int = 0
    kv_transfer_config: Optional[dict] = None
    ec_transfer_config: Optional[dict] = None      # disaggregated vision encoder (encoder-cache transfer)
    speculative_config: Optional[dict] = None
    enable_sleep_mode: bool = False
    load_format: str = "auto"               # auto | netloader | rfork
    model_loader_extra_config: Optional[dict] = None
    async_scheduling: Optional[bool] = None     # None: on for single-process CUDA engines
    enable_lora: bool = False
    max_loras: int = 4
    max_lora_rank: int = 64
