"""RMSNorm folded into the GEMMs on both sides of it (dense bf16 decoders on one GPU).

A pre-norm decoder layer alternates ``add + RMSNorm`` with GEMMs.  The norm is cheap arithmetic but
two full passes over the residual stream in HBM per norm.  Here it disappears from the kernel list:

* the norm weight is multiplied into the consumer GEMM's weight at load time (``W' = W * gamma``,
  exact when gamma is 1, one bf16 rounding per weight otherwise; the norm weights become 1, so the
  parameters still describe the same function and can be saved or reloaded);
* the row-parallel GEMM that produces the sub-layer output adds the residual in its epilogue
  (in place on the residual stream) and accumulates every row's sum of squares;
* the consumer GEMM reads the un-normalised residual rows and scales its accumulators by
  ``rsqrt(ss / H + eps)`` in the epilogue (before the bias / SiLU-mul).

Two fp32 row-statistics buffers alternate.  A producer writes one partial sum per column tile and
row (plain stores, no atomics) and the consumer adds a row's partials in tile order, so the
statistics, and with them the whole step, repeat bit for bit; nothing has to be cleared between
GEMMs.  Steps with fewer rows than the paired-CTA kernel takes run the ordinary layer code (which
sees norm weights of 1).

The reference fuses add + RMSNorm (+ quant) as one kernel behind its compiler passes
(vllm_ascend/compilation/passes/norm_quant_fusion_pass.py:29-403); it has no GEMM-epilogue form.
"""
from __future__ import annotations

import torch

from .. import envs, ops


def supports(model, engine_cfg) -> bool:
    from .layers import GQAAttention, SwiGLUMLP
    cfg = model.cfg
    if envs.VLLM_B200_FOLD_NORM == "0" or model.device.type != "cuda":
        return False
    if model.comm.size != 1 or engine_cfg.enable_lora or engine_cfg.enable_sleep_mode:
        return False
    from ..batch_invariant import is_batch_invariant
    if is_batch_invariant():
        return False          # the folded and the ordinary path round differently; which one runs depends on the step size
    from ..platform_config import get_b200_config
    if get_b200_config().weight_offload_config.enabled:
        return False          # offloaded layers hold their weights on the host between their turns
    if engine_cfg.speculative_config or engine_cfg.kv_transfer_config and \
            (engine_cfg.kv_transfer_config.get("kv_connector") == "LayerwiseConnector"):
        return False
    return (not cfg.use_mla and not cfg.is_moe and model.dtype == torch.bfloat16 and not cfg.is_hybrid
            and not cfg.gemma_norm and not cfg.sandwich_norm and cfg.embed_scale == 1.0
            and cfg.residual_multiplier == 1.0 and cfg.logits_scaling == 1.0 and not cfg.qk_norm_full
            and not cfg.deepnorm_factors and cfg.hc_mult <= 1 and cfg.pre_norm
            and cfg.hidden_act in ("silu", "swish") and not cfg.is_multimodal and not cfg.quantization
            and cfg.hidden_size % 8 == 0 and model.is_first and model.is_last
            and all(isinstance(L.self_attn, GQAAttention) and isinstance(L.mlp, SwiGLUMLP)
                    and L.self_attn.qkv_proj.quant is None and L.mlp.gate_up_proj.quant is None
                    and L.mlp.gate_up_proj.weight.shape[0] // 2 % 128 == 0 for L in model.layers))


@torch.no_grad()
def fold_norms(model) -> None:
    """Multiply every layer's two norm weights into the GEMM that consumes the normalised rows and
    set them to 1.  Idempotent (a weight of 1 folds to nothing); called again after weights were
    reloaded in place."""
    for L in model.layers:
        for norm, lin in ((L.input_layernorm, L.self_attn.qkv_proj), (L.post_attention_layernorm, L.mlp.gate_up_proj)):
            g = norm.weight.float()
            if bool((g == 1).all()):
                continue
            lin.weight.copy_((lin.weight.float() * g[None, :]).to(lin.weight.dtype))
            norm.weight.fill_(1.0)
    model.norm_folded = True


def attach(model, engine_cfg) -> bool:
    if not supports(model, engine_cfg):
        return False
    fold_norms(model)
    n = max(engine_cfg.scheduler.max_num_batched_tokens, engine_cfg.scheduler.max_num_seqs) + 8
    model.fold_ss = [ops.alloc_row_stats(n, model.cfg.hidden_size, model.device) for _ in range(2)]
    model.fold_ones = torch.ones(model.cfg.hidden_size, dtype=model.dtype, device=model.device)
    return True


def min_rows() -> int:
    m = envs.VLLM_B200_GEMM_2CTA_MIN_M
    return m if m > 0 else 1 << 30


def forward_folded(model, input_ids: torch.Tensor, meta, kv_caches: list) -> torch.Tensor:
    """Forward pass with the residual stream updated in place by the GEMM epilogues."""
    cfg = model.cfg
    H, eps = cfg.hidden_size, cfg.rms_norm_eps
    r = model.embed_tokens(input_ids)              # [T, H]: becomes the residual stream
    T = r.shape[0]
    ss_a, ss_b = model.fold_ss[0], model.fold_ss[1]
    x0, _ = ops.rms_norm(r, model.fold_ones, eps)  # first norm: nothing upstream produced its statistics
    for i, (layer, cache) in enumerate(zip(model.layers, kv_caches)):
        a, m = layer.self_attn, layer.mlp
        if i == 0:
            qkv = ops.linear_norm_folded(x0, a.qkv_proj.weight, a.qkv_proj.bias)
        else:
            qkv = ops.linear_norm_folded(r, a.qkv_proj.weight, a.qkv_proj.bias, ss_in=ss_a, norm_dim=H, eps=eps)
        o = a.attend(qkv, meta, cache)
        ops.linear_norm_folded(o, a.o_proj.weight, a.o_proj.bias, residual=r, out=r, ss_out=ss_b)
        act = ops.linear_norm_folded(r, m.gate_up_proj.weight, swiglu=True, ss_in=ss_b, norm_dim=H, eps=eps)
        ops.linear_norm_folded(act, m.down_proj.weight, m.down_proj.bias, residual=r, out=r, ss_out=ss_a)
        if model.layer_hook is not None:
            model.layer_hook(layer.idx)
    h, _ = ops.rms_norm(r, model.norm.weight, eps)
    return h
