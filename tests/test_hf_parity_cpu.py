"""Checkpoint compatibility: random-weight transformers models saved as safetensors, loaded by this
framework from the directory, greedy tokens compared with transformers' own generate()."""
import json

import numpy as np
import pytest
import torch

from vllm_ascend_b200 import LLM, SamplingParams


def _save(model, cfg, path):
    from safetensors.torch import save_file
    path.mkdir()
    sd = {k: v.contiguous().clone() for k, v in model.state_dict().items()}
    if getattr(cfg, "tie_word_embeddings", False):
        sd.pop("lm_head.weight", None)           # tied checkpoints store the embedding only
    save_file(sd, str(path / "model.safetensors"))
    d = cfg.to_dict()
    d["architectures"] = [type(model).__name__]
    (path / "config.json").write_text(json.dumps(d, default=str))


def _cases():
    from transformers import LlamaConfig, LlamaForCausalLM, Qwen2Config, Qwen2ForCausalLM, Qwen3Config, \
        Qwen3ForCausalLM, Qwen3MoeConfig, Qwen3MoeForCausalLM
    common = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=256, rope_theta=50000.0, tie_word_embeddings=False)
    yield "llama", LlamaConfig(**common, rms_norm_eps=1e-5), LlamaForCausalLM
    yield "qwen2", Qwen2Config(**common, rms_norm_eps=1e-6), Qwen2ForCausalLM
    l3 = dict(common, max_position_embeddings=512)
    yield "llama31_rope", LlamaConfig(**l3, rms_norm_eps=1e-5, rope_scaling={
        "rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
        "original_max_position_embeddings": 64}), LlamaForCausalLM
    yield "qwen2_yarn", Qwen2Config(**l3, rms_norm_eps=1e-6, rope_scaling={
        "rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64}), Qwen2ForCausalLM
    yield "qwen3", Qwen3Config(**common, head_dim=32, rms_norm_eps=1e-6), Qwen3ForCausalLM
    yield "qwen3_moe", Qwen3MoeConfig(**common, head_dim=32, rms_norm_eps=1e-6, num_experts=4, num_experts_per_tok=2,
                                      moe_intermediate_size=48, norm_topk_prob=True, decoder_sparse_step=1,
                                      mlp_only_layers=[]), Qwen3MoeForCausalLM
    try:
        from transformers import Qwen2MoeConfig, Qwen2MoeForCausalLM
        yield "qwen2_moe", Qwen2MoeConfig(**common, rms_norm_eps=1e-6, num_experts=4, num_experts_per_tok=2,
                                          moe_intermediate_size=48, shared_expert_intermediate_size=64,
                                          norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[]), Qwen2MoeForCausalLM
    except ImportError:
        pass
    try:
        from transformers import DeepseekV2Config, DeepseekV2ForCausalLM
        yield "deepseek_v2", DeepseekV2Config(
            vocab_size=320, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
            num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1, n_routed_experts=8,
            routed_scaling_factor=1.0, kv_lora_rank=32, q_lora_rank=None, qk_rope_head_dim=16, v_head_dim=32,
            qk_nope_head_dim=32, n_group=1, topk_group=1, num_experts_per_tok=2, first_k_dense_replace=1,
            norm_topk_prob=False, topk_method="greedy", max_position_embeddings=256, rope_theta=10000.0,
            tie_word_embeddings=False, rms_norm_eps=1e-6), DeepseekV2ForCausalLM
    except ImportError:
        pass
    try:
        from transformers import MistralConfig, MistralForCausalLM
        yield "mistral", MistralConfig(**common, rms_norm_eps=1e-5, sliding_window=None), MistralForCausalLM
        yield "mistral_window", MistralConfig(**common, rms_norm_eps=1e-5, sliding_window=16), MistralForCausalLM
    except ImportError:
        pass
    try:
        from transformers import Phi3Config, Phi3ForCausalLM
        yield "phi3", Phi3Config(**{**common, "pad_token_id": 0}, rms_norm_eps=1e-5, sliding_window=None), Phi3ForCausalLM
    except ImportError:
        pass
    try:
        from transformers import GemmaConfig, GemmaForCausalLM
        yield "gemma", GemmaConfig(**{**common, "tie_word_embeddings": True}, head_dim=32, rms_norm_eps=1e-6), GemmaForCausalLM
    except ImportError:
        pass
    try:
        from transformers import Qwen3NextConfig, Qwen3NextForCausalLM
        yield "qwen3_next", Qwen3NextConfig(
            vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
            num_key_value_heads=2, head_dim=32, max_position_embeddings=256, rope_theta=10000.0,
            tie_word_embeddings=False, linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16,
            linear_num_key_heads=2, linear_num_value_heads=4, num_experts=4, num_experts_per_tok=2,
            moe_intermediate_size=32, shared_expert_intermediate_size=32, decoder_sparse_step=1, mlp_only_layers=[],
            full_attention_interval=2, partial_rotary_factor=0.25, rms_norm_eps=1e-6), Qwen3NextForCausalLM
    except ImportError:
        pass
    try:
        from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
        yield "deepseek_v3", DeepseekV3Config(
            vocab_size=320, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
            num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1, n_routed_experts=8,
            routed_scaling_factor=2.5, kv_lora_rank=32, q_lora_rank=48, qk_rope_head_dim=16, v_head_dim=32,
            qk_nope_head_dim=32, n_group=4, topk_group=2, num_experts_per_tok=2, first_k_dense_replace=1,
            norm_topk_prob=True, max_position_embeddings=256, rope_theta=10000.0, tie_word_embeddings=False,
            rms_norm_eps=1e-6), DeepseekV3ForCausalLM
    except ImportError:
        pass
    try:
        from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
        yield "deepseek_v3_yarn", DeepseekV3Config(
            vocab_size=320, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1, n_routed_experts=8,
            routed_scaling_factor=2.5, kv_lora_rank=32, q_lora_rank=48, qk_rope_head_dim=16, v_head_dim=32,
            qk_nope_head_dim=32, n_group=4, topk_group=2, num_experts_per_tok=2, first_k_dense_replace=1,
            norm_topk_prob=True, max_position_embeddings=512, rope_theta=10000.0, tie_word_embeddings=False,
            rms_norm_eps=1e-6, rope_scaling={"rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 64,
                                             "beta_fast": 32, "beta_slow": 1, "mscale": 1.0, "mscale_all_dim": 1.0}),             DeepseekV3ForCausalLM
    except ImportError:
        pass
    try:
        from transformers import Glm4Config, Glm4ForCausalLM, GlmConfig, GlmForCausalLM
        glm = dict(common, head_dim=16, rms_norm_eps=1e-5, attention_bias=True, pad_token_id=0)
        yield "glm", GlmConfig(**glm), GlmForCausalLM
        yield "glm4", Glm4Config(**glm), Glm4ForCausalLM
    except ImportError:
        pass
    try:
        from transformers import Ernie4_5Config, Ernie4_5ForCausalLM
        yield "ernie45", Ernie4_5Config(**common, head_dim=16, rms_norm_eps=1e-5, use_bias=False, pad_token_id=0), \
            Ernie4_5ForCausalLM
    except ImportError:
        pass
    try:
        from transformers import Glm4MoeConfig, Glm4MoeForCausalLM
        yield "glm4_moe", Glm4MoeConfig(
            vocab_size=320, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
            num_attention_heads=4, num_key_value_heads=2, head_dim=16, n_routed_experts=8, n_shared_experts=1,
            num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1, max_position_embeddings=256,
            use_qk_norm=True, attention_bias=True, tie_word_embeddings=False, routed_scaling_factor=1.5,
            norm_topk_prob=True, rms_norm_eps=1e-5, pad_token_id=0), Glm4MoeForCausalLM
    except ImportError:
        pass
    try:
        from transformers import Ernie4_5_MoeConfig, Ernie4_5_MoeForCausalLM
        yield "ernie45_moe", Ernie4_5_MoeConfig(
            vocab_size=320, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=4,
            num_attention_heads=4, num_key_value_heads=2, moe_num_experts=8, moe_num_shared_experts=1, moe_k=2,
            moe_layer_start_index=1, moe_layer_end_index=2, max_position_embeddings=256, tie_word_embeddings=False,
            use_bias=False, rms_norm_eps=1e-5, pad_token_id=0), Ernie4_5_MoeForCausalLM
    except ImportError:
        pass
    try:
        from transformers import OlmoeConfig, OlmoeForCausalLM
        yield "olmoe", OlmoeConfig(
            vocab_size=320, hidden_size=64, intermediate_size=32, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, num_experts=8, num_experts_per_tok=2, max_position_embeddings=256,
            tie_word_embeddings=False, rms_norm_eps=1e-5, pad_token_id=0), OlmoeForCausalLM
    except ImportError:
        pass
    try:
        from transformers import GraniteConfig, GraniteForCausalLM
        yield "granite", GraniteConfig(**common, rms_norm_eps=1e-5, embedding_multiplier=6.0, attention_multiplier=0.2,
                                       residual_multiplier=0.4, logits_scaling=4.0, pad_token_id=0), GraniteForCausalLM
    except ImportError:
        pass
    try:
        from transformers import GraniteMoeHybridConfig, GraniteMoeHybridForCausalLM
        yield "granite4_hybrid", GraniteMoeHybridConfig(
            vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=256, layer_types=["mamba", "attention", "mamba"],
            mamba_n_heads=8, mamba_d_head=16, mamba_n_groups=2, mamba_d_state=16, mamba_d_conv=4, mamba_expand=2,
            mamba_chunk_size=16, num_local_experts=0, shared_intermediate_size=96, position_embedding_type="nope",
            tie_word_embeddings=False, embedding_multiplier=3.0, attention_multiplier=0.2, residual_multiplier=0.5,
            logits_scaling=2.0, rms_norm_eps=1e-5, pad_token_id=0), GraniteMoeHybridForCausalLM
    except ImportError:
        pass
    try:
        import transformers as _tf
        yield "seed_oss", _tf.SeedOssConfig(**common, head_dim=16, pad_token_id=0), _tf.SeedOssForCausalLM
        yield "smollm3", _tf.SmolLM3Config(**{**common, "num_hidden_layers": 4}, no_rope_layer_interval=2, pad_token_id=0), \
            _tf.SmolLM3ForCausalLM                                      # every second layer attends without rotary
        yield "olmo2", _tf.Olmo2Config(**common, pad_token_id=0), _tf.Olmo2ForCausalLM
        yield "arcee", _tf.ArceeConfig(**common, pad_token_id=0), _tf.ArceeForCausalLM          # ReLU^2 MLP without a gate
        yield "ministral", _tf.MinistralConfig(**common, head_dim=16, pad_token_id=0), _tf.MinistralForCausalLM
        yield "helium", _tf.HeliumConfig(**common, head_dim=16, pad_token_id=0), _tf.HeliumForCausalLM
        yield "dots1", _tf.Dots1Config(**common, moe_intermediate_size=32, n_routed_experts=8, n_shared_experts=1,
                                       num_experts_per_tok=2, first_k_dense_replace=1, n_group=2, topk_group=1,
                                       pad_token_id=0), _tf.Dots1ForCausalLM
    except (ImportError, AttributeError):
        pass
    try:
        from transformers import BambaConfig, BambaForCausalLM
        yield "bamba", BambaConfig(
            vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=256, attn_layer_indices=[1, 3], mamba_n_heads=8,
            mamba_d_head=16, mamba_n_groups=2, mamba_d_state=16, mamba_d_conv=4, mamba_expand=2,
            mamba_chunk_size=16, tie_word_embeddings=False, rms_norm_eps=1e-5, pad_token_id=0,
            # this transformers release rotates the whole head whatever the factor says; the factor is honoured here
            partial_rotary_factor=1.0,
            rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 1.0}), \
            BambaForCausalLM
        # one group shared by all heads: under TP every rank keeps it (B / C computed redundantly)
        yield "bamba_g1", BambaConfig(
            vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=256, attn_layer_indices=[1], mamba_n_heads=8,
            mamba_d_head=16, mamba_n_groups=1, mamba_d_state=16, mamba_d_conv=4, mamba_expand=2,
            mamba_chunk_size=16, tie_word_embeddings=False, rms_norm_eps=1e-5, pad_token_id=0, partial_rotary_factor=1.0,
            rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 1.0}), \
            BambaForCausalLM
    except ImportError:
        pass
    try:
        from transformers import MiniMaxConfig, MiniMaxForCausalLM
        yield "minimax_text01", MiniMaxConfig(
            vocab_size=320, hidden_size=64, intermediate_size=32, num_hidden_layers=4, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, num_local_experts=4, num_experts_per_tok=2,
            max_position_embeddings=256, rms_norm_eps=1e-5, tie_word_embeddings=False, block_size=16,
            full_attn_alpha_factor=1.5, full_attn_beta_factor=0.9, linear_attn_alpha_factor=1.4,
            linear_attn_beta_factor=1.1, mlp_alpha_factor=1.3, mlp_beta_factor=0.8,
            rope_parameters={"rope_type": "default", "rope_theta": 10000.0}), MiniMaxForCausalLM
    except ImportError:
        pass
    try:
        from transformers import MiniMaxM2Config, MiniMaxM2ForCausalLM
        yield "minimax_m2", MiniMaxM2Config(
            vocab_size=320, hidden_size=64, intermediate_size=32, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=32, num_local_experts=4, num_experts_per_tok=2,
            max_position_embeddings=256, rms_norm_eps=1e-6, tie_word_embeddings=False,
            rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5}), \
            MiniMaxM2ForCausalLM
    except ImportError:
        pass
    try:
        from transformers import MixtralConfig, MixtralForCausalLM
        yield "mixtral", MixtralConfig(**common, rms_norm_eps=1e-5, num_local_experts=4, num_experts_per_tok=2,
                                       sliding_window=None), MixtralForCausalLM
    except ImportError:
        pass


@pytest.mark.parametrize("name", ["llama", "qwen2", "qwen3", "qwen3_moe", "mixtral", "minimax_m2", "minimax_text01", "bamba", "glm4_moe", "ernie45_moe", "olmoe", "granite", "granite4_hybrid", "seed_oss", "smollm3", "olmo2", "arcee", "ministral", "helium", "dots1", "deepseek_v3", "qwen3_next",
                                  "mistral", "phi3", "gemma", "qwen2_moe",
                                  "deepseek_v2", "llama31_rope", "qwen2_yarn",
                                  "deepseek_v3_yarn", "mistral_window", "glm", "glm4", "ernie45"])
def test_greedy_tokens_match_transformers(name, tmp_path):
    case = {n: (c, m) for n, c, m in _cases()}.get(name)
    if case is None:
        pytest.skip(f"transformers has no {name}")
    cfg, cls = case
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = cls(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("A_log") or n.endswith("dt_bias"):
                p.uniform_(-1.0, 1.0)
            elif "norm" in n:
                p.uniform_(0.5, 1.5)
            else:
                p.normal_(0, 0.08)
        for n, b in hf.named_buffers():
            if n.endswith("e_score_correction_bias"):       # the selection bias must matter
                b.uniform_(-0.3, 0.3)
    _save(hf, cfg, tmp_path / name)
    llm = LLM(str(tmp_path / name), device="cpu", dtype="float32", max_model_len=128, max_num_seqs=4,
              max_num_batched_tokens=24, block_size=16)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(1, 300, size=n).tolist() for n in ((100, 7) if "rope" in name or "yarn" in name else (33, 7))]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for p, o in zip(prompts, outs):
        t = torch.tensor([p])
        with torch.no_grad():
            ref = hf.generate(t, attention_mask=torch.ones_like(t), max_new_tokens=8, do_sample=False,
                              pad_token_id=0)[0, len(p):].tolist()
        assert o.outputs[0].token_ids == ref, name


def test_internlm2_names_and_grouped_wqkv_load_like_llama(tmp_path):
    """InternLM2 checkpoints (tok_embeddings / attention.wqkv grouped per KV head / feed_forward.w1,w3,w2 /
    output) give the same model as the Llama-named tensors they were built from."""
    from vllm_ascend_b200.config import ModelConfig
    kw = dict(device="cpu", max_model_len=64, max_num_seqs=2, block_size=16)
    base = dict(vocab_size=256, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, dtype="float32")
    g = torch.Generator().manual_seed(0)
    Hq, Hkv, D, H, I = 4, 2, 16, 64, 96
    llama, intern = {}, {}
    emb, head = torch.randn(256, H, generator=g) * 0.1, torch.randn(256, H, generator=g) * 0.1
    llama["model.embed_tokens.weight"], intern["model.tok_embeddings.weight"] = emb, emb
    llama["lm_head.weight"], intern["output.weight"] = head, head
    nw = torch.rand(H, generator=g) + 0.5
    llama["model.norm.weight"], intern["model.norm.weight"] = nw, nw
    for i in range(2):
        q, k, v = (torch.randn(n, H, generator=g) * 0.1 for n in (Hq * D, Hkv * D, Hkv * D))
        wqkv = torch.cat([q.view(Hkv, Hq // Hkv, D, H), k.view(Hkv, 1, D, H), v.view(Hkv, 1, D, H)], dim=1).reshape(-1, H)
        o = torch.randn(H, Hq * D, generator=g) * 0.1
        w1, w3, w2 = torch.randn(I, H, generator=g) * 0.1, torch.randn(I, H, generator=g) * 0.1, torch.randn(H, I, generator=g) * 0.1
        n1, n2 = torch.rand(H, generator=g) + 0.5, torch.rand(H, generator=g) + 0.5
        L, N = f"model.layers.{i}.", f"model.layers.{i}."
        llama.update({L + "self_attn.q_proj.weight": q, L + "self_attn.k_proj.weight": k, L + "self_attn.v_proj.weight": v,
                      L + "self_attn.o_proj.weight": o, L + "mlp.gate_proj.weight": w1, L + "mlp.up_proj.weight": w3,
                      L + "mlp.down_proj.weight": w2, L + "input_layernorm.weight": n1, L + "post_attention_layernorm.weight": n2})
        intern.update({N + "attention.wqkv.weight": wqkv, N + "attention.wo.weight": o, N + "feed_forward.w1.weight": w1,
                       N + "feed_forward.w3.weight": w3, N + "feed_forward.w2.weight": w2, N + "attention_norm.weight": n1,
                       N + "ffn_norm.weight": n2})
    a = LLM(ModelConfig(name="a", architecture="LlamaForCausalLM", **base), **kw)
    b = LLM(ModelConfig(name="b", architecture="InternLM2ForCausalLM", **base), **kw)
    assert len(a.engine.runner.model.load_weights(llama.items())) == len(llama)
    assert len(b.engine.runner.model.load_weights(intern.items())) == len(intern)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    p = [[3, 9, 27, 81, 5, 15]]
    assert a.generate(p, sp)[0].outputs[0].token_ids == b.generate(p, sp)[0].outputs[0].token_ids
    pa, pb = dict(a.engine.runner.model.named_parameters()), dict(b.engine.runner.model.named_parameters())
    assert all(torch.equal(pa[k], pb[k]) for k in pa)


@pytest.mark.parametrize("name", ["qwen3_next", "deepseek_v3", "gemma", "qwen2_moe", "minimax_m2", "minimax_text01", "bamba", "bamba_g1", "glm4_moe", "granite4_hybrid", "arcee"])
def test_checkpoint_sharding_tp2_matches_tp1(name, tmp_path):
    """The same checkpoint directory loaded by two tensor-parallel ranks (gloo) gives the single-rank
    tokens: per-rank slicing of grouped GDN projections, gated q_proj, fused expert tensors, MLA."""
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_tp_cpu import _run
    case = {n: (c, m) for n, c, m in _cases()}.get(name)
    if case is None:
        pytest.skip(f"transformers has no {name}")
    cfg, cls = case
    torch.manual_seed(0)
    hf = cls(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("A_log") or n.endswith("dt_bias"):
                p.uniform_(-1.0, 1.0)
            elif "norm" in n:
                p.uniform_(0.5, 1.5)
            else:
                p.normal_(0, 0.08)
    cfg.dtype = torch.float32
    _save(hf, cfg, tmp_path / name)
    path = str(tmp_path / name)
    want = _run(path, 1, 1)
    assert _run(path, 2, 2) == want
    if name == "qwen2_moe":          # experts sharded over the two ranks instead (expert parallel, DP attention)
        assert _run(path, 2, 1, ep=True) == want
