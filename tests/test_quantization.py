"""Quantization configs, scheme registry and reference numerics (CPU)."""
import json

import pytest
import torch

from vllm_ascend_b200 import quantization as Q
from vllm_ascend_b200.config import ModelConfig, get_model_config
from vllm_ascend_b200.models.layers import Linear
from vllm_ascend_b200.ops import reference as ref
from vllm_ascend_b200.quantization import schemes


def test_registry_has_linear_and_moe_schemes():
    have = Q.registered()
    for key in [("FP8_BLOCK", "linear"), ("W8A8_DYNAMIC", "linear"), ("W8A8", "linear"),
                ("W8A8FP8_DYNAMIC", "linear"), ("W4A16", "linear"), ("W8A16", "linear"),
                ("FP8_BLOCK", "moe"), ("W8A8_DYNAMIC", "moe"), ("W8A8FP8_DYNAMIC", "moe")]:
        assert key in have
    with pytest.raises(ValueError):
        Q.get_scheme_class("W3A3", "linear")
    with pytest.raises(ValueError):
        Q.register_scheme("FP8_BLOCK", "linear")(type("Dup", (), {}))


@pytest.mark.parametrize("N,K", [(256, 512), (130, 200)])
def test_block_fp8_weight_roundtrip(N, K):
    w = torch.randn(N, K) * 0.1
    q, s = schemes.quantize_weight_block_fp8(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == ((N + 127) // 128, (K + 127) // 128)
    back = ref.dequant_block_fp8_weight(q, s)
    assert (back - w).abs().max() < 0.07 * w.abs().max()


@pytest.mark.parametrize("name,tol", [("FP8_BLOCK", 0.06), ("W8A8_DYNAMIC", 0.03),
                                      ("W8A8FP8_DYNAMIC", 0.08), ("W8A16", 0.02), ("W4A16", 0.25),
                                      ("W8A8_MXFP8", 0.08), ("W4A4_MXFP4", 0.5), ("W4A8_MXFP", 0.35),
                                      ("W4A8_DYNAMIC", 0.25)])
def test_linear_schemes_approximate_float(name, tol):
    torch.manual_seed(0)
    lin = Linear(torch.randn(96, 256) * 0.1, torch.randn(96) * 0.1)
    x = torch.randn(7, 256)
    exp = x @ lin.weight.t() + lin.bias
    scheme = Q.get_scheme_class(name, "linear")()
    scheme.convert(lin)
    lin.quant = Q.LinearMethod(scheme)
    got = lin(x)
    assert (got - exp).abs().max() < tol * exp.abs().max() + 1e-3
    assert dict(lin.named_tensors()).keys() >= {"weight"}


def test_compressed_tensors_detection():
    grp = lambda w, a: {"config_groups": {"g0": {"weights": w, "input_activations": a}}}
    assert Q.detect_compressed_tensors(grp({"num_bits": 8, "type": "int"}, {"dynamic": True})) == "W8A8_DYNAMIC"
    assert Q.detect_compressed_tensors(grp({"num_bits": 8, "type": "int"}, {"dynamic": False})) == "W8A8"
    assert Q.detect_compressed_tensors(grp({"num_bits": 4, "type": "int"}, None)) == "W4A16"
    assert Q.detect_compressed_tensors(grp({"num_bits": 8, "type": "float", "strategy": "block"}, {"dynamic": True})) == "FP8_BLOCK"
    with pytest.raises(ValueError):
        Q.detect_compressed_tensors({"config_groups": {}})


def test_hf_fp8_config_is_detected():
    d = get_model_config("tiny-qwen").to_hf_dict()
    d["quantization_config"] = {"quant_method": "fp8", "weight_block_size": [128, 128]}
    cfg = ModelConfig.from_hf_dict(d)
    assert cfg.quantization == "fp8" and cfg.weight_block_size == (128, 128)


def test_description_file_routes_layers(tmp_path):
    from vllm_ascend_b200.models.transformer import CausalLM
    cfg = get_model_config("tiny-qwen")
    desc = {"model.layers.0.self_attn.qkv_proj.weight": "W8A8_DYNAMIC",
            "model.layers.0.mlp.down_proj.weight": "FLOAT"}
    (tmp_path / "quant_model_description.json").write_text(json.dumps(desc))
    cfg.quantization, cfg.model_path = None, None
    model = CausalLM(cfg, "cpu", max_model_len=64)
    cfg.quantization, cfg.model_path = "ascend", str(tmp_path)
    chosen = Q.apply_quantization(model, cfg)
    assert chosen["model.layers.0.self_attn.qkv_proj"] == "W8A8_DYNAMIC"
    assert chosen["model.layers.0.mlp.down_proj"] == "FLOAT"
    assert model.layers[0].self_attn.qkv_proj.quant is not None
    assert model.layers[0].mlp.down_proj.quant is None
    assert model.layers[1].self_attn.qkv_proj.quant is None     # not listed -> FLOAT


def test_mx_formats_use_power_of_two_block_scales_and_element_grids():
    torch.manual_seed(1)
    x = torch.randn(5, 128) * torch.logspace(-3, 2, 5).unsqueeze(1)
    for elem, grid_max in (("fp8", 448.0), ("fp4", 6.0)):
        q, s = schemes.mx_quantize(x, elem)
        assert s.shape == (5, 4)
        assert torch.equal(torch.log2(s), torch.log2(s).round())            # e8m0: powers of two only
        assert q.abs().max() <= grid_max
        back = schemes.mx_dequantize(q, s)
        tol = 0.07 if elem == "fp8" else 0.3
        assert ((back - x).abs() <= tol * x.abs().reshape(5, 4, 32).amax(-1, keepdim=True).expand(5, 4, 32).reshape(5, 128) + 1e-9).all()
    q4, _ = schemes.mx_quantize(x, "fp4")
    assert set(q4.abs().unique().tolist()) <= {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0}


def test_moe_schemes_for_compressed_expert_weights():
    from vllm_ascend_b200.ops.fused_moe import fused_experts_ref
    torch.manual_seed(2)
    E, I, H, T = 4, 64, 128, 9
    w13, w2 = torch.randn(E, 2 * I, H) * 0.1, torch.randn(E, H, I) * 0.1
    x = torch.randn(T, H)
    ids = torch.randint(0, E, (T, 2))
    wts = torch.rand(T, 2)
    want = fused_experts_ref(x, w13, w2, wts, ids, None)
    for name, tol in (("W8A8FP8_DYNAMIC", 0.08), ("W8A8_MXFP8", 0.08), ("W4A4_MXFP4", 0.5), ("W4A8_DYNAMIC", 0.3), ("W4A16", 0.3),
                      ("W4A16_MXFP4", 0.5), ("W4A8_MXFP", 0.5)):
        blk = type("B", (), {})()
        blk.w13, blk.w2 = w13.clone(), w2.clone()
        sch = Q.get_scheme_class(name, "moe")()
        sch.convert(blk)
        got = sch.apply_experts(x, blk.w13, blk.w2, wts, ids, None)
        assert (got - want).abs().max() < tol * want.abs().max() + 1e-3, name


def test_kv_cache_fp8_roundtrip():
    x = torch.randn(6, 4, 32)
    scale = x.abs().amax(dim=(0, 2)) / 448.0
    q = schemes.kv_quant_fp8(x, scale)
    assert q.dtype == torch.float8_e4m3fn
    assert (schemes.kv_dequant_fp8(q, scale, torch.float32) - x).abs().max() < 0.07 * x.abs().max()


def test_description_of_fused_layers_and_modelopt_detection():
    """A per-weight description names checkpoint projections; the fused qkv / gate_up layers take the
    type of their parts and refuse parts that disagree.  ModelOpt exports select a scheme by algorithm."""
    import pytest
    from vllm_ascend_b200.quantization import description_quant_type, detect_modelopt
    d = {"model.layers.0.self_attn.q_proj.weight": "W8A8_DYNAMIC", "model.layers.0.self_attn.k_proj.weight": "W8A8_DYNAMIC",
         "model.layers.0.self_attn.v_proj.weight": "W8A8_DYNAMIC", "model.layers.0.mlp.gate_proj.weight": "W8A8",
         "model.layers.0.mlp.up_proj.weight": "FLOAT", "model.layers.0.mlp.down_proj.weight": "w8a8",
         "model.layers.1.self_attn.q_proj.weight": "W4A16", "model.layers.1.self_attn.k_proj.weight": "W4A16"}
    assert description_quant_type(d, "model.layers.0.self_attn.qkv_proj") == "W8A8_DYNAMIC"
    assert description_quant_type(d, "model.layers.0.mlp.down_proj") == "W8A8"
    assert description_quant_type(d, "model.layers.1.self_attn.qkv_proj") == "W4A16"      # k == v checkpoints: no v_proj
    assert description_quant_type(d, "model.layers.2.self_attn.qkv_proj") == "FLOAT"
    with pytest.raises(ValueError, match="quantized differently"):
        description_quant_type(d, "model.layers.0.mlp.gate_up_proj")
    assert detect_modelopt({"quantization": {"quant_algo": "MXFP8"}}) == "W8A8_MXFP8"
    assert detect_modelopt({"quant_algo": "FP8"}) == "W8A8FP8_DYNAMIC"
    with pytest.raises(ValueError):
        detect_modelopt({"quant_algo": "INT3"})
