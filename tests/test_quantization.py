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
                ("FP8_BLOCK", "moe"), ("W8A8_DYNAMIC", "moe")]:
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
                                      ("W8A8FP8_DYNAMIC", 0.08), ("W8A16", 0.02), ("W4A16", 0.25)])
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
