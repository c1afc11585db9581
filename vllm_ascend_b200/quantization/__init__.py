"""Quantization: config detection, per-layer scheme selection, adapters.

Config formats (vllm_ascend/quantization/*_config.py): HF ``quantization_config`` with
``quant_method: fp8`` + ``weight_block_size`` (DeepSeek), ``compressed-tensors`` (static /
dynamic W8A8, W4A16), and a per-weight description file ``quant_model_description.json``
mapping ``"<prefix>.weight" -> "W8A8_DYNAMIC" | "FLOAT" | ...``
(vllm_ascend/quantization/modelslim_config.py:545-774).
"""
from __future__ import annotations

import json
import os
from typing import Optional

from . import schemes  # noqa: F401  (registers the schemes)
from .registry import get_scheme_class, register_scheme, registered  # noqa: F401

_ALIASES = {"fp8": "FP8_BLOCK", "fp8_block": "FP8_BLOCK", "w8a8_dynamic": "W8A8_DYNAMIC",
            "w8a8": "W8A8", "w8a8fp8_dynamic": "W8A8FP8_DYNAMIC", "w4a16": "W4A16",
            "w8a16": "W8A16", "float": "FLOAT", "ascend": "DESCRIPTION",
            "compressed-tensors": "COMPRESSED_TENSORS", "modelopt": "MODELOPT", "modelopt_mxfp8": "MODELOPT_MXFP8",
            "mxfp8": "MXFP8"}


class LinearMethod:
    """Adapter binding a linear scheme to one layer (method_adapters.py:34-292)."""

    def __init__(self, scheme):
        self.scheme = scheme
        # whether fused producers may hand this layer block-scaled fp8 activations
        self.accepts_quant_act = bool(getattr(scheme, "accepts_quant_act", False))

    def apply(self, layer, x, residual=None, skip_bias=False):
        return self.scheme.apply(layer, x, residual, skip_bias)

    def named_tensors(self, layer):
        return self.scheme.named_tensors(layer)


def detect_compressed_tensors(qc: dict) -> str:
    """Map a compressed-tensors config group to a scheme name
    (vllm_ascend/quantization/compressed_tensors_config.py:340-437)."""
    groups = qc.get("config_groups") or {}
    for g in groups.values():
        w, a = g.get("weights") or {}, g.get("input_activations")
        bits, typ = w.get("num_bits"), w.get("type", "int")
        if a is None:
            return "W4A16" if bits == 4 else "W8A16"
        if typ == "float" and bits == 8:
            if w.get("strategy") == "block":
                return "FP8_BLOCK"
            return "W8A8FP8_DYNAMIC"
        if bits == 8:
            return "W8A8_DYNAMIC" if a.get("dynamic") else "W8A8"
    raise ValueError("unsupported compressed-tensors configuration")


def load_description(model_path: Optional[str]) -> Optional[dict]:
    if not model_path:
        return None
    p = os.path.join(model_path, "quant_model_description.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f)
    return None


def detect_quantization(model_path: Optional[str], hf_config=None) -> Optional[str]:
    """Quantization method a checkpoint directory implies when the user named none: a per-weight
    description file selects ``ascend``; a ModelOpt export its own method; otherwise the
    ``quantization_config.quant_method`` of the HF config (the reference detects the description
    file the same way before the engine starts, vllm_ascend/quantization/utils.py
    maybe_auto_detect_quantization)."""
    if model_path and os.path.exists(os.path.join(model_path, "quant_model_description.json")):
        return "ascend"
    if model_path and os.path.exists(os.path.join(model_path, "hf_quant_config.json")):
        return "modelopt"
    qc = getattr(hf_config, "quantization_config", None) if hf_config is not None else None
    if isinstance(qc, dict) and qc.get("quant_method"):
        return str(qc["quant_method"])
    return None


#: fused modules of this package -> the checkpoint projections packed into them: a description file
#: names the checkpoint projections, and all parts of one fused GEMM must share a quant type
#: (vllm_ascend/quantization/modelslim_config.py:105-402 keeps this table per model type).
PACKED_MODULES = {
    "qkv_proj": ["q_proj", "k_proj", "v_proj"],
    "gate_up_proj": ["gate_proj", "up_proj"],
    "kv_a_proj": ["kv_a_proj_with_mqa"],
}


def description_quant_type(description: dict, prefix: str) -> str:
    """Quant type of a (possibly fused) linear layer from a per-weight description.  A fused layer
    takes the type of its parts and raises when they disagree
    (vllm_ascend/quantization/modelslim_config.py:431-470).  A part that the checkpoint does not
    have at all (v_proj of k == v attention) is skipped; a layer without any entry is FLOAT."""
    proj = prefix.rsplit(".", 1)[-1]
    direct = description.get(prefix + ".weight")
    if direct is not None:
        return str(direct).upper()
    parts = PACKED_MODULES.get(proj)
    if not parts:
        return "FLOAT"
    found: dict[str, str] = {}
    for part in parts:
        key = prefix[:-len(proj)] + part + ".weight"
        if key in description:
            found[part] = str(description[key]).upper()
    if not found:
        return "FLOAT"
    kinds = set(found.values())
    if len(kinds) > 1:
        raise ValueError(f"the parts of {prefix} are quantized differently ({found}): a fused GEMM needs "
                         "one quant type for all of them")
    return kinds.pop()


def detect_modelopt(qc: dict) -> str:
    """ModelOpt export (``quant_method: modelopt`` / ``hf_quant_config.json``): the algorithm name
    decides the scheme (vllm_ascend/quantization/modelopt_mxfp8_config.py:28-41 registers the MXFP8
    form)."""
    algo = str((qc.get("quantization") or qc).get("quant_algo", "")).upper()
    table = {"MXFP8": "W8A8_MXFP8", "FP8": "W8A8FP8_DYNAMIC", "FP8_PER_CHANNEL_PER_TOKEN": "W8A8FP8_DYNAMIC",
             "FP8_PB_WO": "FP8_BLOCK", "W4A16_AWQ": "W4A16", "NVFP4": "W4A4_MXFP4"}
    if algo not in table:
        raise ValueError(f"unsupported ModelOpt quant_algo {algo!r}; known: {sorted(table)}")
    return table[algo]


def resolve_quant_type(cfg, prefix: str, description: Optional[dict]) -> str:
    q = _ALIASES.get(str(cfg.quantization).lower(), str(cfg.quantization).upper())
    if q == "DESCRIPTION":
        if description is None:
            raise ValueError("--quantization ascend needs quant_model_description.json")
        return description_quant_type(description, prefix)
    qc = getattr(cfg, "quantization_config", None)
    if q in ("MODELOPT", "MODELOPT_MXFP8", "MXFP8"):
        return detect_modelopt(qc) if qc and q == "MODELOPT" else "W8A8_MXFP8"
    if q == "COMPRESSED_TENSORS":
        return detect_compressed_tensors(qc) if qc else "W8A8_DYNAMIC"
    return q


def _linears(model):
    for L in model.layers:
        p = f"model.layers.{L.idx}"
        a = L.self_attn
        for attr in ("qkv_proj", "o_proj", "q_a_proj", "q_b_proj", "q_proj", "kv_a_proj"):
            lin = getattr(a, attr, None)
            if lin is not None and hasattr(lin, "weight"):
                yield f"{p}.self_attn.{attr}", lin
        m = L.mlp
        for owner, pre in ((m, f"{p}.mlp"), (getattr(m, "shared", None), f"{p}.mlp.shared_experts")):
            if owner is None:
                continue
            for attr in ("gate_up_proj", "down_proj"):
                lin = getattr(owner, attr, None)
                if lin is not None:
                    yield f"{pre}.{attr}", lin


def apply_quantization(model, cfg) -> dict[str, str]:
    """Attach quantization methods to every linear / MoE block; returns {prefix: quant type}."""
    description = load_description(cfg.model_path)
    chosen: dict[str, str] = {}
    for prefix, lin in _linears(model):
        qt = resolve_quant_type(cfg, prefix, description)
        chosen[prefix] = qt
        if qt == "FLOAT":
            continue
        scheme = get_scheme_class(qt, "linear")()
        scheme.convert(lin)
        lin.quant = LinearMethod(scheme)
    for L in model.layers:
        m = L.mlp
        if hasattr(m, "w13"):
            prefix = f"model.layers.{L.idx}.mlp.experts"
            qt = resolve_quant_type(cfg, prefix, description)
            chosen[prefix] = qt
            if qt != "FLOAT":
                scheme = get_scheme_class(qt, "moe")()
                scheme.convert(m)
                m.quant = scheme
    return chosen
