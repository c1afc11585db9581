"""Speculative-decoding proposers and their factory (vllm_ascend/spec_decode/__init__.py:33-58)."""
from __future__ import annotations


def get_spec_decode_method(spec_cfg: dict, runner):
    method = (spec_cfg or {}).get("method", "ngram")
    k = int(spec_cfg.get("num_speculative_tokens", 3))
    if method == "ngram":
        from .ngram import NgramProposer
        return NgramProposer(k, int(spec_cfg.get("prompt_lookup_min", 2)), int(spec_cfg.get("prompt_lookup_max", 5)),
                             runner.max_model_len)
    if method == "suffix":
        from .suffix import SuffixProposer
        return SuffixProposer(k, int(spec_cfg.get("suffix_max_depth", 24)), runner.max_model_len)
    if method in ("draft_model", "eagle", "eagle3", "mtp"):
        from .draft_model import DraftModelProposer
        return DraftModelProposer(method, k, spec_cfg, runner)
    if method == "medusa":
        from .medusa import MedusaProposer
        return MedusaProposer(k, spec_cfg, runner)
    if method == "extract_hidden_states":
        from .extract_hidden import ExtractHiddenStatesProposer
        return ExtractHiddenStatesProposer(spec_cfg, runner)
    raise ValueError(f"unknown speculative method {method!r}")
