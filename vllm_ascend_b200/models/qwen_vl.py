"""Qwen2.5-VL style conditional-generation model: the decoder of ``CausalLM`` with multimodal
rotary positions plus a vision tower whose outputs replace the placeholder-token embeddings.

The reference serves the same family through upstream model code with its own ViT attention,
rotary and Conv3d ops patched in (vllm_ascend/ops/mm_encoder_attention.py,
patch/worker/patch_qwen3_vl*.py); here model, tower and merge are native.
"""
from __future__ import annotations

import re
from typing import Iterable

import torch

from .transformer import CausalLM
from .vision import VisionConfig, VisionTransformer


class QwenVLForConditionalGeneration(CausalLM):
    is_multimodal = True

    def __init__(self, cfg, device, **kw):
        super().__init__(cfg, device, **kw)
        self.vision_cfg = VisionConfig.from_hf(cfg.vision_config or {})
        if self.vision_cfg.out_hidden_size != cfg.hidden_size:
            raise ValueError("vision tower output width must equal the decoder's hidden size")
        self.num_deepstack = len(self.vision_cfg.deepstack_visual_indexes)
        if not self.is_first:
            self.visual = None
        elif self.vision_cfg.num_position_embeddings:
            from .vision import Qwen3VisionTransformer
            self.visual = Qwen3VisionTransformer(self.vision_cfg, self.device, self.dtype)
        else:
            self.visual = VisionTransformer(self.vision_cfg, self.device, self.dtype)

    # -- multimodal interface ------------------------------------------------
    def embed_multimodal(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        """pixel_values [sum patches, patch_dim], grid_thw [n, 3] -> [sum patches / merge^2, hidden]."""
        return self.visual(pixel_values, grid_thw)

    def embed_input_ids(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.embed_tokens(input_ids)

    # -- parameters --------------------------------------------------------------
    def named_parameters(self):
        yield from super().named_parameters()
        if self.visual is not None:
            for n, t in self.visual.named_parameters():
                yield f"visual.{n}", t

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        lm, vis, names = [], [], {}
        for name, w in weights:
            m = re.match(r"(?:model\.)?visual\.(.*)", name)
            if m:
                vis.append((m.group(1), w))
                names[m.group(1)] = name
                continue
            new = re.sub(r"^model\.language_model\.", "model.", name)
            new = re.sub(r"^language_model\.", "", new)
            names[new] = name
            lm.append((new, w))
        loaded = {names[n] for n in super().load_weights(lm)}
        if self.visual is not None:
            loaded |= {names[n] for n in self.visual.load_weights(vis)}
        return loaded
