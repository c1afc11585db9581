"""Multimodal inputs: image / video patches, placeholder expansion, 3-axis rotary positions."""
from .inputs import MMInput, build_mm_request, expand_placeholders, mm_hash
from .mrope import mrope_positions
from .processor import patchify, smart_resize

__all__ = ["MMInput", "build_mm_request", "expand_placeholders", "mm_hash", "mrope_positions", "patchify",
           "smart_resize"]
