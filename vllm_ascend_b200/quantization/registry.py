"""Scheme registry: ``(quant_type, layer_type) -> scheme class``.

Same split as the reference (vllm_ascend/quantization/methods/registry.py:21-62 and
methods/base.py:62-287): a *scheme* knows how to create/convert the weights of one
layer kind and how to apply them; thin *adapters* (``LinearMethod``, ``MoEMethod``)
bind a scheme to a layer object.
"""
from __future__ import annotations

from typing import Callable

_SCHEMES: dict[tuple[str, str], type] = {}


def register_scheme(quant_type: str, layer_type: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        key = (quant_type.upper(), layer_type)
        if key in _SCHEMES:
            raise ValueError(f"scheme {key} registered twice")
        _SCHEMES[key] = cls
        cls.quant_type = quant_type.upper()
        cls.layer_type = layer_type
        return cls
    return deco


def get_scheme_class(quant_type: str, layer_type: str) -> type:
    try:
        return _SCHEMES[(quant_type.upper(), layer_type)]
    except KeyError:
        known = sorted(k for k in _SCHEMES if k[1] == layer_type)
        raise ValueError(f"no {layer_type} scheme for quant type {quant_type!r}; known: {known}") from None


def registered() -> list[tuple[str, str]]:
    return sorted(_SCHEMES)
