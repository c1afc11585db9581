"""Running a tensor-parallel linear layer with its FULL weight for a while.

A TP-sharded layer normally sees a shard of the hidden dimension on every rank.  Some step kinds
shard the *tokens* instead (context-parallel prefill of sparse / compressed attention: every rank
holds other tokens and needs the whole projection), so the layer temporarily needs the complete
weight: the shards of all ranks are all-gathered into pooled buffers, the layer's tensors are
swapped for the gathered ones, and swapped back afterwards.  The gather is asynchronous so that it
can be started a layer ahead and overlap compute.

Behaviour of ``TPWeightSwitchMixin`` (vllm_ascend/quantization/tp_weight_switch.py:26-296): per
scheme a declaration of which layer tensors are sharded along which dimension (gathered) and which
are per-rank constants the full-weight kernel wants once per shard (repeated); row-parallel layers
are input-sharded, column-parallel layers output-sharded; buffers come from a shared pool keyed by
shape so that layers of equal geometry reuse one full-size buffer.

The declarations for this package's schemes live in ``SWITCH_SPECS``: a scheme that is not listed
does not support switching (``supports()`` is the opt-in gate callers check).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class GatherSpec:
    """Layer tensor that is sharded over TP along ``dim`` (after weight post-processing)."""
    attr: str
    dim: int = 0


@dataclass(frozen=True)
class RepeatSpec:
    """Layer tensor that every rank holds identically and the full-weight form wants once per
    shard along ``dim``."""
    attr: str
    dim: int = 0


#: scheme name -> {"input": (specs for row-parallel layers), "output": (specs for column-parallel)}
#: Weights are [N, K]: input-sharded layers are cut along K (dim 1), output-sharded along N (dim 0).
#: Block-scaled fp8 carries one scale per 128 x 128 block, sharded like the weight.
SWITCH_SPECS: dict[str, dict[str, tuple]] = {
    "FLOAT": {"input": (GatherSpec("weight", 1),), "output": (GatherSpec("weight", 0), GatherSpec("bias", 0))},
    "FP8_BLOCK": {"input": (GatherSpec("weight", 1), GatherSpec("weight_scale_inv", 1)),
                  "output": (GatherSpec("weight", 0), GatherSpec("weight_scale_inv", 0), GatherSpec("bias", 0))},
}


def scheme_name(layer) -> str:
    q = getattr(layer, "quant", None)
    if q is None:
        return "FLOAT"
    return getattr(q, "scheme_name", None) or getattr(type(q), "scheme_name", None) or type(q).__name__


def supports(layer) -> bool:
    name = scheme_name(layer)
    if name == "Fp8BlockLinear":
        name = "FP8_BLOCK"
    return name in SWITCH_SPECS


@dataclass
class _Part:
    spec: Any
    tp_tensor: torch.Tensor            # this rank's shard (what the layer holds in TP mode)
    gather_in: Optional[torch.Tensor]  # shard with the gather dim moved to the front
    gather_out: Optional[torch.Tensor]  # pooled buffer [tp * shard_dim, ...]
    full_tensor: torch.Tensor          # view of gather_out in the layer's own layout


@dataclass
class SwitchState:
    axis: str
    parts: dict = field(default_factory=dict)
    handles: list = field(default_factory=list)
    mode: str = "tp"                   # "tp" | "full"
    gathered: bool = False


class TPWeightSwitch:
    """Per-layer controller.  ``group``: a ``GroupCoordinator`` (or anything with ``world_size``,
    ``rank_in_group`` and ``device_group``)."""

    def __init__(self, layer, group, axis: str, pool: Optional[dict] = None, pool_key: Any = None):
        if axis not in ("input", "output"):
            raise ValueError("axis must be 'input' (row-parallel) or 'output' (column-parallel)")
        if not supports(layer):
            raise RuntimeError(f"scheme {scheme_name(layer)} does not support TP weight switching")
        name = scheme_name(layer)
        specs = SWITCH_SPECS["FP8_BLOCK" if name == "Fp8BlockLinear" else name][axis]
        self.layer, self.group = layer, group
        self.tp = group.world_size
        self.state = SwitchState(axis=axis)
        pool = pool if pool is not None else {}
        for spec in specs:
            t = getattr(layer, spec.attr, None)
            if t is None:
                if spec.attr == "bias":
                    continue
                raise RuntimeError(f"layer {getattr(layer, 'name', layer)} has no tensor {spec.attr!r}")
            dim = spec.dim if spec.dim >= 0 else t.dim() + spec.dim
            if not 0 <= dim < t.dim():
                raise RuntimeError(f"bad dim {spec.dim} for {spec.attr!r} of shape {tuple(t.shape)}")
            if isinstance(spec, RepeatSpec):
                full = t.repeat_interleave(self.tp, dim=dim) if self.tp > 1 else t
                self.state.parts[spec.attr] = _Part(spec, t, None, None, full)
                continue
            full_shape = list(t.shape)
            full_shape[dim] *= self.tp
            gshape = (full_shape[dim], *full_shape[:dim], *full_shape[dim + 1:])
            key = (pool_key, spec.attr, t.device.type, t.device.index, t.dtype, dim, tuple(full_shape))
            out = pool.get(key)
            if out is None:
                out = torch.empty(gshape, dtype=t.dtype, device=t.device)
                pool[key] = out
            gin = t if dim == 0 else torch.movedim(t, dim, 0).contiguous()
            full = out if dim == 0 else torch.movedim(out, 0, dim)
            self.state.parts[spec.attr] = _Part(spec, t, gin.contiguous(), out, full)

    # ------------------------------------------------------------------
    def start_gather(self) -> None:
        """Launch the all-gathers (asynchronously when the backend allows)."""
        st = self.state
        st.handles.clear()
        for part in st.parts.values():
            if part.gather_out is None:
                continue
            if self.tp == 1:
                part.gather_out.copy_(part.gather_in)
                continue
            inp, out = part.gather_in, part.gather_out
            # collectives move bytes: 8-bit float tensors travel as uint8
            if inp.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
                inp, out = inp.view(torch.uint8), out.view(torch.uint8)
            st.handles.append(dist.all_gather_into_tensor(out, inp, group=self.group.device_group, async_op=True))
        st.gathered = True

    def wait(self) -> None:
        for h in self.state.handles:
            h.wait()
        self.state.handles.clear()

    def use_full(self) -> None:
        """Point the layer at the gathered tensors (gathers them first if nobody started that)."""
        st = self.state
        if not st.gathered:
            self.start_gather()
        self.wait()
        for attr, part in st.parts.items():
            setattr(self.layer, attr, part.full_tensor)
        st.mode = "full"

    def use_tp(self) -> None:
        st = self.state
        for attr, part in st.parts.items():
            setattr(self.layer, attr, part.tp_tensor)
        st.mode = "tp"
        st.gathered = False          # the pooled buffers may serve another layer now

    def full(self):
        """Context manager: full weights inside, shards afterwards."""
        sw = self

        class _Ctx:
            def __enter__(self):
                sw.use_full()
                return sw.layer

            def __exit__(self, *a):
                sw.use_tp()
                return False
        return _Ctx()


def split_for_tp(t: torch.Tensor, tp: int, rank: int, dim: int = 0) -> torch.Tensor:
    """One rank's shard of a full tensor (the inverse of the gather)."""
    dim = dim if dim >= 0 else t.dim() + dim
    if t.shape[dim] % tp:
        raise RuntimeError(f"dimension {dim} of {tuple(t.shape)} is not divisible by {tp}")
    n = t.shape[dim] // tp
    return t.narrow(dim, rank * n, n).contiguous()
