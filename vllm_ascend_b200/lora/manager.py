"""Adapter registry and per-layer stacked LoRA weights.

``LoRAManager`` keeps up to ``max_loras`` adapters resident in slots of pre-allocated stacked
tensors (one pair per target linear), loads PEFT-format checkpoints, evicts the least
recently used unpinned adapter, and tells the runner each request's slot.  The worker
passthroughs add/remove/list/pin (vllm_ascend/worker/worker.py:1033-1043) land here.
"""
from __future__ import annotations

import json
import os
import re
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Optional

import torch

from .punica import PunicaWrapperB200

# HF sub-module -> (merged layer attribute, slice index)
_TARGETS = {"q_proj": ("qkv_proj", 0), "k_proj": ("qkv_proj", 1), "v_proj": ("qkv_proj", 2),
            "o_proj": ("o_proj", 0), "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1),
            "down_proj": ("down_proj", 0)}


@dataclass
class LoRARequest:
    lora_name: str
    lora_int_id: int
    lora_path: Optional[str] = None
    tensors: Optional[dict] = None          # in-memory adapter {peft name: tensor}
    rank: Optional[int] = None
    alpha: Optional[float] = None


@dataclass
class LoRALayerState:
    """Stacked adapter weights of one (possibly merged) linear layer."""
    a: torch.Tensor                      # [slots, slices*r_max, K_local]
    b: list                              # per slice [slots, N_slice_local, r_max]
    output_slices: list
    rank: int
    punica: PunicaWrapperB200
    scale: float = 1.0                   # per-slot scaling is folded into B at load time
    shard: dict = field(default_factory=dict)

    def apply(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        return self.punica.add_lora_linear(y, x, self.a, self.b, self.scale, self.output_slices, self.rank)


class LoRAManager:
    def __init__(self, model, max_loras: int, max_rank: int, max_tokens: int, max_seqs: int, device, dtype):
        self.model = model
        self.max_loras, self.max_rank = max_loras, (max_rank + 7) // 8 * 8
        self.device, self.dtype = device, dtype
        self.punica = PunicaWrapperB200(max_tokens, max_seqs, device, max_loras)
        self.slots: "OrderedDict[int, int]" = OrderedDict()       # lora id -> slot, LRU order
        self.pinned: set[int] = set()
        self.free_slots = list(range(max_loras))
        self.layers: dict[tuple[int, str], LoRALayerState] = {}
        self.moe_layers: dict[int, object] = {}          # layer index -> lora.moe.MoELoRAState
        self._attach()

    def _attach(self) -> None:
        r = self.max_rank
        for L in self.model.layers:
            mods = {"qkv_proj": getattr(L.self_attn, "qkv_proj", None), "o_proj": getattr(L.self_attn, "o_proj", None)}
            mlp = getattr(L, "mlp", None)
            if mlp is not None and hasattr(mlp, "gate_up_proj"):
                mods["gate_up_proj"], mods["down_proj"] = mlp.gate_up_proj, mlp.down_proj
            if mlp is not None and hasattr(mlp, "w13") and self._experts_supported(mlp):
                from .moe import MoELoRAState
                E, two_i, H = mlp.w13.shape
                Il = two_i // 2
                z = lambda *shape: torch.zeros(shape, dtype=self.dtype, device=self.device)     # noqa: E731
                n = self.max_loras * E
                ep = getattr(mlp, "ep", None) is not None
                emap = mlp.expert_map.tolist() if ep and getattr(mlp, "expert_map", None) is not None else None
                mlp.lora = MoELoRAState(z(n, 2 * r, H), z(n, Il, r), z(n, Il, r), z(n, r, Il), z(n, H, r), E, r,
                                        self.punica, expert_map=emap, sharded=not ep)
                self.moe_layers[L.idx] = mlp.lora
            for name, lin in mods.items():
                if lin is None or getattr(lin, "weight", None) is None:
                    continue
                n_local, k_local = lin.weight.shape
                slices = list(getattr(lin, "local_sizes", [n_local]))
                st = LoRALayerState(
                    a=torch.zeros((self.max_loras, len(slices) * r, k_local), dtype=self.dtype, device=self.device),
                    b=[torch.zeros((self.max_loras, n, r), dtype=self.dtype, device=self.device) for n in slices],
                    output_slices=slices, rank=r, punica=self.punica)
                lin.lora = st
                self.layers[(L.idx, name)] = st

    @staticmethod
    def _experts_supported(mlp) -> bool:
        """Expert adapters under expert parallelism need every EP rank to see the same batch (the
        slot vector travels with the tokens and all ranks must agree on the path): engines without
        data parallelism and without redundant expert replicas."""
        if getattr(mlp, "ep", None) is None:
            return True
        from ..parallel import state as pstate
        return pstate.get_dp_group().world_size == 1 and getattr(mlp, "log2phy", None) is None

    # ------------------------------------------------------------------ registry
    def list(self) -> set:
        return set(self.slots)

    def pin(self, lora_id: int) -> bool:
        if lora_id not in self.slots:
            return False
        self.pinned.add(lora_id)
        return True

    def remove(self, lora_id: int) -> bool:
        slot = self.slots.pop(lora_id, None)
        if slot is None:
            return False
        self.pinned.discard(lora_id)
        self._zero_slot(slot)
        self.free_slots.append(slot)
        return True

    def slot_of(self, lora_id: Optional[int]) -> int:
        if lora_id is None or lora_id not in self.slots:
            return -1
        self.slots.move_to_end(lora_id)
        return self.slots[lora_id]

    def can_activate(self, lora_id: Optional[int], in_use: set) -> bool:
        """True when the adapter is resident, or a slot can be found without evicting an
        adapter that a scheduled request (``in_use``) or a pin holds."""
        if lora_id is None or lora_id in self.slots or self.free_slots:
            return True
        return any(i not in in_use and i not in self.pinned for i in self.slots)

    def add(self, req: LoRARequest, in_use: Optional[set] = None) -> bool:
        if req.lora_int_id in self.slots:
            self.slots.move_to_end(req.lora_int_id)
            return True
        if not self.free_slots:
            victim = next((i for i in self.slots if i not in (in_use or set()) and i not in self.pinned), None)
            if victim is None:
                return False
            self.remove(victim)
        tensors, rank, alpha = self._read(req)
        if rank > self.max_rank:
            raise ValueError(f"adapter rank {rank} exceeds max_lora_rank {self.max_rank}")
        slot = self.free_slots.pop(0)
        self._zero_slot(slot)
        self._fill(slot, tensors, rank, alpha / rank)
        self.slots[req.lora_int_id] = slot
        return True

    # ------------------------------------------------------------------ loading
    @staticmethod
    def _read(req: LoRARequest):
        if req.tensors is not None:
            t = req.tensors
            rank = req.rank or next(v.shape[0] for k, v in t.items() if "lora_A" in k)
            return t, rank, float(req.alpha if req.alpha is not None else rank)
        with open(os.path.join(req.lora_path, "adapter_config.json")) as f:
            cfg = json.load(f)
        path = os.path.join(req.lora_path, "adapter_model.safetensors")
        from safetensors.torch import load_file
        return load_file(path), int(cfg["r"]), float(cfg.get("lora_alpha", cfg["r"]))

    @property
    def graph_safe(self) -> bool:
        """Adapter steps of models with expert adapters take a path with host-side routing reads."""
        return not self.moe_layers

    def _zero_slot(self, slot: int) -> None:
        for ms in self.moe_layers.values():
            ms.zero_slot(slot)
        for st in self.layers.values():
            st.a[slot].zero_()
            for b in st.b:
                b[slot].zero_()

    def _fill(self, slot: int, tensors: dict, rank: int, scaling: float) -> None:
        comm = self.model.comm
        tp, tr = comm.size, comm.rank
        for name, w in tensors.items():
            me = re.search(r"layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.lora_([AB])(?:\.default)?\.weight",
                           name)
            if me:
                ms = self.moe_layers.get(int(me.group(1)))
                if ms is None:
                    continue
                e, proj, which = int(me.group(2)), me.group(3), me.group(4)
                if ms.expert_map is not None:
                    e = ms.expert_map[e] if e < len(ms.expert_map) else -1
                    if e < 0:
                        continue                       # another rank's expert
                row = slot * ms.num_experts + e
                w = w.to(self.device, self.dtype)
                Il = ms.b_gate.shape[1]
                tr = comm.rank if ms.sharded else 0
                if proj in ("gate_proj", "up_proj"):
                    off = 0 if proj == "gate_proj" else ms.rank
                    if which == "A":                   # [r, H]
                        ms.a13[row, off:off + rank] = w
                    else:                              # [I, r] rows sharded like the expert's weight
                        dst = ms.b_gate if proj == "gate_proj" else ms.b_up
                        dst[row, :, :rank] = (w[tr * Il:(tr + 1) * Il].float() * scaling).to(self.dtype)
                elif which == "A":                     # down: [r, I] columns sharded
                    ms.a2[row, :rank] = w[:, tr * Il:(tr + 1) * Il]
                else:                                  # [H, r]
                    ms.b2[row, :, :rank] = (w.float() * scaling).to(self.dtype)
                continue
            m = re.search(r"layers\.(\d+)\.(?:self_attn|mlp)\.(\w+)\.lora_([AB])(?:\.default)?\.weight", name)
            if not m or m.group(2) not in _TARGETS:
                continue
            li, (target, si), which = int(m.group(1)), _TARGETS[m.group(2)], m.group(3)
            st = self.layers.get((li, target))
            if st is None:
                continue
            row_parallel = target in ("o_proj", "down_proj")
            w = w.to(self.device, self.dtype)
            if which == "A":                       # [r, K]
                if row_parallel and tp > 1:        # input dim is sharded
                    k = w.shape[1] // tp
                    w = w[:, tr * k:(tr + 1) * k]
                st.a[slot, si * st.rank: si * st.rank + rank, :w.shape[1]] = w
            else:                                  # [N, r], scaling folded in
                if not row_parallel and tp > 1:    # output dim is sharded
                    n = w.shape[0] // tp
                    w = w[tr * n:(tr + 1) * n]
                st.b[si][slot, :w.shape[0], :rank] = (w.float() * scaling).to(self.dtype)
