"""Expert placement bookkeeping: physical slots, logical→physical tables, JSON I/O, and the
weight moves that turn one placement into another.

A placement is an int array ``[layers, ranks, slots_per_rank]`` of logical expert ids;
physical slot ``(r, s)`` has id ``r * slots_per_rank + s``.  File format and table
generation follow vllm_ascend/eplb/core/eplb_utils.py:27-145 (static map from JSON,
``log2phy`` construction); the per-rank send/recv lists follow
eplb/core/eplb_device_transfer_loader.py:46-138.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

import numpy as np


def initial_placement(num_layers: int, num_experts: int, num_ranks: int, num_redundant: int = 0) -> np.ndarray:
    if num_experts % num_ranks or num_redundant % num_ranks:
        raise ValueError("experts and redundant experts must divide evenly over the ranks")
    base, extra = num_experts // num_ranks, num_redundant // num_ranks
    if extra > num_experts - base:
        raise ValueError("too many redundant experts")
    rows = []
    for r in range(num_ranks):
        own = list(range(r * base, (r + 1) * base))
        # redundant slots start as copies of the next ranks' experts
        red = [((r + 1) * base + j) % num_experts for j in range(extra)]
        rows.append(own + red)
    one = np.array(rows, dtype=np.int32)
    return np.broadcast_to(one, (num_layers,) + one.shape).copy()


def validate(placement: np.ndarray, num_experts: int) -> None:
    for l in range(placement.shape[0]):
        present = np.unique(placement[l])
        if present.min() < 0 or present.max() >= num_experts or len(present) != num_experts:
            raise ValueError(f"layer {l}: placement does not hold every expert exactly or more than once")


def build_log2phy(placement_layer: np.ndarray, num_experts: int, prefer_rank: int = -1):
    """(table [E, max_replicas] of physical slot ids padded with -1, counts [E]).  Replicas on
    ``prefer_rank`` come first so a rank routes to its own copy when it has one."""
    R, S = placement_layer.shape
    lists: list[list[int]] = [[] for _ in range(num_experts)]
    for r in range(R):
        for s in range(S):
            lists[int(placement_layer[r, s])].append(r * S + s)
    if prefer_rank >= 0:
        for l in lists:
            l.sort(key=lambda p: (p // S != prefer_rank, p))
    width = max(len(l) for l in lists)
    table = np.full((num_experts, width), -1, dtype=np.int32)
    for e, l in enumerate(lists):
        table[e, :len(l)] = l
    return table, np.array([len(l) for l in lists], dtype=np.int32)


@dataclass
class Move:
    expert: int
    src_rank: int
    src_slot: int
    dst_rank: int
    dst_slot: int


def plan_moves(old: np.ndarray, new: np.ndarray) -> list[Move]:
    """Weight copies that realise ``new`` from ``old`` for one layer: every slot whose expert
    changes pulls it from a slot that holds it in ``old`` (same rank if possible, else the
    holder with the fewest outgoing copies so far)."""
    R, S = old.shape
    holders: dict[int, list[tuple[int, int]]] = {}
    for r in range(R):
        for s in range(S):
            holders.setdefault(int(old[r, s]), []).append((r, s))
    out_count = np.zeros(R, dtype=np.int64)
    moves = []
    for r in range(R):
        for s in range(S):
            e = int(new[r, s])
            if e == int(old[r, s]):
                continue
            cands = holders[e]
            local = [c for c in cands if c[0] == r]
            src = local[0] if local else min(cands, key=lambda c: (out_count[c[0]], c))
            if src[0] != r:
                out_count[src[0]] += 1
            moves.append(Move(e, src[0], src[1], r, s))
    return moves


def save_placement(path: str, placement: np.ndarray) -> None:
    L, R, S = placement.shape
    doc = {"moe_layer_count": L, "layer_list": [
        {"layer_id": l, "device_count": R, "device_list": [
            {"device_id": r, "device_expert": [int(x) for x in placement[l, r]]} for r in range(R)]}
        for l in range(L)]}
    with open(path, "w") as f:
        json.dump(doc, f)


def load_placement(path: str) -> np.ndarray:
    with open(path) as f:
        doc = json.load(f)
    layers = sorted(doc["layer_list"], key=lambda x: x["layer_id"])
    return np.array([[d["device_expert"] for d in sorted(l["device_list"], key=lambda x: x["device_id"])]
                     for l in layers], dtype=np.int32)
