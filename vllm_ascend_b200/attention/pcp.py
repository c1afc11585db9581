"""Prefill context parallelism: the query tokens of a prefill chunk are split over the ranks of the
PCP group, every rank runs the dense layers on its share only, and K / V of all shares are
all-gathered into every rank's paged cache before attention.

Causal attention costs grow with the query position, so a chunk is cut into 2P pieces and rank r
takes pieces r and 2P-1-r (one cheap, one expensive).  A rank's two pieces become two entries of
the attention batch that share the request's block table; entry (a, b) holds queries [a, b) and
attends to keys [0, b).  Sequences shorter than 2P tokens (decodes included) are replicated on
all ranks.  The last token of every chunk lands on rank 0, which samples and broadcasts.
Decode steps run replicated: after the all-gather every rank holds the full KV.

Role of the reference's prefill-context-parallel path (worker/v2/pcp_manager.py:30-99
partition_batch; attention/attention_v1.py:1744-1785 AscendAttentionPCPImpl, which all-gathers
KV over the PCP group before attention).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch


def split_ranges(start: int, length: int, P: int, rank: int) -> list[tuple[int, int]]:
    """Absolute [a, b) ranges of the chunk [start, start + length) that ``rank`` computes."""
    if length < 2 * P:
        return [(start, start + length)]
    # piece i = [i * length / 2P, (i + 1) * length / 2P): never empty, so the chunk's last token is
    # always in piece 2P-1, i.e. on rank 0
    out = []
    for i in (rank, 2 * P - 1 - rank):
        out.append((start + i * length // (2 * P), start + (i + 1) * length // (2 * P)))
    return out


@dataclass
class PCPPlan:
    local_idx: list          # per rank: int64 indices into the step's global token order
    entries: list            # per rank: list of (request index, a, b)
    t_max: int

    @property
    def is_split(self) -> bool:
        return len(self.local_idx) > 1


def build_plan(starts: np.ndarray, q_lens: np.ndarray, cu: np.ndarray, P: int) -> PCPPlan:
    local_idx, entries = [], []
    for r in range(P):
        idx, ent = [], []
        for i, (s, n) in enumerate(zip(starts.tolist(), q_lens.tolist())):
            for a, b in split_ranges(s, n, P, r):
                ent.append((i, a, b))
                idx.append(np.arange(cu[i] + a - s, cu[i] + b - s, dtype=np.int64))
        local_idx.append(np.concatenate(idx) if idx else np.zeros(0, dtype=np.int64))
        entries.append(ent)
    return PCPPlan(local_idx, entries, max(len(x) for x in local_idx))


@dataclass
class PCPMeta:
    group: object                 # GroupCoordinator of the PCP ranks
    t_max: int                    # rows every rank contributes to the gather (padded)
    gather_slots: torch.Tensor    # int64 [P * t_max] cache slot of every gathered row (-1: padding)


def gather_kv_into_cache(kv: torch.Tensor, pm: PCPMeta, k_cache, v_cache, Hkv: int, D: int, eps: float,
                         cos_sin: torch.Tensor) -> None:
    """kv: [T_local, 2 * Hkv * D] (K already rotated).  All-gathers the rows of every rank and
    scatters them into the paged caches."""
    from .. import ops
    T = kv.shape[0]
    if T < pm.t_max:
        pad = kv.new_zeros((pm.t_max, kv.shape[1]))
        pad[:T] = kv
        kv = pad
    allkv = pm.group.all_gather(kv.contiguous(), dim=0)
    ops.qknorm_rope_kvwrite(allkv, pm.gather_slots, cos_sin, 0, None, None, eps, k_cache, v_cache,
                            pm.gather_slots, 0, Hkv, D)
