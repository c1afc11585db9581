"""Expert-placement policies for dynamic expert-parallel load balancing.

Input: current placement ``[layers, ranks, slots_per_rank]`` of logical expert ids and the
measured load per logical expert ``[layers, num_experts]``.  Output: a new placement of the
same shape.  Policies (numbering of vllm_ascend/eplb/core/policy/policy_factory.py:12-41):

  0  random          shuffle (baseline / tests)
  1  greedy          replicate the hottest experts into the redundant slots, then pack
                     replicas onto ranks heaviest-first into the lightest rank
                     (policy_default_eplb.py:125-236, 283-350)
  2  swift           keep the current placement and apply at most ``max_swaps`` pairwise
                     swaps between the heaviest and lightest rank, so little weight moves
                     (policy_swift_balancer.py:510-751)
  3  flash           per layer, re-plan only when the imbalance exceeds a threshold or moved
                     by more than a fluctuation margin since the last plan (policy_flashlb.py)
"""
from __future__ import annotations

from typing import Optional

import numpy as np


def rank_loads(placement: np.ndarray, load: np.ndarray) -> np.ndarray:
    """[ranks] load of one layer: an expert's load is split evenly over its replicas."""
    E = load.shape[0]
    replicas = np.bincount(placement.reshape(-1), minlength=E).astype(np.float64)
    per_replica = load / np.maximum(replicas, 1)
    return per_replica[placement].sum(axis=1)


def imbalance(placement: np.ndarray, load: np.ndarray) -> float:
    """max rank load / mean rank load (1.0 = perfect)."""
    rl = rank_loads(placement, load)
    m = rl.mean()
    return float(rl.max() / m) if m > 0 else 1.0


class EplbPolicy:
    def rebalance(self, placement: np.ndarray, load: np.ndarray) -> np.ndarray:
        """placement [L, R, S] int, load [L, E] -> new placement [L, R, S]."""
        return np.stack([self.rebalance_layer(placement[l], load[l], l) for l in range(placement.shape[0])])

    def rebalance_layer(self, placement: np.ndarray, load: np.ndarray, layer: int = 0) -> np.ndarray:
        raise NotImplementedError


class RandomPolicy(EplbPolicy):
    def __init__(self, seed: int = 0):
        self.rng = np.random.default_rng(seed)

    def rebalance_layer(self, placement, load, layer=0):
        R, S = placement.shape
        flat = placement.reshape(-1).copy()
        for _ in range(64):                       # a rank must not hold two replicas of one expert
            self.rng.shuffle(flat)
            cand = flat.reshape(R, S)
            if all(len(set(row)) == S for row in cand):
                return cand.copy()
        return placement.copy()


class GreedyPolicy(EplbPolicy):
    def rebalance_layer(self, placement, load, layer=0):
        R, S = placement.shape
        E = load.shape[0]
        slots = R * S
        if slots < E:
            raise ValueError("fewer expert slots than experts")
        # 1. replica counts: give each redundant slot to the expert with the largest load per replica
        replicas = np.ones(E, dtype=np.int64)
        for _ in range(slots - E):
            per = load / replicas
            per[replicas >= R] = -1                 # at most one replica per rank
            replicas[int(per.argmax())] += 1
        # 2. pack replicas heaviest-first onto the lightest rank that has room and no copy yet
        items = sorted(((load[e] / replicas[e], e) for e in range(E) for _ in range(replicas[e])),
                       key=lambda x: (-x[0], x[1]))
        rank_load = np.zeros(R)
        rows: list[list[int]] = [[] for _ in range(R)]
        for w, e in items:
            order = np.argsort(rank_load, kind="stable")
            for r in order:
                if len(rows[r]) < S and e not in rows[r]:
                    rows[r].append(e)
                    rank_load[r] += w
                    break
            else:                                   # only full ranks or ranks holding e are left
                r = next(r for r in order if len(rows[r]) < S)
                rows[r].append(e)
                rank_load[r] += w
        return np.array([sorted(row) for row in rows], dtype=placement.dtype)


class SwiftPolicy(EplbPolicy):
    def __init__(self, max_swaps: int = 4, min_gain: float = 0.01):
        self.max_swaps, self.min_gain = max_swaps, min_gain

    def rebalance_layer(self, placement, load, layer=0):
        p = placement.copy()
        E = load.shape[0]
        for _ in range(self.max_swaps):
            replicas = np.bincount(p.reshape(-1), minlength=E).astype(np.float64)
            w = load / np.maximum(replicas, 1)
            rl = w[p].sum(axis=1)
            hi, lo = int(rl.argmax()), int(rl.argmin())
            gap = rl[hi] - rl[lo]
            if hi == lo or gap <= 0:
                break
            # swap (a in hi, b in lo) that brings the two ranks closest together
            best, best_pair = gap, None
            for ia, a in enumerate(p[hi]):
                for ib, b in enumerate(p[lo]):
                    if a == b or a in p[lo] or b in p[hi]:
                        continue
                    d = w[a] - w[b]
                    new_gap = abs(gap - 2 * d)
                    if new_gap < best:
                        best, best_pair = new_gap, (ia, ib)
            if best_pair is None or (gap - best) < self.min_gain * max(rl.mean(), 1e-9):
                break
            ia, ib = best_pair
            p[hi, ia], p[lo, ib] = p[lo, ib], p[hi, ia]
        return p


class FlashPolicy(EplbPolicy):
    """Greedy re-plan gated per layer: skip layers that are balanced enough or whose imbalance
    did not move since the last plan; limit how many layers change per call."""

    def __init__(self, threshold: float = 1.15, fluctuation: float = 0.05, max_layers_per_call: Optional[int] = None):
        self.threshold, self.fluctuation = threshold, fluctuation
        self.max_layers = max_layers_per_call
        self.inner = GreedyPolicy()
        self.last: dict[int, float] = {}

    def rebalance(self, placement, load):
        L = placement.shape[0]
        imb = np.array([imbalance(placement[l], load[l]) for l in range(L)])
        todo = [l for l in np.argsort(-imb)
                if imb[l] > self.threshold and abs(imb[l] - self.last.get(int(l), 0.0)) > self.fluctuation]
        if self.max_layers is not None:
            todo = todo[:self.max_layers]
        out = placement.copy()
        for l in todo:
            cand = self.inner.rebalance_layer(placement[l], load[l], int(l))
            if imbalance(cand, load[l]) < imb[l]:
                out[l] = cand
            self.last[int(l)] = float(imbalance(out[l], load[l]))
        return out

    def rebalance_layer(self, placement, load, layer=0):
        return self.rebalance(placement[None], load[None])[0]


def make_policy(policy_type: int, **kw) -> EplbPolicy:
    table = {0: RandomPolicy, 1: GreedyPolicy, 2: SwiftPolicy, 3: FlashPolicy}
    if policy_type not in table:
        raise ValueError(f"eplb_policy_type must be one of {sorted(table)}")
    return table[policy_type](**kw)
