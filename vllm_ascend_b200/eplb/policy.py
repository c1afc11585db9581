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
  3  flash           statistical: sliding-window mean / variance of the expert loads, replicas by
                     risk-adjusted load per replica, longest-first packing, renaming that minimises
                     weight movement, per-layer gating by predicted imbalance (policy_flashlb.py)
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


def replica_counts(mu: np.ndarray, var: np.ndarray, slots: int, max_per_expert: int, z: float) -> np.ndarray:
    """Replicas per expert: every expert gets one, each spare slot goes to the expert whose
    risk-adjusted load per replica ``(mu + z * sigma / sqrt(r)) / r`` is largest (a replica takes
    1/r of the mean; tokens spread over replicas independently, so the spread of one replica's
    share falls faster than the mean)."""
    E = mu.shape[0]
    r = np.ones(E, dtype=np.int64)
    sd = np.sqrt(np.maximum(var, 0.0))
    for _ in range(max(0, slots - E)):
        unit = (mu + z * sd / np.sqrt(r)) / r
        unit[r >= max_per_expert] = -np.inf
        e = int(unit.argmax())
        if not np.isfinite(unit[e]):
            break
        r[e] += 1
    return r


def lpt_deploy(unit: np.ndarray, replicas: np.ndarray, R: int, S: int) -> list[list[int]]:
    """Longest-processing-time-first: replicas in descending unit load go to the least loaded
    rank that has a free slot and no copy of the expert."""
    items = sorted(((unit[e], e) for e in range(unit.shape[0]) for _ in range(int(replicas[e]))),
                   key=lambda x: (-x[0], x[1]))
    load = np.zeros(R)
    rows: list[list[int]] = [[] for _ in range(R)]
    for w, e in items:
        order = np.argsort(load, kind="stable")
        pick = next((r for r in order if len(rows[r]) < S and e not in rows[r]), None)
        if pick is None:
            pick = next(r for r in order if len(rows[r]) < S)
        rows[pick].append(e)
        load[pick] += w
    return rows


def minimize_redeploy(old: np.ndarray, rows: list[list[int]]) -> np.ndarray:
    """Name the new rank-sets and order their slots so that as few expert weights as possible
    move: ranks are matched to the new sets by maximum overlap (assignment problem), and inside a
    rank an expert that stays keeps its slot (the reference solves the same matching before it
    transfers weights, policy_flashlb.py:761-845)."""
    R, S = old.shape
    overlap = np.zeros((R, R), dtype=np.int64)
    old_sets = [set(int(x) for x in old[r]) for r in range(R)]
    for i in range(R):
        for j in range(R):
            overlap[i, j] = len(old_sets[i] & set(rows[j]))
    try:
        from scipy.optimize import linear_sum_assignment
        ri, cj = linear_sum_assignment(-overlap)
        match = dict(zip(ri.tolist(), cj.tolist()))
    except Exception:                                    # greedy matching without scipy
        match, used = {}, set()
        for i in np.argsort(-overlap.max(axis=1)):
            j = next(j for j in np.argsort(-overlap[i]) if j not in used)
            match[int(i)] = int(j)
            used.add(int(j))
    out = np.full((R, S), -1, dtype=old.dtype)
    for i in range(R):
        want = list(rows[match[i]])
        for s_ in range(S):                              # experts that stay keep their slot
            e = int(old[i, s_])
            if e in want:
                out[i, s_] = e
                want.remove(e)
        for s_ in range(S):
            if out[i, s_] < 0:
                out[i, s_] = want.pop(0)
    return out


class FlashPolicy(EplbPolicy):
    """Statistical re-planning, gated per layer.

    Loads fluctuate from step to step, so a plan made for the last sample chases noise.  This
    policy keeps a sliding window of load samples per layer and plans for the risk-adjusted load
    ``mu + z * sigma`` of every expert: replicas go to the experts with the largest risk-adjusted
    load per replica, replicas are packed longest-first onto the least loaded rank, and the result
    is renamed to overlap the current placement as far as possible so that few weights move.  A
    layer is re-planned only when its predicted imbalance exceeds ``threshold`` and the new plan
    improves it by more than ``fluctuation``; at most ``max_layers_per_call`` layers change per
    call (weight movement is paid for in serving time).

    Approach of the reference's FlashLB (policy_flashlb.py:515-965: windowed hotness statistics,
    z-score replica allocation, LPT deployment, redeploy minimisation, update gating)."""

    def __init__(self, threshold: float = 1.15, fluctuation: float = 0.05, max_layers_per_call: Optional[int] = None,
                 window: int = 8, z_score: float = 0.674):
        self.threshold, self.fluctuation = threshold, fluctuation
        self.max_layers = max_layers_per_call
        self.window, self.z = max(1, int(window)), float(z_score)
        self.samples: dict[int, list] = {}
        self.last: dict[int, float] = {}
        self.moved_slots = 0

    # ---- statistics
    def register_hotness(self, layer: int, load: np.ndarray) -> None:
        buf = self.samples.setdefault(int(layer), [])
        buf.append(np.asarray(load, dtype=np.float64))
        if len(buf) > self.window:
            del buf[0]

    def statistics(self, layer: int, load: np.ndarray):
        """(mean, variance) per expert over the window (the current sample alone when the window is empty)."""
        buf = self.samples.get(int(layer))
        if not buf:
            x = np.asarray(load, dtype=np.float64)
            return x, np.zeros_like(x)
        X = np.stack(buf)
        return X.mean(axis=0), X.var(axis=0)

    def risk_load(self, layer: int, load: np.ndarray) -> np.ndarray:
        mu, var = self.statistics(layer, load)
        return mu + self.z * np.sqrt(var)

    # ---- planning
    def plan_layer(self, placement: np.ndarray, load: np.ndarray, layer: int = 0) -> np.ndarray:
        R, S = placement.shape
        mu, var = self.statistics(layer, load)
        if R * S < mu.shape[0]:
            raise ValueError("fewer expert slots than experts")
        r = replica_counts(mu, var, R * S, R, self.z)
        unit = (mu + self.z * np.sqrt(var) / np.sqrt(r)) / r
        return minimize_redeploy(placement, lpt_deploy(unit, r, R, S))

    def rebalance(self, placement, load):
        L = placement.shape[0]
        for l in range(L):
            self.register_hotness(l, load[l])
        risk = [self.risk_load(l, load[l]) for l in range(L)]
        imb = np.array([imbalance(placement[l], risk[l]) for l in range(L)])
        todo = [int(l) for l in np.argsort(-imb) if imb[l] > self.threshold]
        out = placement.copy()
        changed = 0
        for l in todo:
            if self.max_layers is not None and changed >= self.max_layers:
                break
            cand = self.plan_layer(placement[l], load[l], l)
            new_imb = imbalance(cand, risk[l])
            if imb[l] - new_imb > self.fluctuation:
                out[l] = cand
                self.moved_slots += int((cand != placement[l]).sum())
                changed += 1
            self.last[l] = float(imbalance(out[l], risk[l]))
        return out

    def rebalance_layer(self, placement, load, layer=0):
        self.register_hotness(layer, load)
        return self.plan_layer(placement, load, layer)


def make_policy(policy_type: int, **kw) -> EplbPolicy:
    table = {0: RandomPolicy, 1: GreedyPolicy, 2: SwiftPolicy, 3: FlashPolicy}
    if policy_type not in table:
        raise ValueError(f"eplb_policy_type must be one of {sorted(table)}")
    return table[policy_type](**kw)
