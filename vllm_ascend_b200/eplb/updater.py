"""Dynamic EPLB: collect expert loads, plan a new placement off the critical path, move
expert weights one layer per engine step, swap the routing tables.

State machine of vllm_ascend/eplb/eplb_updator.py:79-155: COLLECT for
``expert_heat_collection_interval`` steps → all-reduce of the per-layer loads → planner
runs in the background → ``algorithm_execution_interval`` steps later the plan is fetched
→ MOVE: one MoE layer per step, peer-to-peer send/recv of the experts that change rank
into a staging copy, then the slot weights and the ``log2phy`` / ``expert_map`` tables are
swapped between two steps (eplb/core/eplb_device_transfer_loader.py:46-138).  Every rank
plans from the same all-reduced loads with a deterministic policy, so no plan broadcast is
needed.
"""
from __future__ import annotations

from concurrent.futures import Future, ThreadPoolExecutor
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..logger import logger
from . import expert_map as em
from .policy import imbalance, make_policy


class EplbAdaptor:
    """Everything the updater needs from the model: the MoE blocks, their slot weights and
    routing tables (role of eplb/adaptor/vllm_adaptor.py:69-222)."""

    def __init__(self, model, ep_group, num_redundant: int = 0):
        self.blocks = [L.mlp for L in model.layers if hasattr(L.mlp, "gate_weight")]
        if not self.blocks:
            raise ValueError("EPLB needs a model with routed experts")
        self.ep = ep_group
        self.R, self.rank = ep_group.world_size, ep_group.rank_in_group
        self.E = self.blocks[0].cfg.num_experts
        self.L = len(self.blocks)
        base = self.E // self.R
        self.S = base + num_redundant // self.R
        self.device = self.blocks[0].w13.device
        # identity placement first (what the model was built with), padded to S slots by
        # copies of the rank's own experts; the initial redundant layout is then reached by
        # ordinary moves
        ident = em.initial_placement(self.L, self.E, self.R, 0)
        if self.S > base:
            pad = np.stack([np.stack([ident[l, r, np.arange(self.S - base) % base] for r in range(self.R)])
                            for l in range(self.L)])
            self.placement = np.concatenate([ident, pad], axis=2)
            for b in self.blocks:
                idx = torch.arange(self.S, device=self.device) % base
                idx[:base] = torch.arange(base, device=self.device)
                b.w13 = b.w13[idx].contiguous()
                b.w2 = b.w2[idx].contiguous()
        else:
            self.placement = ident
        for l, b in enumerate(self.blocks):
            b.expert_load = torch.zeros(self.E, dtype=torch.int64, device=self.device)
            self._install_tables(l)

    def _install_tables(self, l: int) -> None:
        """Routing tables are updated in place (fixed shapes) so captured graphs keep reading
        the same device buffers."""
        b = self.blocks[l]
        table, counts = em.build_log2phy(self.placement[l], self.E, prefer_rank=self.rank)
        width = min(self.R, 1 + (self.S - self.E // self.R) * self.R)
        full = np.full((self.E, width), -1, dtype=np.int32)
        full[:, :table.shape[1]] = table[:, :width]
        if getattr(b, "log2phy", None) is None or tuple(b.log2phy.shape) != full.shape:
            b.log2phy = torch.from_numpy(full).to(self.device)
            b.log2phy_count = torch.from_numpy(np.minimum(counts, width)).to(self.device).long()
            emap = torch.full((self.R * self.S,), -1, dtype=torch.int32)
            emap[self.rank * self.S:(self.rank + 1) * self.S] = torch.arange(self.S, dtype=torch.int32)
            b.expert_map = emap.to(self.device)
            b.E_local = self.S
            b.expert_start = self.rank * self.S
        else:
            b.log2phy.copy_(torch.from_numpy(full))
            b.log2phy_count.copy_(torch.from_numpy(np.minimum(counts, width)).long())

    def collect_loads(self) -> np.ndarray:
        """[L, E] loads summed over the EP ranks; counters are reset."""
        loads = torch.stack([b.expert_load for b in self.blocks]).to(torch.int64)
        if self.R > 1:
            t = loads.cpu() if loads.device.type == "cpu" else loads
            dist.all_reduce(t, group=self.ep.device_group)
            loads = t
        for b in self.blocks:
            b.expert_load.zero_()
        return loads.cpu().numpy().astype(np.float64)

    def move_layer(self, l: int, new_layer: np.ndarray) -> int:
        """Bring layer ``l`` to ``new_layer`` ([R, S]).  Returns the number of experts that
        crossed ranks."""
        moves = em.plan_moves(self.placement[l], new_layer)
        if not moves:
            return 0
        b = self.blocks[l]
        staged: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
        ops, crossed = [], 0
        for i, m in enumerate(moves):
            if m.src_rank == m.dst_rank:
                if m.dst_rank == self.rank:
                    staged[m.dst_slot] = (b.w13[m.src_slot].clone(), b.w2[m.src_slot].clone())
                continue
            crossed += 1
            if m.src_rank == self.rank:
                for t in (b.w13[m.src_slot], b.w2[m.src_slot]):
                    ops.append(dist.P2POp(dist.isend, t.contiguous(), self.ep.ranks[m.dst_rank],
                                          group=self.ep.device_group))
            elif m.dst_rank == self.rank:
                bufs = (torch.empty_like(b.w13[m.dst_slot]), torch.empty_like(b.w2[m.dst_slot]))
                staged[m.dst_slot] = bufs
                for t in bufs:
                    ops.append(dist.P2POp(dist.irecv, t, self.ep.ranks[m.src_rank], group=self.ep.device_group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        # every send read the old slot contents above; now overwrite
        for slot, (w13, w2) in staged.items():
            b.w13[slot].copy_(w13)
            b.w2[slot].copy_(w2)
        self.placement[l] = new_layer
        self._install_tables(l)
        return crossed


class EplbUpdater:
    COLLECT, PLAN, MOVE = "collect", "plan", "move"

    def __init__(self, adaptor: EplbAdaptor, cfg, initial: Optional[np.ndarray] = None):
        self.a = adaptor
        self.cfg = cfg
        self.policy = make_policy(cfg.eplb_policy_type)
        self.state = self.COLLECT
        self.steps = 0
        self.future: Optional[Future] = None
        self.pending: Optional[np.ndarray] = None
        self.next_layer = 0
        self.pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="eplb-planner")
        self.stats = {"updates": 0, "experts_moved": 0, "imbalance_before": 0.0, "imbalance_after": 0.0}
        target = initial
        if target is None and cfg.expert_map_path:
            target = em.load_placement(cfg.expert_map_path)
        if target is None and adaptor.S > adaptor.E // adaptor.R:
            target = em.initial_placement(adaptor.L, adaptor.E, adaptor.R, (adaptor.S - adaptor.E // adaptor.R) * adaptor.R)
        if target is not None:
            if target.shape != adaptor.placement.shape:
                raise ValueError(f"expert map shape {target.shape} does not match {adaptor.placement.shape}")
            em.validate(target, adaptor.E)
            for l in range(adaptor.L):
                adaptor.move_layer(l, target[l])

    def _plan(self, placement: np.ndarray, loads: np.ndarray) -> np.ndarray:
        new = self.policy.rebalance(placement, loads)
        em.validate(new, self.a.E)
        return new

    def step(self) -> None:
        """Call once per engine step, between two forward passes, on every EP rank."""
        if not self.cfg.dynamic_eplb:
            return
        self.steps += 1
        if self.state == self.COLLECT:
            if self.steps >= self.cfg.expert_heat_collection_interval:
                loads = self.a.collect_loads()
                self.loads = loads
                self.future = self.pool.submit(self._plan, self.a.placement.copy(), loads)
                self.state, self.steps = self.PLAN, 0
        elif self.state == self.PLAN:
            if self.steps >= self.cfg.algorithm_execution_interval:
                self.pending = self.future.result()          # same input, same policy: same plan on every rank
                before = np.mean([imbalance(self.a.placement[l], self.loads[l]) for l in range(self.a.L)])
                after = np.mean([imbalance(self.pending[l], self.loads[l]) for l in range(self.a.L)])
                self.stats["imbalance_before"], self.stats["imbalance_after"] = float(before), float(after)
                self.state, self.next_layer = self.MOVE, 0
        elif self.state == self.MOVE:
            l = self.next_layer
            self.stats["experts_moved"] += self.a.move_layer(l, self.pending[l])
            self.next_layer += 1
            if self.next_layer >= self.a.L:
                self.stats["updates"] += 1
                if self.cfg.expert_map_record_path and self.a.rank == 0:
                    em.save_placement(self.cfg.expert_map_record_path, self.a.placement)
                logger.info("EPLB update %d: imbalance %.3f -> %.3f, %d experts moved so far",
                            self.stats["updates"], self.stats["imbalance_before"],
                            self.stats["imbalance_after"], self.stats["experts_moved"])
                self.state, self.steps, self.pending = self.COLLECT, 0, None
                for b in self.a.blocks:
                    b.expert_load.zero_()

    def close(self) -> None:
        self.pool.shutdown(wait=False)
