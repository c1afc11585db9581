"""Expert-parallel token exchange around the grouped expert GEMMs.

Three methods, selected per step from the largest token count over the DP ranks
so every rank picks the same one (rule of
vllm_ascend/ascend_forward_context.py:223-343):

  ALLGATHER  all-gather tokens + routing over the EP group, run the local experts
             on everything, reduce-scatter the result
             (vllm_ascend/ops/fused_moe/token_dispatcher.py:367-461)
  ALLTOALL   permute by destination rank, all-to-all-v with split sizes from the
             routing histogram, local experts, reverse all-to-all, weighted
             un-permute (token_dispatcher.py:464-744)
  FUSED      device-initiated dispatch + grouped GEMM + combine over peer memory
             for small (decode) batches — the reference's MC2 / dispatch_ffn_combine
             (ops/fused_moe/moe_comm_method.py:283-447); overflow beyond the
             configured capacity falls back to ALLTOALL for that step
"""
from __future__ import annotations

import enum
from typing import Optional

import torch

from .. import envs
from ..parallel import state as pstate
from ..platform_config import get_b200_config
from . import fused_moe


class MoECommType(enum.Enum):
    ALLGATHER = 0
    FUSED = 1       # reference: MC2 / FUSED_MC2
    ALLTOALL = 2


def select_moe_comm_method(max_tokens_across_dp: int, ep_size: int, fused_available: bool,
                           capacity: int, is_cuda: bool, override: str = "") -> MoECommType:
    if override:
        return {"allgather": MoECommType.ALLGATHER, "alltoall": MoECommType.ALLTOALL,
                "fused": MoECommType.FUSED}[override]
    if ep_size <= 1:
        return MoECommType.ALLGATHER
    if fused_available and is_cuda and max_tokens_across_dp <= capacity:
        return MoECommType.FUSED
    return MoECommType.ALLTOALL


class MoERuntime:
    def __init__(self, engine_cfg, device: torch.device):
        self.cfg = engine_cfg
        self.device = device
        self.ep = pstate.get_ep_group()
        self.b200 = get_b200_config()
        self.capacity = self.b200.fused_moe_max_tokens
        if self.b200.enable_prefill_fused_moe:
            # prefill-sized steps stay on the fused path too when its pools fit comfortably
            # (the reference caps its device-initiated path at 512 tokens per rank; with 180 GB
            # per GPU the packed pools of a full step are affordable here)
            m = engine_cfg.model
            want = engine_cfg.scheduler.max_num_batched_tokens + engine_cfg.scheduler.max_num_seqs
            rows = self.ep.world_size * want * m.num_experts_per_tok
            pool_bytes = rows * (m.hidden_size + m.moe_intermediate_size) * 2 + \
                want * m.num_experts_per_tok * m.hidden_size * 2
            if pool_bytes <= int(self.b200.fused_moe_pool_limit_gb * (1 << 30)):
                self.capacity = max(self.capacity, want)
        self.max_tokens_across_dp = 0          # set per step by the engine's DP sync
        self.fused = None
        if device.type == "cuda" and self.b200.enable_fused_moe_comm and self.ep.world_size > 1:
            try:
                from .moe_fused import FusedMoEComm
                self.fused = FusedMoEComm(engine_cfg, device, self.ep, capacity=self.capacity)
            except ImportError:
                self.fused = None
        self.last_method: Optional[MoECommType] = None
        self.counts = {t: 0 for t in MoECommType}

    def select(self, num_tokens: int, is_cuda: bool = True) -> MoECommType:
        """The method every EP rank uses this step (same inputs on every rank: the largest token
        count over the DP ranks, agreed by the engine before the forward pass)."""
        n_max = max(self.max_tokens_across_dp, num_tokens)
        return select_moe_comm_method(n_max, self.ep.world_size, self.fused is not None,
                                      self.capacity, is_cuda, envs.VLLM_B200_MOE_COMM)

    def graph_safe(self, num_tokens: int) -> bool:
        """Only the fused path has no host synchronisation and can live in a captured graph."""
        return self.select(num_tokens) == MoECommType.FUSED

    def forward(self, block, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        n_max = max(self.max_tokens_across_dp, x.shape[0])
        method = self.select(x.shape[0], x.is_cuda)
        if x.is_cuda and method != MoECommType.FUSED and torch.cuda.is_current_stream_capturing():
            raise RuntimeError(f"MoE path {method.name} cannot be captured into a CUDA graph "
                               f"({x.shape[0]} tokens, fused capacity {self.capacity})")
        lora = getattr(block, "lora", None)
        if lora is not None and lora.punica.any_active and block.quant is None:
            # adapter steps: the slot of every token travels with it, which the fused kernel's
            # packed pools do not carry
            if method == MoECommType.FUSED:
                method = MoECommType.ALLGATHER
            self.last_method = method
            self.counts[method] += 1
            slots = lora.punica.token_slots[:x.shape[0]]
            if method == MoECommType.ALLGATHER:
                return self._allgather(block, x, topk_w, topk_ids, n_max, lora, slots)
            return self._alltoall(block, x, topk_w, topk_ids, lora, slots)
        self.last_method = method
        self.counts[method] += 1
        if method == MoECommType.FUSED and self.fused is not None:
            return self.fused.forward(block, x, topk_w, topk_ids)
        if method == MoECommType.ALLGATHER:
            return self._allgather(block, x, topk_w, topk_ids, n_max)
        return self._alltoall(block, x, topk_w, topk_ids)

    # ------------------------------------------------------------------ all-gather path
    def _allgather(self, block, x, topk_w, topk_ids, n_max: int, lora=None, slots=None) -> torch.Tensor:
        ep = self.ep
        T, H = x.shape
        pad = n_max - T
        if lora is not None:
            slots = torch.cat([slots, slots.new_full((pad,), -1)]) if pad else slots
        if pad:
            x = torch.cat([x, x.new_zeros(pad, H)])
            topk_w = torch.cat([topk_w, topk_w.new_zeros(pad, topk_w.shape[1])])
            # padded rows route to expert 0 with weight 0
            topk_ids = torch.cat([topk_ids, topk_ids.new_zeros(pad, topk_ids.shape[1])])
        xg = ep.all_gather(x, 0)
        wg = ep.all_gather(topk_w, 0)
        ig = ep.all_gather(topk_ids, 0)
        if lora is not None:
            from ..lora.moe import fused_experts_lora
            y = fused_experts_lora(xg, block.w13, block.w2, wg, ig, block.expert_map, lora,
                                   slots=ep.all_gather(slots.contiguous(), 0))
        else:
            y = fused_moe.fused_experts(xg, block.w13, block.w2, wg, ig, block.expert_map, block.quant)
        if x.is_cuda:
            y = ep.reduce_scatter(y, 0)
        else:   # gloo has no reduce-scatter
            y = ep.all_reduce(y)[ep.rank_in_group * n_max:(ep.rank_in_group + 1) * n_max]
        return y[:T]

    # ------------------------------------------------------------------ all-to-all-v path
    def _alltoall(self, block, x, topk_w, topk_ids, lora=None, slots=None) -> torch.Tensor:
        ep = self.ep
        n, E_local = ep.world_size, block.E_local
        T, H = x.shape
        k = topk_ids.shape[1]
        flat_ids = topk_ids.reshape(-1).long()                      # [T*k]
        dest = flat_ids // E_local                                  # owning rank
        order = torch.argsort(dest, stable=True)
        send_tok = order // k
        send_x = x[send_tok]
        send_e = flat_ids[order]
        send_counts = torch.bincount(dest, minlength=n)
        # every rank learns how much it will receive from everybody
        all_counts = ep.all_gather(send_counts.view(1, n), 0)      # [n(src), n(dst)]
        recv_counts = all_counts[:, ep.rank_in_group]
        in_splits = send_counts.tolist()
        out_splits = recv_counts.tolist()
        recv_x = ep.all_to_all_single(send_x, out_splits, in_splits)
        recv_e = ep.all_to_all_single(send_e, out_splits, in_splits)
        # local experts on the received rows (each row is one (token, expert) pair, weight 1)
        R = recv_x.shape[0]
        recv_s = ep.all_to_all_single(slots[send_tok].contiguous(), out_splits, in_splits) if lora is not None else None
        if R > 0 and lora is not None:
            from ..lora.moe import fused_experts_lora
            ones = torch.ones(R, 1, dtype=topk_w.dtype, device=x.device)
            y = fused_experts_lora(recv_x, block.w13, block.w2, ones, recv_e.view(R, 1).to(torch.int32),
                                   block.expert_map, lora, slots=recv_s)
        elif R > 0:
            ones = torch.ones(R, 1, dtype=topk_w.dtype, device=x.device)
            y = fused_moe.fused_experts(recv_x, block.w13, block.w2, ones,
                                        recv_e.view(R, 1).to(torch.int32), block.expert_map,
                                        block.quant)
        else:
            y = recv_x
        back = ep.all_to_all_single(y, in_splits, out_splits)       # rows return in send order
        out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
        w_sorted = topk_w.reshape(-1)[order].float()
        out.index_add_(0, send_tok, back.float() * w_sorted.unsqueeze(-1))
        return out.to(x.dtype)
