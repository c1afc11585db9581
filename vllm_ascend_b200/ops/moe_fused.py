"""Fused expert-parallel MoE path over peer memory (small, decode-sized batches).

Four launches, no NCCL call and no host synchronisation: dispatch (histogram exchange +
direct stores of token rows into the expert owners' packed receive pools), grouped
GEMM1+SwiGLU that starts when the rows have landed, grouped GEMM2 whose epilogue stores
every output row into the token owner's combine buffer, weighted reduce.  Role of the
reference's ``FusedMC2CommImpl`` (vllm_ascend/ops/fused_moe/moe_comm_method.py:283-447) and
its symmetric-buffer sizing from rank-invariant configuration (:283-336).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_long, c_void_p

import torch

from .. import _native
from ..parallel.symm_mem import SymmetricMemory

P, I, L = c_void_p, c_int, c_long
_native.register_signature("b200_moe_ctl_bytes", [])
_native.register_signature("b200_moe_dispatch", [P, L, P, I, I, I, I, I, I, I, P, P, P, P, P, P, L, P, P])
_native.register_signature("b200_moe_reduce", [P, P, P, P, L, I, I, I, I, P, P, P])
_native.register_signature("b200_moe_gemm1_bf16", [P, P, P, P, I, L, I, I, P, I, P, P])
_native.register_signature("b200_moe_gemm2_scatter_bf16", [P, P, P, P, I, L, I, I, P, P, I, I, P, P])


class FusedMoEComm:
    def __init__(self, engine_cfg, device: torch.device, ep_group, capacity: int = 0):
        from ..platform_config import get_b200_config
        m = engine_cfg.model
        self.device = device
        self.ep = ep_group
        self.world, self.rank = ep_group.world_size, ep_group.rank_in_group
        self.capacity = capacity or get_b200_config().fused_moe_max_tokens
        self.H, self.I = m.hidden_size, m.moe_intermediate_size
        # physical expert slots: logical experts plus the redundant replicas of EPLB
        self.E = m.num_experts + get_b200_config().eplb_config.num_redundant_experts
        self.topk = m.num_experts_per_tok
        if self.E % self.world:
            raise ImportError("fused MoE path needs num_experts divisible by the EP size")
        if self.I % 128 or self.H % 8 or self.E > 512:
            raise ImportError("fused MoE path: unsupported expert geometry")
        self.E_local = self.E // self.world
        # worst case: every rank routes all of its capacity*topk pairs to this rank
        self.pool_rows = self.world * self.capacity * self.topk
        lib = _native.lib()
        ctl_bytes = (lib.b200_moe_ctl_bytes() + 255) // 256 * 256
        sizes = {"ctl": ctl_bytes, "hist": self.world * self.E * 4,
                 "recv_x": self.pool_rows * self.H * 2, "recv_meta": self.pool_rows * 4,
                 "comb": self.capacity * self.topk * self.H * 2}
        self.symm = SymmetricMemory(ep_group, device, sum((v + 1023) // 1024 * 1024 for v in sizes.values()))
        self.off = {k: self.symm.region(v) for k, v in sizes.items()}
        self.symm.local.zero_()          # control block, histogram and pools start from zero
        torch.cuda.synchronize(device)
        ep_group.barrier()
        self.ptrs = {k: self.symm.ptr_array(o) for k, o in self.off.items()}
        self.recv_x = self.symm.tensor(self.off["recv_x"], (self.pool_rows, self.H), torch.bfloat16)
        self.recv_meta = self.symm.tensor(self.off["recv_meta"], (self.pool_rows,), torch.int32)
        self.comb = self.symm.tensor(self.off["comb"], (self.capacity * self.topk, self.H), torch.bfloat16)
        self.ctl_ptr = self.symm.local_ptr + self.off["ctl"]
        # local scratch
        self.act = torch.zeros((self.pool_rows, self.I), dtype=torch.bfloat16, device=device)
        self.cursor = torch.zeros(self.E, dtype=torch.int32, device=device)
        self.group_offsets = torch.zeros(self.E_local + 1, dtype=torch.int32, device=device)
        self.calls = 0

    def forward(self, block, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        T, H = x.shape
        if T > self.capacity:
            raise ValueError(f"fused MoE path got {T} tokens, capacity {self.capacity}")
        if block.quant is not None:
            raise NotImplementedError("fused MoE path runs bf16 experts")
        lib = _native.lib()
        st = _native.status_word(self.device).data_ptr()
        stream = _native.stream_ptr()
        x = x if x.stride(1) == 1 else x.contiguous()
        ids = topk_ids.to(torch.int32).contiguous()
        w = topk_w.to(torch.float32).contiguous()
        out = torch.empty((T, H), dtype=torch.bfloat16, device=x.device)
        _native.check(lib.b200_moe_dispatch(
            x.data_ptr(), x.stride(0), ids.data_ptr(), T, self.topk, H, self.E, self.E_local, self.rank,
            self.world, self.ptrs["hist"], self.ptrs["recv_x"], self.ptrs["recv_meta"], self.ptrs["ctl"],
            self.cursor.data_ptr(), self.group_offsets.data_ptr(), self.pool_rows, st, stream), "moe_dispatch")
        _native.check(lib.b200_moe_gemm1_bf16(
            self.recv_x.data_ptr(), block.w13.data_ptr(), self.act.data_ptr(), self.group_offsets.data_ptr(),
            self.E_local, self.pool_rows, self.I, H, self.ctl_ptr, self.world, st, stream), "moe_gemm1")
        _native.check(lib.b200_moe_gemm2_scatter_bf16(
            self.act.data_ptr(), block.w2.data_ptr(), self.group_offsets.data_ptr(), self.recv_meta.data_ptr(),
            self.E_local, self.pool_rows, H, self.I, self.ptrs["comb"], self.ptrs["ctl"], self.rank,
            self.world, st, stream), "moe_gemm2_scatter")
        _native.check(lib.b200_moe_reduce(
            self.comb.data_ptr(), w.data_ptr(), ids.data_ptr(), out.data_ptr(), out.stride(0), T, self.topk, H,
            self.world, self.ctl_ptr, st, stream), "moe_reduce")
        _native.count_launch(4)
        self.calls += 1
        return out

    def close(self) -> None:
        self.symm.close()
