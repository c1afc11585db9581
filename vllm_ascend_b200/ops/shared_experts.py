"""Shared experts of a MoE block under tensor parallelism: four activation / weight layouts.

A shared expert is a dense gated MLP every token passes through next to its routed experts.  How
it should run depends on what the surrounding layer hands it:

=========================  ====================  ===================  ==========================================
mode                       activations           weights              communication
=========================  ====================  ===================  ==========================================
``TENSOR_PARALLEL``        full ``[T, H]``       TP shards            partial sums; one all-reduce (shared with
                                                                      the routed experts' sum when they are TP
                                                                      shards too)
``DATA_PARALLEL_ONLY``     full ``[T, H]``       replicated           every rank runs ``T / tp`` of the rows
                                                                      through the whole MLP, all-gather of rows
``SEQUENCE_PARALLEL_ONLY`` rows ``[T / tp, H]``  TP shards            all-gather rows, partial sums,
                                                                      reduce-scatter back to rows
``SEQUENCE_PARALLEL_SEDP`` rows ``[T / tp, H]``  replicated           none
=========================  ====================  ===================  ==========================================

Replicated weights cost memory (the whole shared expert on every rank) and buy full-width GEMMs
and half the bytes on the wire (``DATA_PARALLEL_ONLY``) or no collective at all
(``SEQUENCE_PARALLEL_SEDP``).  The executor also offers the split form the side-stream overlap
uses (``part1``: gate/up projection + activation, ``part2``: down projection) and checks once
after loading that the split form reproduces the integrated one.

The reference's executor has the same four modes and the same split
(vllm_ascend/ops/fused_moe/shared_experts.py:49-349, ``SharedExpertParallelMode``; replicated
weights are its ``enable_shared_expert_dp`` option).
"""
from __future__ import annotations

import enum
from typing import Optional

import torch

from .. import ops


class SharedExpertParallelMode(enum.Enum):
    TENSOR_PARALLEL = "tp"
    DATA_PARALLEL_ONLY = "sedp"
    SEQUENCE_PARALLEL_ONLY = "sp"
    SEQUENCE_PARALLEL_SEDP = "sp+sedp"


def select_mode(weights_replicated: bool, activations_sharded: bool) -> SharedExpertParallelMode:
    if activations_sharded:
        return (SharedExpertParallelMode.SEQUENCE_PARALLEL_SEDP if weights_replicated
                else SharedExpertParallelMode.SEQUENCE_PARALLEL_ONLY)
    return (SharedExpertParallelMode.DATA_PARALLEL_ONLY if weights_replicated
            else SharedExpertParallelMode.TENSOR_PARALLEL)


class SharedExperts:
    """Runs ``mlp`` (a ``SwiGLUMLP`` built with ``reduce_results=False``) in one of the four modes.

    ``comm``: the TP communicator of the surrounding layer (``size``, ``rank``, ``all_reduce``,
    ``all_gather``, ``reduce_scatter``).  ``weights_replicated``: ``mlp`` was built over a
    single-rank communicator and holds the whole weights.  ``gate_weight``: optional ``[1, H]``
    vector of checkpoints that scale the shared expert by ``sigmoid(x . w)``.
    """

    def __init__(self, mlp, comm, weights_replicated: bool, gate_weight: Optional[torch.Tensor] = None):
        self.mlp, self.comm = mlp, comm
        self.weights_replicated = bool(weights_replicated)
        self.gate_weight = gate_weight

    # ------------------------------------------------------------------ split form
    def part1(self, x: torch.Tensor) -> torch.Tensor:
        """Gate/up projection + activation."""
        m = self.mlp
        gu = m.gate_up_proj
        if m.act is not None:
            return ops.activation(gu(x).contiguous(), m.act, gated=True)
        if gu.quant is None and gu.bias is None and not gu.gather_output and not gu._lora_on():
            return ops.linear_swiglu(x, gu.weight)
        return ops.silu_and_mul(gu(x))

    def part2(self, x: torch.Tensor, act: torch.Tensor) -> torch.Tensor:
        """Down projection (+ the sigmoid gate); partial sums when the weights are TP shards."""
        y = self.mlp.down_proj(act)
        return self._gate(x, y)

    def _gate(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        if self.gate_weight is None:
            return y
        return y * torch.sigmoid(torch.nn.functional.linear(x.float(), self.gate_weight.float())).to(y.dtype)

    def local(self, x: torch.Tensor) -> torch.Tensor:
        """The MLP on the given rows with this rank's weights, no communication."""
        return self._gate(x, self.mlp(x))

    def validate_split(self, device, dtype, hidden: int, rows: int = 10) -> None:
        """The split form must reproduce the integrated one (checked once after weight loading)."""
        g = torch.Generator(device="cpu").manual_seed(0)
        x = (torch.rand(rows, hidden, generator=g) * 2 - 1).to(device=device, dtype=dtype)
        a, b = self.local(x), self.part2(x, self.part1(x))
        if not torch.allclose(a.float(), b.float(), rtol=1e-2, atol=1e-2):
            raise ValueError("shared experts: split computation does not match the integrated computation "
                             f"(max abs diff {float((a.float() - b.float()).abs().max())})")

    # ------------------------------------------------------------------ modes
    def mode(self, activations_sharded: bool) -> SharedExpertParallelMode:
        if self.comm.size == 1:
            return SharedExpertParallelMode.SEQUENCE_PARALLEL_SEDP if activations_sharded \
                else SharedExpertParallelMode.DATA_PARALLEL_ONLY
        return select_mode(self.weights_replicated, activations_sharded)

    def forward(self, x: torch.Tensor, activations_sharded: bool = False, reduce: bool = True) -> torch.Tensor:
        """``x``: ``[T, H]`` (full) or this rank's rows ``[T / tp, H]`` (sharded).  Returns the same
        layout.  ``reduce=False`` (``TENSOR_PARALLEL`` only) leaves the partial sum to the caller,
        who adds the routed experts' partial sum and reduces once."""
        mode = self.mode(activations_sharded)
        tp = self.comm.size
        if mode is SharedExpertParallelMode.TENSOR_PARALLEL:
            y = self.local(x)
            return self.comm.all_reduce(y) if (reduce and tp > 1) else y
        if mode is SharedExpertParallelMode.SEQUENCE_PARALLEL_SEDP:
            return self.local(x)
        if mode is SharedExpertParallelMode.DATA_PARALLEL_ONLY:
            if tp == 1:
                return self.local(x)
            T = x.shape[0]
            per = (T + tp - 1) // tp
            lo = min(T, self.comm.rank * per)
            mine = x[lo:min(T, lo + per)]
            y = self.local(mine) if mine.shape[0] else x.new_zeros((0, x.shape[1]))
            if y.shape[0] < per:                       # equal pieces for the gather
                y = torch.cat([y, y.new_zeros((per - y.shape[0], y.shape[1]))])
            return self.comm.all_gather(y.contiguous(), dim=0)[:T]
        # SEQUENCE_PARALLEL_ONLY
        full = self.comm.all_gather(x.contiguous(), dim=0)
        y = self.local(full)
        return self.comm.reduce_scatter(y, dim=0)
