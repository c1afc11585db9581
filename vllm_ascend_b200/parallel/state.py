"""Process groups: one process per GPU, ``torch.distributed`` (NCCL on GPU,
gloo on CPU) for the plumbing.

Rank layout follows upstream vLLM (``world = DP x PP x TP``, TP fastest) and
adds the groups the reference creates in
vllm_ascend/distributed/parallel_state.py:21-134: an EP group spanning
``DP x TP`` (the reference's ``_MC2`` group has the same ranks), a dedicated
group for dynamic-EPLB weight moves, a prefill head-split group ``_P_TP`` and
the fine-grained TP groups (``o_proj`` / ``lm_head`` / ``embedding`` / ``mlp``)
that are carved out of the DP axis.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..logger import logger


@dataclass
class GroupCoordinator:
    name: str
    ranks: list[int]
    rank_in_group: int
    device_group: Optional[dist.ProcessGroup] = None
    cpu_group: Optional[dist.ProcessGroup] = None

    @property
    def world_size(self) -> int:
        return len(self.ranks)

    @property
    def is_first_rank(self) -> bool:
        return self.rank_in_group == 0

    @property
    def is_last_rank(self) -> bool:
        return self.rank_in_group == self.world_size - 1

    # -- collectives (no-ops for single-rank groups) ------------------
    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world_size > 1:
            dist.all_reduce(t, group=self.device_group)
        return t

    def all_gather(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        if self.world_size == 1:
            return t
        t = t.contiguous()
        if t.dim() == 0:
            t = t.view(1)
        flat = torch.empty((self.world_size * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype,
                           device=t.device)
        dist.all_gather_into_tensor(flat, t, group=self.device_group)
        out = flat.view((self.world_size,) + tuple(t.shape))
        if dim < 0:
            dim += t.dim()
        out = out.movedim(0, dim)
        shape = list(t.shape)
        shape[dim] *= self.world_size
        return out.reshape(shape)

    def reduce_scatter(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        if self.world_size == 1:
            return t
        if dim != 0:
            t = t.movedim(dim, 0)
        t = t.contiguous()
        out = torch.empty((t.shape[0] // self.world_size,) + tuple(t.shape[1:]), dtype=t.dtype,
                          device=t.device)
        dist.reduce_scatter_tensor(out, t, group=self.device_group)
        if dim != 0:
            out = out.movedim(0, dim)
        return out

    def all_to_all_single(self, t: torch.Tensor, out_splits=None, in_splits=None) -> torch.Tensor:
        if self.world_size == 1:
            return t
        t = t.contiguous()
        if out_splits is None:
            out = torch.empty_like(t)
        else:
            out = torch.empty((int(sum(out_splits)),) + tuple(t.shape[1:]), dtype=t.dtype,
                              device=t.device)
        dist.all_to_all_single(out, t, out_splits, in_splits, group=self.device_group)
        return out

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world_size > 1:
            dist.broadcast(t, src=self.ranks[src], group=self.device_group)
        return t

    def broadcast_object(self, obj, src: int = 0):
        if self.world_size == 1:
            return obj
        lst = [obj]
        dist.broadcast_object_list(lst, src=self.ranks[src], group=self.cpu_group)
        return lst[0]

    def all_gather_object(self, obj) -> list:
        if self.world_size == 1:
            return [obj]
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.cpu_group)
        return out

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier(group=self.cpu_group)

    def send(self, t: torch.Tensor, dst: int) -> None:
        dist.send(t, dst=self.ranks[dst], group=self.device_group)

    def recv(self, t: torch.Tensor, src: int) -> None:
        dist.recv(t, src=self.ranks[src], group=self.device_group)


@dataclass
class ParallelState:
    world: Optional[GroupCoordinator] = None
    tp: Optional[GroupCoordinator] = None
    pp: Optional[GroupCoordinator] = None
    dp: Optional[GroupCoordinator] = None
    ep: Optional[GroupCoordinator] = None
    dcp: Optional[GroupCoordinator] = None
    pcp: Optional[GroupCoordinator] = None
    extra: dict = field(default_factory=dict)   # mc2, dynamic_eplb, p_tp, otp, lmtp, embed_tp, mlp_tp


_STATE = ParallelState()
_SINGLE = GroupCoordinator("single", [0], 0)


def single_rank_group() -> GroupCoordinator:
    """A group of this rank alone (modules that hold whole, replicated weights)."""
    return _SINGLE


def _layout(world_size: int, tp: int, pp: int, dp: int, pcp: int = 1) -> torch.Tensor:
    assert world_size == tp * pp * dp * pcp, (world_size, tp, pp, dp, pcp)
    return torch.arange(world_size).reshape(dp, pp, pcp * tp)


def group_rank_lists(world_size: int, tp: int, pp: int = 1, dp: int = 1, pcp: int = 1) -> dict[str, list[list[int]]]:
    """Pure function (unit-testable without torch.distributed).  Rank order, outermost first:
    data, pipeline, prefill-context, tensor.  A prefill-context group joins the ranks that hold the
    same tensor shard of the same replica and stage."""
    lay = _layout(world_size, tp, pp, dp, pcp)
    wide = pcp * tp                                   # ranks of one (replica, stage)
    lay4 = lay.reshape(dp, pp, pcp, tp)
    return {
        "tp": lay.reshape(-1, tp).tolist(),
        "pp": lay.transpose(1, 2).reshape(-1, pp).tolist(),
        "dp": lay.permute(1, 2, 0).reshape(-1, dp).tolist(),
        "pcp": lay4.transpose(2, 3).reshape(-1, pcp).tolist(),
        # experts are sharded over DP x PCP x TP inside one PP stage
        "ep": lay.transpose(0, 1).reshape(pp, dp * wide).tolist(),
    }


def finegrained_rank_lists(world_size: int, tp: int, pp: int, dp: int, size: int) -> list[list[int]]:
    """Fine-grained TP of size ``size`` built across the DP axis
    (vllm_ascend/distributed/parallel_state.py:95-134): when ``size`` is a
    multiple of tp it spans ``size // tp`` consecutive DP replicas."""
    lay = _layout(world_size, tp, pp, dp)
    if size <= tp:
        assert tp % size == 0
        return lay.reshape(-1, size).tolist()
    assert size % tp == 0 and dp % (size // tp) == 0, (size, tp, dp)
    span = size // tp
    out = []
    for p in range(pp):
        for d0 in range(0, dp, span):
            out.append(lay[d0:d0 + span, p, :].reshape(-1).tolist())
    return out


# every multi-rank group this process created, in creation order: what suspend / restore replays
_RECORDS: list = []
_SUSPENDED = False


def _make(name: str, lists: Sequence[Sequence[int]], rank: int, backend: str,
          timeout: Optional[timedelta]) -> GroupCoordinator:
    mine = None
    for ranks in lists:
        ranks = list(ranks)
        if len(ranks) == 1:
            if rank in ranks:
                mine = GroupCoordinator(name, ranks, 0)
            continue
        dg = dist.new_group(ranks, backend=backend, timeout=timeout)
        cg = dist.new_group(ranks, backend="gloo", timeout=timeout) if backend != "gloo" else dg
        if rank in ranks:
            mine = GroupCoordinator(name, ranks, ranks.index(rank), dg, cg)
    assert mine is not None, f"rank {rank} not in any {name} group"
    _RECORDS.append((mine, [list(r) for r in lists], rank, backend, timeout))
    return mine


def has_nccl_groups() -> bool:
    """True when a model-parallel group of more than one rank runs over NCCL."""
    return any(b == "nccl" and any(len(r) > 1 for r in lists) for _, lists, _, b, _ in _RECORDS)


def suspend_groups() -> int:
    """Destroys the device communicators of all model-parallel groups (their buffers are device
    memory a sleeping engine gives back); the coordinators stay and are refilled by
    ``restore_groups``.  Collective: every rank calls it at the same point, with no collective in
    flight.  The host-side (gloo) companions of NCCL groups are kept.  Returns how many
    communicators this rank destroyed.  Same step as the reference's optimised sleep
    (vllm_ascend/device_allocator/sleep_mem_optimized.py:34-186 destroys the process groups before
    the allocator releases memory and re-creates them on wake-up)."""
    global _SUSPENDED
    if _SUSPENDED:
        return 0
    if any(b == "nccl" for _, _, _, b, _ in _RECORDS):
        # NCCL communicators are kept: on two B200s a wake-up after destroying and re-creating them
        # did not return (twice, cause not found); their buffers are small next to weights and KV
        logger.warning("sleep: NCCL communicators are kept (destroy / re-create is limited to host-side groups)")
        return 0
    n = 0
    for mine, _, _, _, _ in _RECORDS:
        dg = mine.device_group
        if dg is None:
            continue
        same = mine.cpu_group is dg
        dist.destroy_process_group(dg)
        mine.device_group = None
        if same:
            mine.cpu_group = None
        n += 1
    _SUSPENDED = True
    return n


def restore_groups() -> int:
    """Re-creates the communicators destroyed by ``suspend_groups`` in their original order and
    puts them back into the same coordinator objects (layers keep their references)."""
    global _SUSPENDED
    if not _SUSPENDED:
        return 0
    n = 0
    for mine, lists, rank, backend, timeout in _RECORDS:
        for ranks in lists:
            if len(ranks) == 1:
                continue
            dg = dist.new_group(ranks, backend=backend, timeout=timeout)
            if rank in ranks:
                mine.device_group = dg
                if mine.cpu_group is None:
                    mine.cpu_group = dg
                n += 1
                if backend == "nccl" and torch.cuda.is_available():
                    # a device communicator is built by its first collective: do that here, outside
                    # any stream capture (graphs are re-captured right after wake-up)
                    t = torch.zeros(1, device=torch.device("cuda", torch.cuda.current_device()))
                    dist.all_reduce(t, group=dg)
    if n and torch.cuda.is_available():
        torch.cuda.synchronize()
    _SUSPENDED = False
    return n


def groups_suspended() -> bool:
    return _SUSPENDED


def init_distributed(backend: Optional[str] = None, timeout_s: Optional[float] = None) -> tuple[int, int, int]:
    """Join the default process group from torchrun-style env vars."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if timeout_s:
            kw["timeout"] = timedelta(seconds=timeout_s)
        if backend == "nccl":
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kw)
    return rank, local, world


def initialize_model_parallel(tp: int = 1, pp: int = 1, dp: int = 1, dcp: int = 1,
                              backend: Optional[str] = None,
                              finegrained: Optional[dict] = None,
                              timeout_s: Optional[float] = None, pcp: int = 1) -> ParallelState:
    global _STATE
    world_size = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    if world_size == 1:
        _STATE = ParallelState(world=_SINGLE, tp=_SINGLE, pp=_SINGLE, dp=_SINGLE, ep=_SINGLE,
                               dcp=_SINGLE, pcp=_SINGLE)
        return _STATE
    if backend is None:
        backend = dist.get_backend()
    timeout = timedelta(seconds=timeout_s) if timeout_s else None
    _RECORDS.clear()
    lists = group_rank_lists(world_size, tp, pp, dp, pcp)
    st = ParallelState()
    st.world = _make("world", [list(range(world_size))], rank, backend, timeout)
    st.tp = _make("tp", lists["tp"], rank, backend, timeout)
    st.pp = _make("pp", lists["pp"], rank, backend, timeout)
    st.dp = _make("dp", lists["dp"], rank, backend, timeout)
    st.ep = _make("ep", lists["ep"], rank, backend, timeout)
    # DCP splits each TP group into tp/dcp groups of dcp consecutive ranks
    if dcp > 1:
        dl = [g[i:i + dcp] for g in lists["tp"] for i in range(0, tp, dcp)]
        st.dcp = _make("dcp", dl, rank, backend, timeout)
    else:
        st.dcp = GroupCoordinator("dcp", [rank], 0)
    st.pcp = _make("pcp", lists["pcp"], rank, backend, timeout) if pcp > 1 else GroupCoordinator("pcp", [rank], 0)
    st.extra["mc2"] = st.ep                      # same ranks as EP, as in the reference
    st.extra["dynamic_eplb"] = _make("dynamic_eplb", lists["ep"], rank, backend, timeout)
    for key, size in (finegrained or {}).items():
        if size and size > 0:
            st.extra[key] = _make(key, finegrained_rank_lists(world_size, tp, pp, dp, size),
                                  rank, backend, timeout)
    _STATE = st
    return st


def destroy_model_parallel() -> None:
    global _STATE, _SUSPENDED
    _STATE = ParallelState()
    _RECORDS.clear()
    _SUSPENDED = False


def get_state() -> ParallelState:
    return _STATE


def _get(name: str) -> GroupCoordinator:
    g = getattr(_STATE, name)
    return g if g is not None else _SINGLE


def get_tp_group() -> GroupCoordinator:
    return _get("tp")


def get_pp_group() -> GroupCoordinator:
    return _get("pp")


def get_dp_group() -> GroupCoordinator:
    return _get("dp")


def get_ep_group() -> GroupCoordinator:
    return _get("ep")


def get_dcp_group() -> GroupCoordinator:
    return _get("dcp")


def get_pcp_group() -> GroupCoordinator:
    return _get("pcp")


def get_world_group() -> GroupCoordinator:
    return _get("world")


def get_extra_group(name: str) -> GroupCoordinator:
    return _STATE.extra.get(name) or _SINGLE


def tp_size() -> int:
    return get_tp_group().world_size


def tp_rank() -> int:
    return get_tp_group().rank_in_group
