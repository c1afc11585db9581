"""KV connector contract shared by every connector.

Scheduler side (runs in the engine loop) and worker side (touches device memory)
are methods of one object here because engine and worker share a process.  The
scheduler-side methods and the ``kv_transfer_params`` fields follow
vllm_ascend/distributed/kv_transfer/kv_p2p/mooncake_connector.py:1843-2001.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

KV_PARAM_FIELDS = ("do_remote_prefill", "do_remote_decode", "remote_block_ids", "remote_engine_id",
                   "remote_host", "remote_port", "remote_request_id", "remote_tp_size",
                   "remote_pcp_size", "remote_dcp_size", "last_token_id", "num_prompt_blocks",
                   "remote_block_size")


@dataclass
class ConnectorMetadata:
    """Per-step message from the scheduler side to the worker side."""
    reqs_to_recv: dict = field(default_factory=dict)     # request_id -> TransferJob
    reqs_to_send: dict = field(default_factory=dict)     # request_id -> block ids kept for a peer
    finished_ids: list = field(default_factory=list)


class KVConnectorBase:
    role = "kv_both"

    # ---- scheduler side
    def get_num_new_matched_tokens(self, req, num_computed_tokens: int) -> tuple[int, bool]:
        """(tokens whose KV an external source will provide, load asynchronously?)"""
        return 0, False

    def update_state_after_alloc(self, req, block_ids: list, num_external_tokens: int) -> None:
        pass

    def build_connector_meta(self, scheduler_output) -> Optional[ConnectorMetadata]:
        return None

    def request_finished(self, req, block_ids: list) -> tuple[bool, Optional[dict]]:
        """(delay freeing the blocks?, kv_transfer_params to hand back to the client)"""
        return False, None

    def is_ready(self, req) -> bool:
        return True

    def take_failed_requests(self) -> list[str]:
        return []

    # ---- worker side
    def register_kv_caches(self, kv_caches: list) -> None:
        pass

    def start_load_kv(self, scheduler_output) -> None:
        pass

    def step_finished(self, scheduler_output, scheduler) -> None:
        pass

    def close(self) -> None:
        pass


def plan_head_slices(tp_src: int, tp_dst: int, num_kv_heads: int, dst_rank: int) -> list[tuple[int, int, int, int]]:
    """Which KV heads a decode rank pulls from which prefill rank when the two sides use
    different TP sizes: list of (src_rank, src_head0, dst_head0, num_heads), heads indexed
    inside each rank's local cache.  KV heads are replicated when a side has more ranks than
    heads.  (The reference derives the same mapping from ``pd_tp_ratio``:
    vllm_ascend/ascend_config.py:205-232 and pulls head slices accordingly,
    mooncake_connector.py:1271-1296.)"""
    def local(tp, rank):
        if num_kv_heads >= tp:
            per = num_kv_heads // tp
            return rank * per, per            # global head start, count
        rep = tp // num_kv_heads
        return rank // rep, 1
    g0, n = local(tp_dst, dst_rank)
    out = []
    h = g0
    while h < g0 + n:
        # first src rank holding global head h
        if num_kv_heads >= tp_src:
            per = num_kv_heads // tp_src
            src_rank = h // per
            s0 = src_rank * per
            cnt = min(g0 + n, s0 + per) - h
            out.append((src_rank, h - s0, h - g0, cnt))
        else:
            rep = tp_src // num_kv_heads
            src_rank = h * rep + (dst_rank % rep)     # spread pulls over the replicas
            cnt = 1
            out.append((src_rank, 0, h - g0, 1))
        h += cnt
    return out
