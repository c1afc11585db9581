"""P→D connector for hybrid models (attention layers + recurrent linear-attention layers).

Attention layers hand over paged KV blocks exactly like ``NVLinkConnector``.  Recurrent layers
have no per-token cache: what the decode engine needs is the layer's state after the whole prompt
(the short-convolution window and the fp32 delta-rule matrix of the sequence).  A state cannot be
rolled back by one token, so the decode engine does not recompute the last prompt token: it takes
the KV of all prompt tokens, the states, and the first output token the prefill engine sampled,
and continues with a plain decode step.

The prefill engine keeps the finished request's batch row (where its states live) until every
decode rank has pulled; the states are pulled with the block-copy kernel, one "block" per state
tensor row, from the same exported arena as the KV (same process: direct; same node: CUDA IPC
over NVLink; otherwise the TCP side channel).  Prefill and decode engines must use the same TP
size (states are sharded by value head).

Role of the reference's hybrid connector (vllm_ascend/distributed/kv_transfer/kv_p2p/
mooncake_hybrid_connector.py: attention + mamba cache groups in one transfer).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ... import _native
from ...logger import logger
from .nvlink_connector import _LOCAL_ENGINES, NVLinkConnector, TransferJob, _nullctx
from .side_channel import SideChannelError
from .side_channel import request as sc_request


class HybridConnector(NVLinkConnector):
    holds_state_rows = True

    def __init__(self, engine_cfg, runner):
        self.state_tensors: list[torch.Tensor] = []
        self._held_rows: dict[str, int] = {}
        super().__init__(engine_cfg, runner)
        self.stats.update({"pulled_states": 0, "state_bytes": 0})

    # ------------------------------------------------------------------ caches
    def register_kv_caches(self, kv_caches: list) -> None:
        layers = self.runner.model.layers
        attn = [pair for layer, pair in zip(layers, kv_caches)
                if not getattr(layer.self_attn, "is_linear_attention", False)]
        self.state_tensors = [t for layer, pair in zip(layers, kv_caches)
                              if getattr(layer.self_attn, "is_linear_attention", False) for t in pair]
        super().register_kv_caches(attn)
        self._state_ptrs = None
        if self.is_cuda and self.state_tensors:
            dev = self.state_tensors[0].device
            # one launch per distinct row size (conv windows, delta-rule matrices)
            by_size: dict[int, list[int]] = {}
            for i, t in enumerate(self.state_tensors):
                by_size.setdefault(t[0].numel() * t.element_size(), []).append(i)
            self._state_groups = [(nbytes, idx, torch.tensor([self.state_tensors[i].data_ptr() for i in idx],
                                                             dtype=torch.int64, device=dev))
                                  for nbytes, idx in by_size.items()]

    def _meta(self) -> dict:
        m = super()._meta()
        m["state_tensors"] = [{"rows": int(t.shape[0]), "row_bytes": t[0].numel() * t.element_size(),
                               "offset": (t.data_ptr() - self.arena.ptr) if self.arena else -1}
                              for t in self.state_tensors]
        return m

    # ------------------------------------------------------------------ scheduler side
    def get_num_new_matched_tokens(self, req, num_computed_tokens: int) -> tuple[int, bool]:
        p = req.kv_transfer_params
        if not p or not p.get("do_remote_prefill") or self.role == "kv_producer":
            return 0, False
        if p.get("last_token_id") is None or p.get("remote_state_row") is None or not p.get("remote_block_ids"):
            return 0, False
        if num_computed_tokens:
            return 0, False              # a recurrent state cannot be combined with a cached prefix
        return req.num_prompt_tokens, True

    def update_state_after_alloc(self, req, block_ids: list, num_external_tokens: int) -> None:
        p = req.kv_transfer_params
        if num_external_tokens <= 0 or not p or not p.get("do_remote_prefill"):
            return
        p["do_remote_prefill"] = False
        nblk = (req.num_prompt_tokens + self.block_size - 1) // self.block_size
        remote = list(p["remote_block_ids"])
        job = TransferJob(req.request_id, list(block_ids[:nblk]), remote[:nblk], dict(p))
        job.local_row, job.remote_row = int(req.row), int(p["remote_state_row"])
        if int(p.get("remote_block_size", self.block_size)) != self.block_size:
            job.state, job.error = "failed", "prefill and decode engines use different block sizes"
        elif len(job.remote_blocks) != len(job.local_blocks):
            job.state, job.error = "failed", "remote block list does not cover the prompt"
        elif int(p.get("remote_tp_size", 1)) != self.tp_size:
            job.state, job.error = "failed", "hybrid models need equal TP sizes on both engines"
        # the prefill engine's sampled token becomes this request's first output token
        req.output_token_ids = [int(p["last_token_id"])]
        req.num_output_tokens = 1
        self._pending.append(job)
        self._inflight[req.request_id] = job

    def request_finished(self, req, block_ids: list) -> tuple[bool, Optional[dict]]:
        row = req.row
        delay, out = super().request_finished(req, block_ids)
        if delay and out is not None:
            out["remote_state_row"] = int(row)
            self._held_rows[req.request_id] = int(row)
        return delay, out

    def step_finished(self, scheduler_output, scheduler) -> None:
        before = set(self._delayed)
        super().step_finished(scheduler_output, scheduler)
        for rid in before - set(self._delayed):          # released or expired: the row is free again
            row = self._held_rows.pop(rid, None)
            if row is not None:
                scheduler.release_row_id(row)

    # ------------------------------------------------------------------ worker side
    def _handle(self, msg: dict):
        if msg.get("op") == "read_state" and not self.drop_all_messages:
            rid = msg["request_id"]
            if rid not in self._delayed:
                return {"ok": False, "error": f"request {rid} is not held here (expired or unknown)"}
            row = int(msg["row"])
            if self.is_cuda:
                torch.cuda.current_stream(self.state_tensors[0].device).synchronize()
            return {"ok": True, "data": [t[row].contiguous().view(torch.uint8).reshape(-1).cpu().numpy().tobytes()
                                         for t in self.state_tensors]}
        return super()._handle(msg)

    def _launch(self, job: TransferJob) -> None:
        super()._launch(job)
        if not self.state_tensors:
            return
        p = job.params
        key = (str(p.get("remote_engine_id")), self.tp_rank)
        host, port = p.get("remote_host", "127.0.0.1"), int(p.get("remote_port", 0)) + self.tp_rank
        mode, local = self._resolve_mode(key, host, port)
        if mode == "local":
            if len(local.state_tensors) != len(self.state_tensors):
                raise SideChannelError("prefill and decode engines hold different numbers of state tensors")
            self._copy_states(job, [g[2] for g in local._state_groups], int(local.state_tensors[0].shape[0]))
        elif mode == "ipc":
            meta = self._get_meta(key, host, port)
            self._copy_states(job, self._ipc_state_ptrs(key, meta), int(meta["state_tensors"][0]["rows"]))
        else:
            job.futures.append(self._pool.submit(self._pull_states_tcp, job, host, port))

    def _ipc_state_ptrs(self, key, meta) -> list:
        cached = meta.get("_state_ptrs")
        if cached is not None:
            return cached
        self._ipc_sources(key, meta)                     # opens the arena, sets meta["_base"]
        st = meta.get("state_tensors") or []
        if len(st) != len(self.state_tensors) or any(s["offset"] < 0 for s in st):
            raise SideChannelError("remote engine does not export its state tensors")
        dev = self.state_tensors[0].device
        out = []
        for nbytes, idx, _ in self._state_groups:
            if any(st[i]["row_bytes"] != nbytes for i in idx):
                raise SideChannelError("remote state tensors differ in geometry")
            out.append(torch.tensor([meta["_base"] + st[i]["offset"] for i in idx], dtype=torch.int64, device=dev))
        meta["_state_ptrs"] = out
        return out

    def _copy_states(self, job: TransferJob, src_ptr_groups: list, src_rows: int) -> None:
        dev = self.state_tensors[0].device
        lib = _native.lib()
        with torch.cuda.device(dev), torch.cuda.stream(self.stream):
            sb = torch.tensor([job.remote_row], dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            db = torch.tensor([job.local_row], dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            status = _native.status_word(dev)
            for (nbytes, idx, dst_ptrs), src_ptrs in zip(self._state_groups, src_ptr_groups):
                rc = lib.b200_kv_block_copy(
                    src_ptrs.data_ptr(), dst_ptrs.data_ptr(), sb.data_ptr(), db.data_ptr(), 1, len(idx),
                    1, nbytes, 1, 0, 0, nbytes, nbytes, nbytes, nbytes, nbytes, nbytes,
                    src_rows, int(self.state_tensors[0].shape[0]), status.data_ptr(), self.stream.cuda_stream)
                _native.check(rc, "state row copy")
                self.stats["state_bytes"] += nbytes * len(idx)
            ev = torch.cuda.Event()
            ev.record(self.stream)
            job.events.append(ev)
            job._keep_state = (sb, db)
        self.stats["pulled_states"] += 1

    def _pull_states_tcp(self, job: TransferJob, host, port) -> None:
        reply = sc_request(host, port, {"op": "read_state", "request_id": job.params.get("remote_request_id"),
                                        "row": job.remote_row}, self.timeout_ms)
        data = reply["data"]
        if len(data) != len(self.state_tensors):
            raise SideChannelError("state payload does not match the local caches")
        ctx = torch.cuda.stream(self.stream) if self.is_cuda else _nullctx()
        if self.is_cuda:
            torch.cuda.set_device(self.state_tensors[0].device)
        with ctx:
            for t, raw in zip(self.state_tensors, data):
                src = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(t.dtype).view(t[0].shape)
                t[job.local_row].copy_(src.to(t.device))
                self.stats["state_bytes"] += len(raw)
            if self.is_cuda:
                self.stream.synchronize()
        self.stats["pulled_states"] += 1
